"""Static (weight-side) outlier-column detection and splitting for the LLM.int8 variant of
the W8A16 layer.  Behaviour follows cublade/quantization/outlier_utils.py:12-101: a column
(input feature) is an outlier when any ``abs(weight[:, j])`` exceeds the threshold."""
from __future__ import annotations

from typing import List, Tuple

import torch


def detect_outlier_columns(weight: torch.Tensor, threshold: float = 6.0) -> List[int]:
    """Indices ``j`` with ``max_i |weight[i, j]| > threshold`` for ``weight [out, in]``, ascending."""
    peak_per_col = weight.abs().amax(dim=0)
    return torch.nonzero(peak_per_col > threshold, as_tuple=True)[0].tolist()


def split_weights_by_outliers(weight: torch.Tensor, outlier_cols: List[int]
                              ) -> Tuple[torch.Tensor, torch.Tensor, List[int], List[int]]:
    """Split ``weight [out, in]`` by columns.

    Returns ``(weight_normal [out, in - o], weight_outlier [out, o], normal_cols, outlier_cols)``;
    ``normal_cols`` is every column not listed, ascending; ``outlier_cols`` is returned as given.
    """
    listed = set(outlier_cols)
    normal_cols = [j for j in range(weight.shape[1]) if j not in listed]
    return weight[:, normal_cols], weight[:, outlier_cols], normal_cols, outlier_cols


def separate_outliers(weight: torch.Tensor, threshold: float = 6.0
                      ) -> Tuple[torch.Tensor, torch.Tensor, List[int], List[int]]:
    """``detect_outlier_columns`` followed by ``split_weights_by_outliers``."""
    return split_weights_by_outliers(weight, detect_outlier_columns(weight, threshold))
