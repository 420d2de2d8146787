"""Test infrastructure: CPU restatements of the reference's quantization arithmetic.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of
``bench.py`` may import this package, and only as the checker or the timed CPU baseline.
Nothing under ``cublade_b200/`` imports it.
"""
