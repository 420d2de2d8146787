// The one exchange of the multi-GPU path -- the maximum of the ranks' local amax between the two phases of a
// sharded per-tensor quantization -- as peer-memory stores and loads over NVLink instead of a collective call.
//
// Every rank owns a small slot array in memory that its peers have mapped (the caller obtains the mappings, e.g. from
// torch's symmetric memory).  One warp per rank: lane r writes {call number, bits of the local amax} as ONE 64-bit word
// into slot [parity][my rank] of rank r's array (a single naturally aligned 64-bit store: the flag and the value
// cannot be seen apart, so no fence is needed), then polls slot [parity][r] of its OWN array until it carries this
// call's number, and the warp folds the values.  Slots alternate with the parity of the call number: a rank can be at
// most one call ahead of a peer (its next call's wait needs that peer's store of the next call, which the peer issues
// only after its own wait of this call has ended), so a slot is never overwritten before it has been read.
//
// The wait is bounded (about a second of SM clocks); a rank whose peers do not arrive raises the per-device error
// word, writes NaN as the result and returns -- the context stays usable.  The kernels of different ranks wait for one
// another, so every rank must be a process on a GPU of its own.
#include "launch.h"

namespace cb {

unsigned int* w8a16_tc_error_word();

namespace {

constexpr int kMaxRanks = 16;
constexpr int kStateWords = 2 * kMaxRanks + 1;  // two slot sets + this rank's call counter

struct PeerSlots {
    unsigned long long* p[kMaxRanks];
};

__global__ void __launch_bounds__(32) amax_peer_exchange_kernel(const float* __restrict__ local_amax, PeerSlots peers,
                                                                int rank, int world, float* __restrict__ out_amax,
                                                                unsigned int* __restrict__ error_flag) {
    pdl_wait();  // the local amax comes from the kernel ahead in the stream
    pdl_trigger();
    const int lane = threadIdx.x;
    unsigned long long* mine = peers.p[rank];
    const unsigned long long call = mine[2 * kMaxRanks] + 1ULL;  // written only by this kernel, on this GPU
    const unsigned long long* slot = mine + (call & 1ULL) * kMaxRanks;
    const unsigned int bits = __float_as_uint(fmaxf(*local_amax, 0.0f));  // non-negative: the bit pattern orders like the value
    unsigned int got = 0u;
    int ok = 1;
    if (lane < world) {
        const unsigned long long word = (call << 32) | bits;
        unsigned long long* dst = peers.p[lane] + (call & 1ULL) * kMaxRanks + rank;
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(word) : "memory");
        const long long t0 = clock64();
        for (;;) {
            unsigned long long w;
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(slot + lane) : "memory");
            if ((w >> 32) == (call & 0xffffffffULL)) {
                got = (unsigned int)w;
                break;
            }
            if (clock64() - t0 > 2000000000LL) {
                ok = 0;
                break;
            }
            __nanosleep(64);
        }
    }
    ok = __all_sync(0xffffffffu, ok);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) got = max(got, __shfl_xor_sync(0xffffffffu, got, off));
    if (lane == 0) {
        mine[2 * kMaxRanks] = call;
        *out_amax = ok ? __uint_as_float(got) : __uint_as_float(0x7fc00000u);
        if (!ok) atomicExch(error_flag, 1u);
    }
}

}  // namespace

int peer_exchange_state_words() { return kStateWords; }
int peer_exchange_max_ranks() { return kMaxRanks; }

cudaError_t launch_amax_peer_exchange(const float* local_amax, const void* const* peer_state, int rank, int world,
                                      float* out_amax, cudaStream_t s) {
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return cudaErrorInvalidValue;
    unsigned int* err = w8a16_tc_error_word();
    if (!err) return cudaErrorUnknown;
    PeerSlots peers;
    for (int r = 0; r < kMaxRanks; ++r)
        peers.p[r] = r < world ? static_cast<unsigned long long*>(const_cast<void*>(peer_state[r])) : nullptr;
    for (int r = 0; r < world; ++r)
        if (!peers.p[r] || (reinterpret_cast<uintptr_t>(peers.p[r]) & 7)) return cudaErrorInvalidValue;
    return launch_dependent(amax_peer_exchange_kernel, 1u, 32u, 0, s, local_amax, peers, rank, world, out_amax, err);
}

}  // namespace cb
