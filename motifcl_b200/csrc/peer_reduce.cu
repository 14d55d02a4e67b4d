// One-shot sum of a small fp32 vector over the GPUs of one node, through plain peer loads and stores.
//
// A row-parallel decode GEMV leaves a partial result [M, out] on every rank (16 to 256 KB).  Summing it with a
// library collective costs one collective launch and its hand-shake per layer, several times the 1 to 8 us of the
// GEMV before it.  Here every rank's partial sits in a buffer that all ranks have mapped (symmetric memory: the same
// allocation made on every rank and exchanged once), and one kernel per rank does the rest:
//   1. take the next call number from a counter in this rank's own flag area (so a recorded batch can be replayed:
//      nothing about the hand-shake is baked into the launch) and tell every peer "my partial number `seq` is written"
//      (a release store of seq into the peer's flag word for this rank; the partial was written by an earlier kernel of
//      the same stream);
//   2. wait until every peer has said the same (acquire loads of this rank's own flag words: local polling, with a
//      time limit, after which the context's error word is set and the kernel returns);
//   3. load all partials (peer loads that bypass L1) and add them in rank order, so every rank gets the same bits.
// Two partial buffers alternate (the caller's `parity`): a rank may run ahead into the next GEMV while a peer still
// reads the last partial, and by the time a buffer comes round again every peer has passed the hand-shake after its
// last read.  All ranks must make the same sequence of calls.  One CTA: the vectors are 16 to 256 KB.
// Plain loads and stores only; no load from a peer before its flag says the data is there; no wait without a limit.
#include "kernels.h"

namespace mcl {
namespace {

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float4* p) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

constexpr unsigned long long kPeerWaitNs = 2000000000ull;      // 2 s: a peer that has not arrived by then is gone

__global__ void __launch_bounds__(1024) peer_allreduce_kernel(const PeerTable tab, const int n4, const int parity,
                                                             float4* __restrict__ out, int* __restrict__ err) {
    __shared__ int give_up;
    __shared__ uint32_t seq_s;
    if (threadIdx.x == 0) {
        give_up = (*reinterpret_cast<volatile int*>(err) != 0);
        uint32_t* counter = tab.flags[tab.rank] + kPeerCounterWord;      // only this kernel, on this rank, touches it
        seq_s = *counter + 1u;
        *counter = seq_s;
    }
    __syncthreads();
    if (give_up) return;
    const uint32_t seq = seq_s;
    // 1. tell every rank (itself included) that this rank's partial `seq` is in place
    if ((int)threadIdx.x < tab.world) st_release_sys(tab.flags[threadIdx.x] + tab.rank, seq);
    // 2. wait for every rank's word in THIS rank's flag area
    if ((int)threadIdx.x < tab.world) {
        const uint32_t* f = tab.flags[tab.rank] + threadIdx.x;
        unsigned long long t0 = 0;
        unsigned spins = 0;
        while ((int)(ld_acquire_sys(f) - seq) < 0) {
            __nanosleep(64);
            if ((++spins & 0xFFu) == 0) {
                unsigned long long now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) t0 = now;
                if (now - t0 > kPeerWaitNs || *reinterpret_cast<volatile int*>(err) != 0) {
                    atomicExch(err, kPeerErrCode);
                    give_up = 1;
                    break;
                }
            }
        }
    }
    __syncthreads();
    if (give_up) return;
    // 3. the sum, in rank order
    const size_t off4 = (size_t)parity * tab.parity_stride4;
    for (int i = threadIdx.x; i < n4; i += blockDim.x) {
        float4 a = ld_peer_f4(reinterpret_cast<const float4*>(tab.data[0]) + off4 + i);
        for (int r = 1; r < tab.world; ++r) {
            const float4 b = ld_peer_f4(reinterpret_cast<const float4*>(tab.data[r]) + off4 + i);
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        out[i] = a;
    }
}

}  // namespace

cudaError_t launch_peer_allreduce(const PeerTable& tab, size_t n, int parity, float* out, int* err_word, cudaStream_t stream) {
    peer_allreduce_kernel<<<1, 1024, 0, stream>>>(tab, (int)(n / 4), parity & 1, reinterpret_cast<float4*>(out), err_word);
    return cudaGetLastError();
}

}  // namespace mcl
