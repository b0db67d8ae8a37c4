// CTA-wide building blocks of the MoE routing kernels: histogram of expert ids, and the stable counting-sort
// positions of (token, k) pairs by expert. Shared by the stand-alone routing kernels (kernels/moe.cu) and by the
// dispatch kernel that routes in place (kernels/moe_ep.cu). All functions are called by every thread of a CTA of
// kMoeThreads threads.
#pragma once
#include <cuda_runtime.h>

#include "signal.cuh"

namespace tdist {

constexpr int kKernelMoe = 6;
constexpr int kMoeThreads = 512;
constexpr int kMoeWarps = kMoeThreads / 32;

__device__ __forceinline__ unsigned lanemask_lt() {
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// An expert id outside [0, E) (a dropped or padded pair, e.g. -1) never indexes shared memory: the pair is
// left out of the histogram and of the sort, and the first such id is recorded in the status block
// (kStatusBadArgument: index = position of the pair, seen = the id, expected = E) for the host to raise.
__device__ __forceinline__ bool expert_in_range(int e, int E) { return e >= 0 && e < E; }
__device__ __forceinline__ void report_bad_expert(const WaitCtx& w, int i, int e, int E, int where) {
    report_timeout(w, kStatusBadArgument, -1, i, E, e, where);
}

// CTA-wide stable counting-sort positions. `running[e]` (smem) holds the next free position of
// expert e and is advanced; `cnt` is smem scratch of kMoeWarps * E ints. emit(i, pos) is called
// once per element in [0, n) whose id is a valid expert; the others get emit(i, -1).
template <typename F>
__device__ __forceinline__ void stable_positions(const int* ids, int n, int E, int* running, int* cnt, const WaitCtx& w,
                                                 F emit) {
    const int tid = static_cast<int>(threadIdx.x);
    const int warp = tid >> 5;
    for (int base = 0; base < n; base += kMoeThreads) {
        for (int j = tid; j < kMoeWarps * E; j += kMoeThreads) cnt[j] = 0;
        __syncthreads();
        const int i = base + tid;
        const int e = i < n ? ids[i] : 0;
        const bool valid = i < n && expert_in_range(e, E);
        if (i < n && !valid) {
            report_bad_expert(w, i, e, E, 2);
            emit(i, -1);
        }
        const int key = valid ? e : E + (tid & 31);  // idle lanes and rejected ids never match anybody
        const unsigned mask = __match_any_sync(0xffffffffu, key);
        const int rank_in_warp = __popc(mask & lanemask_lt());
        if (valid && rank_in_warp == 0) cnt[warp * E + e] = __popc(mask);
        __syncthreads();
        if (valid) {
            int pos = running[e] + rank_in_warp;
            for (int w = 0; w < warp; ++w) pos += cnt[w * E + e];
            emit(i, pos);
        }
        __syncthreads();
        for (int x = tid; x < E; x += kMoeThreads) {
            int s = 0;
            for (int w = 0; w < kMoeWarps; ++w) s += cnt[w * E + x];
            running[x] += s;
        }
        __syncthreads();
    }
}

__device__ __forceinline__ void histogram(const int* ids, int n, int E, int* hist, const WaitCtx& w) {
    for (int x = threadIdx.x; x < E; x += kMoeThreads) hist[x] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += kMoeThreads) {
        const int e = ids[i];
        if (expert_in_range(e, E)) atomicAdd(&hist[e], 1);
        else report_bad_expert(w, i, e, E, 1);
    }
    __syncthreads();
}

}  // namespace tdist
