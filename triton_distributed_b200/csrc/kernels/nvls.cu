// Collectives through the NVSwitch multicast engine (NVLS): all-gather with multimem.st,
// reduce-scatter and all-reduce with multimem.ld_reduce (the switch adds the ranks' copies in flight).
//
// The buffer is symmetric memory that every rank also bound to one multicast object; `mc` is the
// multicast alias of it in this process. A multimem.st to mc + x stores to offset x of EVERY rank's
// copy; a multimem.ld_reduce from mc + x returns the sum of all ranks' values at offset x.
//
//   all-gather      rank r multicasts its segment r, then raises its flag on every peer and waits for theirs.
//   reduce-scatter  entry barrier (every rank's input is written), rank r reads the reduced segment r into
//                   its output, exit barrier (nobody overwrites an input a peer still reads).
//   all-reduce      the same, but the reduced segment is multicast back in place instead.
//
// Every wait is bounded and reports through the status block. Reference counterparts:
// kernels/nvidia/low_latency_allgather.py:570-697 (`_forward_push_2d_ll_multimem_kernel`, multimem.st),
// test/nvidia/test_nvshmem_api.py:532-569 (multicast pointer); the reference has no multimem reduce.
#include <cuda_runtime.h>

#include <cstring>

#include "../device/shmem.cuh"
#include "../include/tdist.h"
#include "../runtime/host_common.h"

namespace tdist {

constexpr int kKernelNvls = 8;
constexpr int kNvlsThreads = 512;

struct NvlsParams {
    char* mc;                        // multicast alias of the symmetric buffer [world * seg_bytes]
    char* local;                     // this rank's unicast alias
    uint64_t* sig_peer[kMaxRanks];   // per rank: [0, world) "ready" flags, [world, 2 world) "done" flags
    uint32_t* counters;              // local uint32[2], zero between calls
    char* output;                    // reduce-scatter: local [seg_bytes]
    size_t seg_bytes;
    int world, rank, op, dtype;
    uint64_t epoch;
    WaitCtx wctx;
};

__device__ __forceinline__ void multimem_st_v4(char* mc_addr, const uint4& v) {
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
template <int DTYPE>
__device__ __forceinline__ uint4 multimem_ld_reduce_v4(const char* mc_addr) {
    uint4 v;
    if constexpr (DTYPE == TDIST_BF16)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
    else if constexpr (DTYPE == TDIST_F16)
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
    else
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc_addr) : "memory");
    return v;
}

// The last CTA to get here (its and every earlier CTA's stores fenced) raises flag `slot + rank` on every peer.
__device__ __forceinline__ void last_cta_signals(const NvlsParams& p, int counter, int slot) {
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t old = atom_add_acq_rel_gpu_u32(p.counters + counter, 1);
        if (old == gridDim.x - 1) {
            p.counters[counter] = 0;
            fence_acq_rel_sys();
            for (int r = 0; r < p.world; ++r)
                if (r != p.rank) st_release_sys_u64(p.sig_peer[r] + slot + p.rank, p.epoch);
        }
    }
}
__device__ __forceinline__ void wait_all(const NvlsParams& p, int slot, int where) {
    if (static_cast<int>(threadIdx.x) < p.world && static_cast<int>(threadIdx.x) != p.rank)
        signal_wait_until(p.sig_peer[p.rank] + slot + threadIdx.x, kCmpGe, p.epoch, p.wctx, threadIdx.x, where);
    __syncthreads();
}

constexpr int kNvlsUnroll = 4;  // multimem operations in flight per thread: a switch round trip is long

template <int DTYPE>
__device__ __forceinline__ void reduce_segment(const NvlsParams& p) {
    const size_t nvec = p.seg_bytes / 16;
    const size_t base = static_cast<size_t>(p.rank) * p.seg_bytes;
    const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t nthr = static_cast<size_t>(gridDim.x) * blockDim.x;
    for (size_t i = tid; i < nvec; i += nthr * kNvlsUnroll) {
        uint4 v[kNvlsUnroll];
#pragma unroll
        for (int u = 0; u < kNvlsUnroll; ++u)
            if (i + u * nthr < nvec) v[u] = multimem_ld_reduce_v4<DTYPE>(p.mc + base + (i + u * nthr) * 16);
#pragma unroll
        for (int u = 0; u < kNvlsUnroll; ++u) {
            if (i + u * nthr >= nvec) break;
            if (p.op == TDIST_NVLS_REDUCE_SCATTER) st_v4(p.output + (i + u * nthr) * 16, v[u]);
            else multimem_st_v4(p.mc + base + (i + u * nthr) * 16, v[u]);
        }
    }
}

__global__ void __launch_bounds__(kNvlsThreads) nvls_kernel(const NvlsParams p) {
    if (p.op == TDIST_NVLS_ALLGATHER) {
        const size_t nvec = p.seg_bytes / 16;
        const size_t base = static_cast<size_t>(p.rank) * p.seg_bytes;
        const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
        const size_t nthr = static_cast<size_t>(gridDim.x) * blockDim.x;
        for (size_t i = tid; i < nvec; i += nthr * kNvlsUnroll) {
            uint4 v[kNvlsUnroll];
#pragma unroll
            for (int u = 0; u < kNvlsUnroll; ++u)
                if (i + u * nthr < nvec) v[u] = ld_nc_v4(p.local + base + (i + u * nthr) * 16);
#pragma unroll
            for (int u = 0; u < kNvlsUnroll; ++u)
                if (i + u * nthr < nvec) multimem_st_v4(p.mc + base + (i + u * nthr) * 16, v[u]);
        }
        last_cta_signals(p, 0, 0);
        if (blockIdx.x == 0) wait_all(p, 0, 1);
        return;
    }
    // entry barrier: CTA 0 announces (the inputs were written by earlier work of this stream), every CTA waits
    if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < p.world && static_cast<int>(threadIdx.x) != p.rank) {
        fence_acq_rel_sys();
        st_release_sys_u64(p.sig_peer[threadIdx.x] + p.rank, p.epoch);
    }
    wait_all(p, 0, 2);
    switch (p.dtype) {
        case TDIST_BF16: reduce_segment<TDIST_BF16>(p); break;
        case TDIST_F16: reduce_segment<TDIST_F16>(p); break;
        default: reduce_segment<TDIST_F32>(p); break;
    }
    // exit barrier
    last_cta_signals(p, 1, p.world);
    if (blockIdx.x == 0) wait_all(p, p.world, 3);
}

}  // namespace tdist

using namespace tdist;
using tdist_host::fail;

extern "C" int tdist_nvls(const TdistNvlsArgs* a) {
    if (a == nullptr) return fail(TDIST_EINVAL, "null args");
    if (a->world < 2 || a->world > TDIST_MAX_RANKS || a->rank < 0 || a->rank >= a->world) return fail(TDIST_EINVAL, "nvls: world/rank out of range");
    if (a->op < TDIST_NVLS_ALLGATHER || a->op > TDIST_NVLS_ALLREDUCE) return fail(TDIST_EINVAL, "nvls: bad op");
    if (!a->mc || !a->local || !a->counters) return fail(TDIST_EINVAL, "nvls: null buffer (is the heap bound to a multicast object?)");
    if (a->seg_bytes == 0 || a->seg_bytes % 16 != 0) return fail(TDIST_EINVAL, "nvls: the segment size must be a positive multiple of 16 bytes");
    if (a->op != TDIST_NVLS_ALLGATHER && a->dtype != TDIST_BF16 && a->dtype != TDIST_F16 && a->dtype != TDIST_F32)
        return fail(TDIST_EINVAL, "nvls: reductions take bf16, fp16 or fp32");
    if (a->op == TDIST_NVLS_REDUCE_SCATTER && !a->output) return fail(TDIST_EINVAL, "nvls: reduce-scatter needs an output");
    NvlsParams p;
    memset(&p, 0, sizeof(p));
    p.mc = static_cast<char*>(a->mc);
    p.local = static_cast<char*>(a->local);
    for (int r = 0; r < a->world; ++r) {
        p.sig_peer[r] = static_cast<uint64_t*>(a->sig_peer[r]);
        if (!p.sig_peer[r]) return fail(TDIST_EINVAL, "nvls: null flag pointer");
    }
    p.counters = static_cast<uint32_t*>(a->counters);
    p.output = static_cast<char*>(a->output);
    p.seg_bytes = a->seg_bytes;
    p.world = a->world;
    p.rank = a->rank;
    p.op = a->op;
    p.dtype = a->dtype;
    p.epoch = a->epoch;
    p.wctx.status = static_cast<Status*>(a->status);
    p.wctx.timeout_ns = a->timeout_ns;
    p.wctx.kernel_id = kKernelNvls;
    p.wctx.rank = a->rank;
    int ctas = a->ctas > 0 ? a->ctas : static_cast<int>((a->seg_bytes / 16 + kNvlsThreads * kNvlsUnroll - 1) / (kNvlsThreads * kNvlsUnroll));
    if (ctas < 1) ctas = 1;
    if (ctas > 128) ctas = 128;  // CTAs wait on peers' flags only, never on one another, but stay below one wave
    nvls_kernel<<<ctas, kNvlsThreads, 0, static_cast<cudaStream_t>(a->stream)>>>(p);
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}
