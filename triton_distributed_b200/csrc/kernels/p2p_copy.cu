// Peer-to-peer copy kernels over NVLink, in the five data paths the fused ops choose between.
// They back `tdist.utils.p2p_bandwidth` (a topology / bandwidth probe like the GB/s printouts of
// the reference's test_all_gather.py and tutorials/03-inter-node-allgather.py:223-237) and the
// standalone collectives.
//
//   mode 0  push, TMA both ways:   bulk load local -> smem, bulk store smem -> peer (one thread)
//   mode 1  push, TMA in / LSU out: bulk load local -> smem, all threads st.global.v4 to the peer
//   mode 2  push, LSU both ways:   every thread ld.global.v4 local, st.global.v4 peer
//   mode 3  pull, TMA both ways:   bulk load peer -> smem, bulk store smem -> local
//   mode 4  pull, LSU both ways:   every thread ld.global.v4 peer, st.global.v4 local
//
// `src` / `dst` are plain device pointers: the caller passes a peer-mapped address for whichever
// side is remote. The copy is split evenly over the CTAs; sizes must be multiples of 16 bytes.
#include <cuda_runtime.h>

#include "../device/ptx.cuh"
#include "../device/signal.cuh"
#include "../include/tdist.h"
#include "../runtime/host_common.h"

namespace tdist {

constexpr int kCopyStages = 8;
constexpr int kKernelCopy = 2;

struct CopyParams {
    const char* src;
    char* dst;
    size_t bytes;
    int mode;
    int chunk;   // bytes per bulk operation (modes 0, 1, 3), multiple of 16, <= smem / stages
    WaitCtx wctx;
};

__device__ __forceinline__ uint4 ld_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_v4(void* p, const uint4& v) {
    asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__global__ void __launch_bounds__(512, 1) p2p_copy_kernel(const CopyParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    __shared__ uint64_t full[kCopyStages];
    __shared__ uint64_t empty[kCopyStages];

    // this CTA's slice, 16-byte granular
    const size_t units = p.bytes / 16;
    const size_t per = (units + gridDim.x - 1) / gridDim.x;
    const size_t u0 = min(units, per * blockIdx.x);
    const size_t u1 = min(units, u0 + per);
    const char* src = p.src + u0 * 16;
    char* dst = p.dst + u0 * 16;
    const size_t bytes = (u1 - u0) * 16;
    if (bytes == 0) return;

    if (p.mode == 2 || p.mode == 4) {
        constexpr int U = 8;
        const size_t n = bytes / 16;
        const size_t stride = static_cast<size_t>(blockDim.x);
        size_t i = threadIdx.x;
        for (; i + (U - 1) * stride < n; i += U * stride) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) v[u] = ld_v4(src + (i + u * stride) * 16);
#pragma unroll
            for (int u = 0; u < U; ++u) st_v4(dst + (i + u * stride) * 16, v[u]);
        }
        for (; i < n; i += stride) st_v4(dst + i * 16, ld_v4(src + i * 16));
        return;
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < kCopyStages; ++s) {
            mbar_init(smem_u32(&full[s]), 1);
            mbar_init(smem_u32(&empty[s]), blockDim.x - 32);
        }
        fence_mbar_init();
    }
    __syncthreads();
    const int nchunks = static_cast<int>((bytes + p.chunk - 1) / p.chunk);

    if (p.mode == 0 || p.mode == 3) {
        if (threadIdx.x != 0) return;
        constexpr int AHEAD = kCopyStages - 2;
        for (int c = 0; c < nchunks + AHEAD; ++c) {
            if (c < nchunks) {
                const int s = c % kCopyStages;
                if (c >= kCopyStages) bulk_wait_read<kCopyStages - AHEAD - 1>();
                const size_t off = static_cast<size_t>(c) * p.chunk;
                const uint32_t sz = static_cast<uint32_t>(min(static_cast<size_t>(p.chunk), bytes - off));
                mbar_expect_tx(smem_u32(&full[s]), sz);
                bulk_load(smem_u32(smem + static_cast<size_t>(s) * p.chunk), src + off, sz, smem_u32(&full[s]));
            }
            if (c >= AHEAD) {
                const int cs = c - AHEAD;
                const int s = cs % kCopyStages;
                mbar_wait(smem_u32(&full[s]), (cs / kCopyStages) & 1u, p.wctx, 1);
                const size_t off = static_cast<size_t>(cs) * p.chunk;
                const uint32_t sz = static_cast<uint32_t>(min(static_cast<size_t>(p.chunk), bytes - off));
                bulk_store(dst + off, smem_u32(smem + static_cast<size_t>(s) * p.chunk), sz);
                bulk_commit();
            }
        }
        bulk_wait<0>();
        return;
    }

    // mode 1: warp 0 feeds smem with bulk loads, the other warps drain it with vector stores
    if (threadIdx.x < 32) {
        if (threadIdx.x == 0) {
            for (int c = 0; c < nchunks; ++c) {
                const int s = c % kCopyStages;
                mbar_wait(smem_u32(&empty[s]), ((c / kCopyStages) & 1u) ^ 1u, p.wctx, 2);
                const size_t off = static_cast<size_t>(c) * p.chunk;
                const uint32_t sz = static_cast<uint32_t>(min(static_cast<size_t>(p.chunk), bytes - off));
                mbar_expect_tx(smem_u32(&full[s]), sz);
                bulk_load(smem_u32(smem + static_cast<size_t>(s) * p.chunk), src + off, sz, smem_u32(&full[s]));
            }
        }
        return;
    }
    const int t = static_cast<int>(threadIdx.x) - 32;
    const int nt = static_cast<int>(blockDim.x) - 32;
    for (int c = 0; c < nchunks; ++c) {
        const int s = c % kCopyStages;
        mbar_wait(smem_u32(&full[s]), (c / kCopyStages) & 1u, p.wctx, 3);
        const size_t off = static_cast<size_t>(c) * p.chunk;
        const int sz = static_cast<int>(min(static_cast<size_t>(p.chunk), bytes - off));
        const uint8_t* sp = smem + static_cast<size_t>(s) * p.chunk;
        for (int i = t * 16; i < sz; i += nt * 16) st_v4(dst + off + i, *reinterpret_cast<const uint4*>(sp + i));
        mbar_arrive(smem_u32(&empty[s]));
    }
}

}  // namespace tdist

extern "C" int tdist_p2p_copy(const void* src, void* dst, size_t bytes, int mode, int ctas, int threads, int chunk,
                              void* status, uint64_t timeout_ns, void* stream) {
    using namespace tdist;
    if (bytes % 16 != 0 || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15))
        return tdist_host::fail(TDIST_EINVAL, "p2p_copy: pointers and size must be 16-byte aligned");
    if (mode < 0 || mode > 4) return tdist_host::fail(TDIST_EINVAL, "p2p_copy: mode must be 0..4");
    if (ctas < 1) ctas = 1;
    if (threads < 64) threads = 64;
    if (threads > 512) threads = 512;
    threads = threads / 32 * 32;
    if (chunk <= 0) chunk = 16384;
    chunk = chunk / 16 * 16;
    if (chunk > 24 * 1024) chunk = 24 * 1024;
    CopyParams p;
    p.src = static_cast<const char*>(src);
    p.dst = static_cast<char*>(dst);
    p.bytes = bytes;
    p.mode = mode;
    p.chunk = chunk;
    p.wctx.status = static_cast<Status*>(status);
    p.wctx.timeout_ns = timeout_ns;
    p.wctx.kernel_id = kKernelCopy;
    p.wctx.rank = 0;
    const int smem = kCopyStages * chunk + 256;
    static bool attr_set[64] = {};
    int dev = 0;
    TDIST_CUDA_OK(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        TDIST_CUDA_OK(cudaFuncSetAttribute(p2p_copy_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        attr_set[dev] = true;
    }
    p2p_copy_kernel<<<ctas, threads, smem, static_cast<cudaStream_t>(stream)>>>(p);
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}

// ---- stream-ordered signal operations on raw (already peer-mapped) addresses: the host face of
// signal_op / signal_wait_until (reference pynvshmem putmem_signal_on_stream, common_ops.py set_signal / wait_eq).
namespace tdist {
__global__ void signal_op_kernel(uint64_t* sig, uint64_t value, int sig_op) {
    // everything the stream did before this kernel (e.g. the copy of putmem_signal_on_stream) is complete
    fence_acq_rel_sys();
    if (sig_op == kSignalAdd) red_release_sys_add_u64(sig, value);
    else st_release_sys_u64(sig, value);
}
__global__ void signal_wait_kernel(const uint64_t* sig, int cmp, uint64_t value, WaitCtx wctx) {
    signal_wait_until(sig, cmp, value, wctx, -1, 1);
}
}  // namespace tdist

extern "C" int tdist_signal_op_on_stream(void* sig, uint64_t value, int sig_op, void* stream) {
    if (sig == nullptr || (reinterpret_cast<uintptr_t>(sig) & 7)) return tdist_host::fail(TDIST_EINVAL, "signal_op: the signal must be an 8-byte aligned address");
    if (sig_op != tdist::kSignalSet && sig_op != tdist::kSignalAdd) return tdist_host::fail(TDIST_EINVAL, "signal_op: sig_op must be 9 (set) or 10 (add)");
    tdist::signal_op_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint64_t*>(sig), value, sig_op);
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}

extern "C" int tdist_signal_wait_on_stream(const void* sig, int cmp, uint64_t value, void* status, uint64_t timeout_ns, void* stream) {
    if (sig == nullptr || (reinterpret_cast<uintptr_t>(sig) & 7)) return tdist_host::fail(TDIST_EINVAL, "signal_wait: the signal must be an 8-byte aligned address");
    if (cmp < 0 || cmp > 5) return tdist_host::fail(TDIST_EINVAL, "signal_wait: cmp must be 0..5 (EQ NE GT LE LT GE)");
    tdist::WaitCtx w;
    w.status = static_cast<tdist::Status*>(status);
    w.timeout_ns = timeout_ns;
    w.kernel_id = tdist::kKernelCopy;
    w.rank = 0;
    tdist::signal_wait_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint64_t*>(sig), cmp, value, w);
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}
