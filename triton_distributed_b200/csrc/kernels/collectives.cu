// Standalone intra-node collectives on symmetric buffers: barrier, all-gather (pull / push /
// LL-packet), reduce-scatter (push-scatter + fp32 local reduce). One kernel launch per call; the
// data moves with ld/st over NVLink issued by the kernel itself and every wait is bounded.
//
// Reference counterparts: kernels/nvidia/common_ops.py:88-175 (barriers),
// kernels/nvidia/low_latency_allgather.py:48-71 (pull), :345-397 (push), :531-567,700-778 (LL),
// kernels/nvidia/reduce_scatter.py:344-426,527-685 (scatter + ring reduce). The PCIe / NUMA /
// multi-node variants of the reference collapse to these on one NVSwitch node.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../device/ll.cuh"
#include "../device/shmem.cuh"
#include "../include/tdist.h"
#include "../runtime/host_common.h"

namespace tdist {

constexpr int kKernelColl = 2;
constexpr int kCollThreads = 512;

struct CollParams {
    char* buf_peer[kMaxRanks];       // all-gather: the in-place buffer; reduce-scatter: staging of this call's parity
    uint64_t* sig_peer[kMaxRanks];   // [world] arrival flags on every rank
    char* ll_peer[kMaxRanks];        // LL staging of this call's parity: [world][2 * seg_bytes]
    uint32_t* counters;              // local, [world], zero between calls
    const char* input;               // reduce-scatter: local [world * seg] input
    char* output;                    // reduce-scatter: local [seg] output
    size_t seg_bytes;
    int world, rank, mode, phase, ctas_per_peer, dtype;
    uint64_t epoch;
    // fused top-k reduce (reduce-scatter of MoE outputs): row t of the logical input is
    // sum_k topk_w[t*topk+k] * input_row[pos_of[t*topk+k]], computed on the fly (bf16 only); topk == 0 = plain input
    const int* pos_of;
    const float* topk_w;
    int topk, row_bytes;
    WaitCtx wctx;
};

// The CTA group `g` (1..world-1) of this kernel talks to peer (rank + g) % world; group 0 is a
// single CTA that only announces / waits.
__device__ __forceinline__ void group_of(const CollParams& p, int* group, int* slice) {
    if (blockIdx.x == 0) {
        *group = 0;
        *slice = 0;
    } else {
        *group = (static_cast<int>(blockIdx.x) - 1) / p.ctas_per_peer + 1;
        *slice = (static_cast<int>(blockIdx.x) - 1) % p.ctas_per_peer;
    }
}

// [begin, end) of slice `i` of `n` when `bytes` is cut into 16-byte-aligned pieces.
__device__ __forceinline__ void slice_range(size_t bytes, int i, int n, size_t* begin, size_t* end) {
    const size_t units = (bytes + 15) / 16;
    const size_t per = (units + n - 1) / n;
    *begin = min(bytes, per * i * 16);
    *end = min(bytes, per * (i + 1) * 16);
}

// Last CTA of the group of `ctas` (all its stores fenced) publishes this rank's flag on `peer`.
__device__ __forceinline__ void group_signal(const CollParams& p, int peer, int ctas) {
    // one fencing thread per CTA: the barrier orders the CTA's stores before thread 0's release
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t old = atom_add_acq_rel_gpu_u32(p.counters + peer, 1);
        if (old == static_cast<uint32_t>(ctas - 1)) {
            p.counters[peer] = 0;
            fence_acq_rel_sys();
            st_release_sys_u64(p.sig_peer[peer] + p.rank, p.epoch);
        }
    }
}

__global__ void __launch_bounds__(kCollThreads) allgather_kernel(const CollParams p) {
    int g, slice;
    group_of(p, &g, &slice);
    const int peer = (p.rank + g) % p.world;
    char* local = p.buf_peer[p.rank];
    const size_t seg = p.seg_bytes;
    size_t b0, b1;
    slice_range(seg, slice, p.ctas_per_peer, &b0, &b1);

    if (p.mode == TDIST_AG_PUSH) {
        if (g == 0) {
            if ((p.phase & 2) && static_cast<int>(threadIdx.x) < p.world && static_cast<int>(threadIdx.x) != p.rank)
                signal_wait_until(p.sig_peer[p.rank] + threadIdx.x, kCmpGe, p.epoch, p.wctx, threadIdx.x, 1);
            return;
        }
        if (p.phase & 1) {
            copy_coop(p.buf_peer[peer] + p.rank * seg + b0, local + p.rank * seg + b0, b1 - b0, threadIdx.x, blockDim.x);
            group_signal(p, peer, p.ctas_per_peer);
        }
    } else if (p.mode == TDIST_AG_PUSH_ORDERED) {
        if (g == 0) {
            if ((p.phase & 2) && static_cast<int>(threadIdx.x) < p.world && static_cast<int>(threadIdx.x) != p.rank)
                signal_wait_until(p.sig_peer[p.rank] + threadIdx.x, kCmpGe, p.epoch, p.wctx, threadIdx.x, 1);
            return;
        }
        if (p.phase & 1) {
            // every copy CTA sends its slice of the segment to one destination after the other, the rank before this
            // one first: a consumer that starts at its own rows and goes on with rank + 1, rank + 2, ... finds each
            // segment complete about when it gets there, instead of all of them at the end
            const int ctas = (p.world - 1) * p.ctas_per_peer;
            size_t s0, s1;
            slice_range(seg, static_cast<int>(blockIdx.x) - 1, ctas, &s0, &s1);
            for (int h = 1; h < p.world; ++h) {
                int dest = p.rank - h;
                if (dest < 0) dest += p.world;
                copy_coop(p.buf_peer[dest] + p.rank * seg + s0, local + p.rank * seg + s0, s1 - s0, threadIdx.x, blockDim.x);
                group_signal(p, dest, ctas);
            }
        }
    } else if (p.mode == TDIST_AG_PULL) {
        if (g == 0) {
            if ((p.phase & 1) && static_cast<int>(threadIdx.x) < p.world && static_cast<int>(threadIdx.x) != p.rank) {
                fence_acq_rel_sys();
                st_release_sys_u64(p.sig_peer[threadIdx.x] + p.rank, p.epoch);
            }
            return;
        }
        if (p.phase & 2) {
            if (threadIdx.x == 0) signal_wait_until(p.sig_peer[p.rank] + peer, kCmpGe, p.epoch, p.wctx, peer, 2);
            __syncthreads();
            copy_coop(local + peer * seg + b0, p.buf_peer[peer] + peer * seg + b0, b1 - b0, threadIdx.x, blockDim.x);
        }
    } else {  // TDIST_AG_LL
        if (g == 0) return;
        const uint32_t flag = static_cast<uint32_t>(p.epoch);
        const size_t w0 = b0 / 8, w1 = (b1 + 7) / 8;  // 8-byte payload words of this slice
        if (p.phase & 1) {
            const uint64_t* src = reinterpret_cast<const uint64_t*>(local + p.rank * seg);
            char* dst = p.ll_peer[peer] + static_cast<size_t>(p.rank) * seg * 2;
            for (size_t i = w0 + threadIdx.x; i < w1; i += blockDim.x) ll_store(dst + i * 16, src[i], flag);
        }
        if (p.phase & 2) {
            const char* src = p.ll_peer[p.rank] + static_cast<size_t>(peer) * seg * 2;
            uint64_t* dst = reinterpret_cast<uint64_t*>(local + peer * seg);
            for (size_t i = w0 + threadIdx.x; i < w1; i += blockDim.x) {
                uint64_t v;
                ll_load(src + i * 16, flag, &v, p.wctx, peer, static_cast<int>(i));
                dst[i] = v;
            }
        }
    }
}

// 8 bf16 columns (vector c) of logical row t in top-k mode: sum_k w * gathered row, fp32.
__device__ __forceinline__ void topk_vec(const CollParams& p, size_t t, size_t c, float (&acc)[8]) {
    const size_t vpr = static_cast<size_t>(p.row_bytes) / 16;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k0 = 0; k0 < p.topk; k0 += 8) {
        uint4 q[8];
        float w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            w[j] = 0.f;
            q[j] = make_uint4(0, 0, 0, 0);
            if (k0 + j < p.topk) {
                const size_t pair = t * p.topk + k0 + j;
                w[j] = p.topk_w ? p.topk_w[pair] : 1.f;
                q[j] = ld_nc_v4(p.input + (static_cast<size_t>(p.pos_of[pair]) * vpr + c) * 16);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t u[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                acc[2 * i] += w[j] * __uint_as_float(u[i] << 16);
                acc[2 * i + 1] += w[j] * __uint_as_float(u[i] & 0xffff0000u);
            }
        }
    }
}

// out[i] = sum over sources of (staging[src][i] | own input rows), 16 bytes per thread per step.
template <typename T, typename Acc>
__device__ __forceinline__ void reduce_sources(const CollParams& p, size_t first, size_t step) {
    constexpr int V = 16 / sizeof(T);
    const size_t nvec = p.seg_bytes / 16;
    const char* stage = p.buf_peer[p.rank];
    const char* own = p.input + static_cast<size_t>(p.rank) * p.seg_bytes;
    for (size_t i = first; i < nvec; i += step) {
        Acc acc[V];
        bool own_done = false;
        if constexpr (sizeof(T) == 2 && sizeof(Acc) == 4) {
            if (p.topk > 0) {  // bf16 only (checked on the host)
                const size_t vpr = static_cast<size_t>(p.row_bytes) / 16;
                const size_t mpr = p.seg_bytes / p.row_bytes;
                float a8[8];
                topk_vec(p, static_cast<size_t>(p.rank) * mpr + i / vpr, i % vpr, a8);
#pragma unroll
                for (int j = 0; j < V; ++j) acc[j] = static_cast<Acc>(a8[j]);
                own_done = true;
            }
        }
        if (!own_done) {
            const uint4 q = ld_nc_v4(own + i * 16);
            const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
            for (int j = 0; j < V; ++j) acc[j] = static_cast<Acc>(e[j]);
        }
        for (int s = 0; s < p.world; ++s) {
            if (s == p.rank) continue;
            const uint4 q = ld_nc_v4(stage + static_cast<size_t>(s) * p.seg_bytes + i * 16);
            const T* e = reinterpret_cast<const T*>(&q);
#pragma unroll
            for (int j = 0; j < V; ++j) acc[j] += static_cast<Acc>(e[j]);
        }
        uint4 o;
        T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int j = 0; j < V; ++j) oe[j] = static_cast<T>(acc[j]);
        st_v4(p.output + i * 16, o);
    }
}

__global__ void __launch_bounds__(kCollThreads) reduce_scatter_kernel(const CollParams p) {
    int g, slice;
    group_of(p, &g, &slice);
    const int peer = (p.rank + g) % p.world;
    const size_t seg = p.seg_bytes;
    if (g > 0 && (p.phase & 1)) {
        size_t b0, b1;
        slice_range(seg, slice, p.ctas_per_peer, &b0, &b1);
        char* dst = p.buf_peer[peer] + static_cast<size_t>(p.rank) * seg;
        if (p.topk > 0) {
            // the peer's rows do not exist anywhere yet: reduce the top-k expert outputs of each token straight
            // into the peer's staging
            const size_t vpr = static_cast<size_t>(p.row_bytes) / 16;
            const size_t mpr = seg / p.row_bytes;
            for (size_t v = b0 / 16 + threadIdx.x; v < b1 / 16; v += blockDim.x) {
                float a8[8];
                topk_vec(p, static_cast<size_t>(peer) * mpr + v / vpr, v % vpr, a8);
                uint4 o;
                o.x = pack_bf16x2(a8[0], a8[1]);
                o.y = pack_bf16x2(a8[2], a8[3]);
                o.z = pack_bf16x2(a8[4], a8[5]);
                o.w = pack_bf16x2(a8[6], a8[7]);
                st_v4(dst + v * 16, o);
            }
        } else {
            copy_coop(dst + b0, p.input + static_cast<size_t>(peer) * seg + b0, b1 - b0, threadIdx.x, blockDim.x);
        }
        group_signal(p, peer, p.ctas_per_peer);
    }
    if (!(p.phase & 2)) return;
    // every CTA waits for all sources, then takes its share of the reduction
    if (static_cast<int>(threadIdx.x) < p.world && static_cast<int>(threadIdx.x) != p.rank)
        signal_wait_until(p.sig_peer[p.rank] + threadIdx.x, kCmpGe, p.epoch, p.wctx, threadIdx.x, 3);
    __syncthreads();
    const size_t first = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    const size_t step = static_cast<size_t>(gridDim.x) * blockDim.x;
    switch (p.dtype) {
        case TDIST_BF16: reduce_sources<__nv_bfloat16, float>(p, first, step); break;
        case TDIST_F16: reduce_sources<__half, float>(p, first, step); break;
        case TDIST_F32: reduce_sources<float, float>(p, first, step); break;
        default: reduce_sources<int, int>(p, first, step); break;
    }
}

// out[i] = sum over the `splits` row blocks of `in` (block stride `block_bytes`), fp32 accumulation, visiting the
// blocks in ring order from `begin`. (reference kernels/nvidia/reduce_scatter.py:616-685 `kernel_ring_reduce_*`)
template <typename T, typename Acc>
__global__ void __launch_bounds__(kCollThreads) ring_reduce_kernel(const char* in, char* out, size_t block_bytes, int splits, int begin) {
    constexpr int V = 16 / sizeof(T);
    const size_t nvec = block_bytes / 16;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        Acc acc[V];
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] = Acc(0);
        for (int s0 = 0; s0 < splits; s0 += 4) {
            uint4 q[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                int s = begin + s0 + u;
                if (s >= splits) s -= splits;
                if (s0 + u < splits) q[u] = ld_nc_v4(in + static_cast<size_t>(s) * block_bytes + i * 16);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (s0 + u >= splits) break;
                const T* e = reinterpret_cast<const T*>(&q[u]);
#pragma unroll
                for (int j = 0; j < V; ++j) acc[j] += static_cast<Acc>(e[j]);
            }
        }
        uint4 o;
        T* oe = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int j = 0; j < V; ++j) oe[j] = static_cast<T>(acc[j]);
        st_v4(out + i * 16, o);
    }
}

__global__ void barrier_all_kernel(SymmWindow win, BarrierState st, WaitCtx wctx) {
    barrier_all_block(win, st, wctx);
}

}  // namespace tdist

using namespace tdist;
using tdist_host::fail;

static int fill_params(const TdistCollArgs* a, CollParams* p) {
    if (a->world < 1 || a->world > TDIST_MAX_RANKS || a->rank < 0 || a->rank >= a->world)
        return fail(TDIST_EINVAL, "collective: world/rank out of range");
    memset(p, 0, sizeof(*p));
    for (int r = 0; r < a->world; ++r) {
        p->buf_peer[r] = static_cast<char*>(a->buf_peer[r]);
        p->sig_peer[r] = static_cast<uint64_t*>(a->sig_peer[r]);
        p->ll_peer[r] = static_cast<char*>(a->ll_peer[r]);
        if (p->buf_peer[r] == nullptr || p->sig_peer[r] == nullptr) return fail(TDIST_EINVAL, "collective: null peer pointer");
    }
    p->counters = static_cast<uint32_t*>(a->counters);
    p->input = static_cast<const char*>(a->input);
    p->output = static_cast<char*>(a->output);
    p->seg_bytes = a->seg_bytes;
    p->world = a->world;
    p->rank = a->rank;
    p->mode = a->mode;
    p->phase = a->phase ? a->phase : 3;
    p->dtype = a->dtype;
    p->epoch = a->epoch;
    p->pos_of = static_cast<const int*>(a->pos_of);
    p->topk_w = static_cast<const float*>(a->topk_w);
    p->topk = a->topk;
    p->row_bytes = a->row_bytes;
    p->ctas_per_peer = a->ctas_per_peer > 0 ? a->ctas_per_peer : 4;
    // plain copies saturate NVLink with a few CTAs per peer; the fused top-k reduce is compute and wants the whole GPU
    if (p->ctas_per_peer > (a->topk > 0 ? 144 : 16)) p->ctas_per_peer = a->topk > 0 ? 144 : 16;
    p->wctx.status = static_cast<Status*>(a->status);
    p->wctx.timeout_ns = a->timeout_ns;
    p->wctx.kernel_id = kKernelColl;
    p->wctx.rank = a->rank;
    if (p->counters == nullptr) return fail(TDIST_EINVAL, "collective: counters pointer is null");
    return 0;
}

extern "C" int tdist_allgather(const TdistCollArgs* a) {
    CollParams p;
    int rc = fill_params(a, &p);
    if (rc) return rc;
    if (a->mode < TDIST_AG_PULL || a->mode > TDIST_AG_PUSH_ORDERED) return fail(TDIST_EINVAL, "allgather: bad mode");
    if (a->mode == TDIST_AG_LL) {
        if (a->seg_bytes % 8 != 0) return fail(TDIST_EINVAL, "LL all-gather needs a segment size that is a multiple of 8 bytes");
        for (int r = 0; r < a->world; ++r)
            if (p.ll_peer[r] == nullptr) return fail(TDIST_EINVAL, "LL all-gather needs the LL staging of every rank");
    }
    if (a->world == 1) return 0;
    const int grid = 1 + (a->world - 1) * p.ctas_per_peer;
    allgather_kernel<<<grid, kCollThreads, 0, static_cast<cudaStream_t>(a->stream)>>>(p);
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}

extern "C" int tdist_reduce_scatter(const TdistCollArgs* a) {
    CollParams p;
    int rc = fill_params(a, &p);
    if (rc) return rc;
    if (a->seg_bytes % 16 != 0) return fail(TDIST_EINVAL, "reduce-scatter needs a segment size that is a multiple of 16 bytes");
    if (a->input == nullptr || a->output == nullptr) return fail(TDIST_EINVAL, "reduce-scatter: null input/output");
    if (a->dtype < TDIST_BF16 || a->dtype > TDIST_I32) return fail(TDIST_EINVAL, "reduce-scatter: bad dtype");
    if (a->topk < 0 || a->topk > 64) return fail(TDIST_EINVAL, "reduce-scatter: topk out of range");
    if (a->topk > 0) {
        if (a->dtype != TDIST_BF16) return fail(TDIST_EINVAL, "reduce-scatter with top-k reduce takes bf16");
        if (a->pos_of == nullptr || a->row_bytes <= 0 || a->row_bytes % 16 != 0 || a->seg_bytes % a->row_bytes != 0)
            return fail(TDIST_EINVAL, "reduce-scatter with top-k reduce needs pos_of and a row size that is a multiple of 16 bytes and divides the segment");
    }
    const int grid = 1 + (a->world - 1) * p.ctas_per_peer;
    reduce_scatter_kernel<<<grid, kCollThreads, 0, static_cast<cudaStream_t>(a->stream)>>>(p);
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}

extern "C" int tdist_barrier_all(void* const* flags_peer, void* epoch_local, int world, int rank, void* status,
                                 uint64_t timeout_ns, void* stream) {
    if (world < 1 || world > TDIST_MAX_RANKS) return fail(TDIST_EINVAL, "barrier: world out of range");
    SymmWindow win;
    memset(&win, 0, sizeof(win));
    for (int r = 0; r < world; ++r) win.base[r] = static_cast<char*>(flags_peer[r]);
    win.rank = rank;
    win.world = world;
    win.bytes = 0;   // the caller passes bare pointers: the size of the flag object is not known here
    win.dbg = static_cast<Status*>(status);
    BarrierState st;
    st.flags = static_cast<uint64_t*>(flags_peer[rank]);
    st.epoch = static_cast<uint64_t*>(epoch_local);
    WaitCtx w;
    w.status = static_cast<Status*>(status);
    w.timeout_ns = timeout_ns;
    w.kernel_id = kKernelColl;
    w.rank = rank;
    barrier_all_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(win, st, w);
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}

extern "C" int tdist_ring_reduce(const void* in, void* out, size_t block_bytes, int splits, int begin, int dtype, void* stream) {
    if (in == nullptr || out == nullptr || splits < 1 || begin < 0 || begin >= splits) return fail(TDIST_EINVAL, "ring_reduce: bad arguments");
    if (block_bytes == 0 || block_bytes % 16 != 0) return fail(TDIST_EINVAL, "ring_reduce: the block size must be a positive multiple of 16 bytes");
    if ((reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15)) return fail(TDIST_EINVAL, "ring_reduce: pointers must be 16-byte aligned");
    int grid = static_cast<int>((block_bytes / 16 + kCollThreads - 1) / kCollThreads);
    if (grid > 1184) grid = 1184;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const char* i8 = static_cast<const char*>(in);
    char* o8 = static_cast<char*>(out);
    switch (dtype) {
        case TDIST_BF16: ring_reduce_kernel<__nv_bfloat16, float><<<grid, kCollThreads, 0, st>>>(i8, o8, block_bytes, splits, begin); break;
        case TDIST_F16: ring_reduce_kernel<__half, float><<<grid, kCollThreads, 0, st>>>(i8, o8, block_bytes, splits, begin); break;
        case TDIST_F32: ring_reduce_kernel<float, float><<<grid, kCollThreads, 0, st>>>(i8, o8, block_bytes, splits, begin); break;
        case TDIST_I32: ring_reduce_kernel<int, int><<<grid, kCollThreads, 0, st>>>(i8, o8, block_bytes, splits, begin); break;
        default: return fail(TDIST_EINVAL, "ring_reduce: bad dtype");
    }
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}
