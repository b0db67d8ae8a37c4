// MoE routing kernels: softmax + top-k selection, expert-sorted permutation of (token, k) pairs,
// and the block-aligned, rank-major sort that the MoE group-GEMMs consume.
//
// Reference counterparts: `select_experts` (torch softmax/topk; kernels/nvidia/moe_reduce_rs.py:180-197),
// `kernel_bincount` + torch argsort/cumsum (kernels/nvidia/ep_a2a.py:309-321, test_all_to_all.py
// `calc_gather_index`), and the hand-written `moe_ag_scatter_align_block_size_kernel`
// (csrc/lib/moe_utils.cu:60-192) with its Python oracle `full_moe_align_block_size`
// (kernels/nvidia/moe_reduce_rs.py:87-177). The sorts here are stable (ascending pair index inside
// an expert), so results are reproducible and comparable element by element with the oracle.
#include <cuda_runtime.h>
#include <math_constants.h>

#include "../device/moe_sort.cuh"
#include "../device/signal.cuh"
#include "../include/tdist.h"
#include "../runtime/host_common.h"

namespace tdist {

// ---------------------------------------------------------------------------- routing for EP
// ids[n] (n = tokens * topk, token-major) -> splits[E], cumsum[E+1], sorted_token[n] (token of the
// pair at each sorted position), slot_of[n] (sorted position of each pair). One CTA.
__global__ void __launch_bounds__(kMoeThreads) moe_route_kernel(const int* ids, int n, int topk, int E, int* splits,
                                                                int* cumsum, int* sorted_token, int* slot_of,
                                                                WaitCtx w) {
    extern __shared__ int sm[];
    int* hist = sm;
    int* running = sm + E;
    int* cnt = sm + 2 * E;
    histogram(ids, n, E, hist, w);
    if (threadIdx.x < 32) {
        // exclusive scan of the histogram by one warp: a contiguous chunk of experts per lane
        const int lane = threadIdx.x;
        const int per = (E + 31) / 32;
        const int e0 = min(E, lane * per), e1 = min(E, e0 + per);
        int local = 0;
        for (int e = e0; e < e1; ++e) local += hist[e];
        int incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        int acc = incl - local;
        for (int e = e0; e < e1; ++e) {
            running[e] = acc;
            cumsum[e] = acc;
            splits[e] = hist[e];
            acc += hist[e];
        }
        if (lane == 31) cumsum[E] = incl;
    }
    __syncthreads();
    stable_positions(ids, n, E, running, cnt, w, [&](int i, int pos) {
        slot_of[i] = pos;   // -1 for a pair whose expert id was rejected
        if (pos >= 0) sorted_token[pos] = i / topk;
    });
}

// ---------------------------------------------------------------------------- block-aligned sort
// One CTA per source rank. See the header comment for the layout.
__global__ void __launch_bounds__(kMoeThreads) moe_align_kernel(const int* ids, int numel_per_rank, int E, int num_ranks,
                                                                int block_size, int* sorted_ids, int sorted_cap,
                                                                int* expert_ids, int* block_barrier_ids,
                                                                int* rank_block_num, int* num_tokens_post_pad,
                                                                WaitCtx w) {
    extern __shared__ int sm[];
    int* hist = sm;
    int* running = sm + E;
    int* cnt = sm + 2 * E;
    __shared__ int base_s, total_s;
    const int r = static_cast<int>(blockIdx.x);
    const int pad_value = numel_per_rank * num_ranks;
    if (threadIdx.x == 0) base_s = 0;
    // padded sizes of the earlier ranks give this rank's base offset
    for (int q = 0; q <= r; ++q) {
        histogram(ids + static_cast<size_t>(q) * numel_per_rank, numel_per_rank, E, hist, w);
        if (threadIdx.x == 0) {
            int acc = 0;
            for (int e = 0; e < E; ++e) {
                if (q == r) running[e] = acc;
                acc += (hist[e] + block_size - 1) / block_size * block_size;
            }
            if (q < r) base_s += acc;
            else total_s = acc;
        }
        __syncthreads();
    }
    const int base = base_s, total = total_s;
    if (threadIdx.x == 0) {
        rank_block_num[r] = total / block_size;
        if (r == num_ranks - 1) *num_tokens_post_pad = base + total;
    }
    // block -> expert / source-rank tables and padding of this rank's region (and of the tail)
    for (int e = threadIdx.x; e < E; e += kMoeThreads) {
        const int b0 = running[e] / block_size;
        const int nb = (hist[e] + block_size - 1) / block_size;
        for (int b = 0; b < nb; ++b) {
            expert_ids[base / block_size + b0 + b] = e;
            block_barrier_ids[base / block_size + b0 + b] = r;
        }
    }
    const int fill_end = (r == num_ranks - 1) ? sorted_cap : base + total;
    for (int i = base + threadIdx.x; i < fill_end; i += kMoeThreads) sorted_ids[i] = pad_value;
    __syncthreads();
    const int* my = ids + static_cast<size_t>(r) * numel_per_rank;
    stable_positions(my, numel_per_rank, E, running, cnt, w, [&](int i, int pos) {
        if (pos >= 0) sorted_ids[base + pos] = i + r * numel_per_rank;
    });
}

// ---------------------------------------------------------------------------- softmax + top-k
// One warp per token; E <= 1024. weights = softmax probabilities of the selected experts,
// optionally renormalised to sum to one. Ties go to the lower expert index.
__global__ void moe_topk_softmax_kernel(const float* logits, int ntok, int E, int topk, int renorm, int* ids, float* w) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= ntok) return;
    const float* row = logits + static_cast<size_t>(warp) * E;
    float v[32];
    float mx = -CUDART_INF_F;
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const int e = j * 32 + lane;
        v[j] = e < E ? row[e] : -CUDART_INF_F;
        mx = fmaxf(mx, v[j]);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 32; ++j) sum += (j * 32 + lane < E) ? __expf(v[j] - mx) : 0.f;
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    float picked_sum = 0.f;
    float my_w = 0.f;
    int my_id = 0;
    for (int k = 0; k < topk; ++k) {
        float best = -CUDART_INF_F;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            const int e = j * 32 + lane;
            if (v[j] > best) {
                best = v[j];
                best_e = e;
            }
        }
#pragma unroll
        for (int o = 16; o; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) {
                best = ob;
                best_e = oe;
            }
        }
        const float prob = __expf(best - mx) / sum;
        picked_sum += prob;
        if (lane == k) {
            my_w = prob;
            my_id = best_e;
        }
        if ((best_e & 31) == lane) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (j == (best_e >> 5)) v[j] = -CUDART_INF_F;
        }
    }
    if (lane < topk) {
        ids[static_cast<size_t>(warp) * topk + lane] = my_id;
        w[static_cast<size_t>(warp) * topk + lane] = renorm ? my_w / picked_sum : my_w;
    }
}

// ---------------------------------------------------------------------------- row gather / top-k reduce
// dst[p] = src[index[p] / div] for index[p] < limit, zeros otherwise (padding rows of the aligned
// sort); optionally records the inverse map pos_of[index[p]] = p. One warp per row, 16-byte vectors.
__global__ void gather_rows_kernel(const uint4* src, const int* index, int rows_out, int div, int limit, int vec_per_row,
                                   uint4* dst, int* pos_of) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    for (int p = warp; p < rows_out; p += nwarps) {
        const int id = index[p];
        const bool live = id >= 0 && id < limit;
        if (live && pos_of != nullptr && lane == 0) pos_of[id] = p;
        const uint4* s = src + static_cast<size_t>(live ? id / div : 0) * vec_per_row;
        uint4* d = dst + static_cast<size_t>(p) * vec_per_row;
        for (int c = lane; c < vec_per_row; c += 32) d[c] = live ? s[c] : make_uint4(0, 0, 0, 0);
    }
}

// out[t] = sum_k w[t*topk+k] * y[pos_of[t*topk+k]] in fp32 (bf16 in/out). One warp per token.
__global__ void topk_reduce_kernel(const uint4* y, const int* pos_of, const float* w, int ntok, int topk, int vec_per_row,
                                   uint4* out) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    for (int t = warp; t < ntok; t += nwarps) {
        for (int c = lane; c < vec_per_row; c += 32) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int k = 0; k < topk; ++k) {
                const int pos = pos_of[t * topk + k];
                if (pos < 0) continue;   // a pair that routing rejected contributes nothing
                const float wk = w ? w[t * topk + k] : 1.f;
                const uint4 q = y[static_cast<size_t>(pos) * vec_per_row + c];
                const uint32_t u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    acc[2 * i] += wk * __uint_as_float(u[i] << 16);
                    acc[2 * i + 1] += wk * __uint_as_float(u[i] & 0xffff0000u);
                }
            }
            uint4 o;
            uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t r;
                asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(acc[2 * i + 1]), "f"(acc[2 * i]));
                ow[i] = r;
            }
            out[static_cast<size_t>(t) * vec_per_row + c] = o;
        }
    }
}

}  // namespace tdist

using namespace tdist;
using tdist_host::fail;

static int moe_smem_bytes(int E) { return (2 * E + kMoeWarps * E) * static_cast<int>(sizeof(int)); }

template <typename K>
static int ensure_smem(K kernel, int bytes) {
    if (bytes > 48 * 1024) TDIST_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    return 0;
}

static WaitCtx moe_wctx(void* status) {
    WaitCtx w;
    w.status = static_cast<Status*>(status);
    w.timeout_ns = 0;
    w.kernel_id = kKernelMoe;
    w.rank = 0;
    return w;
}

extern "C" int tdist_moe_route(const void* ids, int n, int topk, int num_experts, void* splits, void* cumsum,
                               void* sorted_token, void* slot_of, void* status, void* stream) {
    if (num_experts < 1 || num_experts > 2048) return fail(TDIST_ELIMIT, "moe_route: at most 2048 experts");
    if (topk < 1 || n < 0) return fail(TDIST_EINVAL, "moe_route: bad sizes");
    const int smem = moe_smem_bytes(num_experts);
    int rc = ensure_smem(moe_route_kernel, smem);
    if (rc) return rc;
    moe_route_kernel<<<1, kMoeThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const int*>(ids), n, topk, num_experts, static_cast<int*>(splits), static_cast<int*>(cumsum),
        static_cast<int*>(sorted_token), static_cast<int*>(slot_of), moe_wctx(status));
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}

extern "C" int tdist_moe_align_block_size(const void* ids, int numel_per_rank, int num_experts, int num_ranks,
                                          int block_size, void* sorted_ids, int sorted_cap, void* expert_ids,
                                          void* block_barrier_ids, void* rank_block_num, void* num_tokens_post_pad,
                                          void* status, void* stream) {
    if (num_experts < 1 || num_experts > 2048) return fail(TDIST_ELIMIT, "moe_align: at most 2048 experts");
    if (block_size < 1 || num_ranks < 1) return fail(TDIST_EINVAL, "moe_align: bad sizes");
    const int smem = moe_smem_bytes(num_experts);
    int rc = ensure_smem(moe_align_kernel, smem);
    if (rc) return rc;
    moe_align_kernel<<<num_ranks, kMoeThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const int*>(ids), numel_per_rank, num_experts, num_ranks, block_size, static_cast<int*>(sorted_ids),
        sorted_cap, static_cast<int*>(expert_ids), static_cast<int*>(block_barrier_ids), static_cast<int*>(rank_block_num),
        static_cast<int*>(num_tokens_post_pad), moe_wctx(status));
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}

extern "C" int tdist_moe_topk_softmax(const void* logits, int ntok, int num_experts, int topk, int renormalize,
                                      void* ids, void* weights, void* stream) {
    if (num_experts < 1 || num_experts > 1024) return fail(TDIST_ELIMIT, "moe_topk_softmax: at most 1024 experts");
    if (topk < 1 || topk > 32 || topk > num_experts) return fail(TDIST_EINVAL, "moe_topk_softmax: topk must be in [1, min(32, experts)]");
    if (ntok <= 0) return 0;
    const int warps_per_block = 8;
    const int blocks = (ntok + warps_per_block - 1) / warps_per_block;
    moe_topk_softmax_kernel<<<blocks, warps_per_block * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float*>(logits), ntok, num_experts, topk, renormalize, static_cast<int*>(ids),
        static_cast<float*>(weights));
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}

extern "C" int tdist_gather_rows(const void* src, const void* index, int rows_out, int div, int limit, int row_bytes,
                                 void* dst, void* pos_of, void* stream) {
    if (row_bytes % 16 || div < 1) return fail(TDIST_EINVAL, "gather_rows: rows must be multiples of 16 bytes");
    if (rows_out <= 0) return 0;
    const int blocks = (rows_out + 7) / 8 < 1184 ? (rows_out + 7) / 8 : 1184;
    gather_rows_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(src), static_cast<const int*>(index), rows_out, div, limit, row_bytes / 16,
        static_cast<uint4*>(dst), static_cast<int*>(pos_of));
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}

extern "C" int tdist_topk_reduce(const void* y, const void* pos_of, const void* weights, int ntok, int topk, int row_bytes,
                                 void* out, void* stream) {
    if (row_bytes % 16 || topk < 1) return fail(TDIST_EINVAL, "topk_reduce: rows must be multiples of 16 bytes");
    if (ntok <= 0) return 0;
    const int blocks = (ntok + 7) / 8 < 1184 ? (ntok + 7) / 8 : 1184;
    topk_reduce_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(y), static_cast<const int*>(pos_of), static_cast<const float*>(weights), ntok, topk,
        row_bytes / 16, static_cast<uint4*>(out));
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}
