// GQA flash-decode over a paged KV cache, split along the KV sequence, with the split merge — and
// in sequence-parallel mode the cross-rank exchange and merge — fused into the same launch.
//
// Grid = batch x kv_heads x splits CTAs of 4 warps. A CTA owns one (batch, kv head, KV range): the
// G = Hq/Hkv query heads sharing that kv head form the rows of a 16-row Q tile (rows >= G are
// zero), each warp streams 16-token K/V blocks of the range through its own cp.async ring
// (no CTA barrier in the main loop) and runs QK^T and PV on tensor cores (mma.sync m16n8k16: at 4..16
// live rows a tcgen05 tile would be mostly padding and the kernel is HBM-bound anyway), with an
// online softmax in the exp2 domain. Warps are merged through shared memory, the split result
// (normalised O, natural-log LSE) goes to a workspace, and the LAST CTA to finish a (batch, kv head)
// merges all splits. With up to eight splits the CTAs of a (batch, kv head) are launched as one thread-block
// cluster instead: every CTA stores its result straight into the first CTA's shared memory (st.shared::cluster), a
// cluster barrier follows, and that CTA merges out of its own shared memory: no workspace, no fence, no counter.
// In sequence-parallel mode the merging CTA then writes the merged O||LSE of its heads
// into every rank's gather buffer as LL packets (payload + flag in one 16-byte store, no fence),
// spins (bounded) on the packets of the other ranks and writes the final output, so one launch
// per rank is the whole distributed decode step.
//
// Reference counterparts: kernels/nvidia/flash_decode.py:129-239 (split kernel), :307-360 /
// :392-449 (split merges), :481-532 (inter-rank merge), :586-760 (persistent fused variant, grid
// hard-wired to 132 SMs), layers/nvidia/sp_flash_decode_layer.py:78-184 (3 kernels + an allgather).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include <cstdlib>
#include <mutex>
#include <string>

#include "../device/ll.cuh"
#include "../device/ptx.cuh"
#include "../device/signal.cuh"
#include "../include/tdist.h"
#include "../include/tdist_noalloc.h"
#include "../runtime/host_common.h"

namespace tdist {

constexpr int kKernelDecode = 4;
constexpr int kDecodeWarps = 4;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kTok = 16;  // tokens per warp step

struct DecodeParams {
    const void* q;          // [B, Hq, D]
    const void* k_cache;    // [blocks, page, Hkv, D]
    const void* v_cache;
    const int* block_table; // [B, max_blocks]
    const int* kv_lens;     // [B] (this rank's shard)
    float* partial;         // [B, Hq, splits, D + 2]
    unsigned* counters;     // [B * Hkv], zero between calls
    void* out;              // mode 0/2: T [B, Hq, D]; mode 1: float [B, Hq, D + 1]
    char* ll_peer[kMaxRanks];  // SP: this call's parity of every rank: [world][B*Hq*(D+2)/2] packets
    int B, Hq, Hkv, page_size, max_blocks, splits;
    int cluster_merge;      // 1: the splits of a (batch, kv head) are one thread-block cluster and merge through shared memory
    long long stride_block, stride_token, stride_head;  // cache strides in elements
    float scale, soft_cap;
    int mode;               // 0 final, 1 O||LSE (fp32), 2 sequence-parallel
    int world, rank;
    int push_only;          // SP: stop after the exchange's send half (ranks emulated one at a time)
    unsigned epoch;
    unsigned* epoch_ptr;    // SP, optional: device-resident call number (see TdistDecodeArgs)
    unsigned* epoch_done;
    char* ll_peer_alt[kMaxRanks];
    char* ll_mc;            // SP, optional: multicast alias of this call's parity of the gather buffer: one
    char* ll_mc_alt;        // multimem.st per packet reaches every rank (alt = odd call numbers, device-resident epoch)
    WaitCtx wctx;
};

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t (&r)[4]) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) { return pack_bf16x2(lo, hi); }
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) { return pack_f16x2(lo, hi); }
template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

// Shared-memory tiles hold rows of D elements; the 16-byte chunk index is XOR-ed with the row
// so that ldmatrix (8 rows x 16 bytes) and cp.async (one row per half-warp) are conflict-free.
template <int D>
__device__ __forceinline__ uint32_t tile_off(int row, int chunk) {
    return static_cast<uint32_t>(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

// Ring depth: D <= 64 -> 4 stages (68 KB, 3 CTAs/SM); D = 128 -> 3 stages (100 KB, 2 CTAs/SM);
// D = 256 -> 2 stages (136 KB, 1 CTA/SM).
__host__ __device__ constexpr int decode_stages(int d) { return d <= 64 ? 4 : (d <= 128 ? 3 : 2); }

template <typename T, int D>
__global__ void __launch_bounds__(kDecodeThreads, (D <= 128 ? 2 : 1)) flash_decode_kernel(const DecodeParams p) {
    constexpr int CH = D / 8;                      // 16-byte chunks per row
    constexpr int TILE = kTok * D * 2;             // bytes of one K or V block
    constexpr int NS = decode_stages(D);           // cp.async ring depth per warp
    constexpr int KS = D / 16;                     // k-steps of QK^T
    constexpr int NT = D / 8;                      // n-tiles of PV
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* q_s = smem;                                            // 16 x D
    uint8_t* ring = smem + kTok * D * 2;                            // [warps][NS][K|V]
    __shared__ float m_s[kDecodeWarps][16], l_s[kDecodeWarps][16];
    __shared__ int last_s;

    const int tid = static_cast<int>(threadIdx.x);
    const int warp = tid >> 5, lane = tid & 31;
    const int split = static_cast<int>(blockIdx.x) % p.splits;
    const int kvh = (static_cast<int>(blockIdx.x) / p.splits) % p.Hkv;
    const int b = static_cast<int>(blockIdx.x) / (p.splits * p.Hkv);
    const int G = p.Hq / p.Hkv;
    const T* q = static_cast<const T*>(p.q) + (static_cast<size_t>(b) * p.Hq + static_cast<size_t>(kvh) * G) * D;
    const T* kc = static_cast<const T*>(p.k_cache) + static_cast<size_t>(kvh) * p.stride_head;
    const T* vc = static_cast<const T*>(p.v_cache) + static_cast<size_t>(kvh) * p.stride_head;
    const int* table = p.block_table + static_cast<size_t>(b) * p.max_blocks;

    // ---- Q tile into shared memory (rows >= G are zero)
    for (int c = tid; c < 16 * CH; c += kDecodeThreads) {
        const int row = c / CH, ch = c % CH;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < G) v = *reinterpret_cast<const uint4*>(q + static_cast<size_t>(row) * D + ch * 8);
        *reinterpret_cast<uint4*>(q_s + tile_off<D>(row, ch)) = v;
    }
    __syncthreads();

    // ---- this CTA's KV range, in 16-token blocks dealt round-robin to the warps
    const int kv_len = p.kv_lens[b];
    const int nblk_total = (kv_len + kTok - 1) / kTok;
    const int blk_per_split = (nblk_total + p.splits - 1) / p.splits;
    const int blk0 = split * blk_per_split;
    const int blk1 = min(nblk_total, blk0 + blk_per_split);
    const int my_blocks = (blk1 - blk0 - warp + kDecodeWarps - 1) / kDecodeWarps;  // may be <= 0

    uint8_t* my_ring = ring + static_cast<size_t>(warp) * NS * 2 * TILE;
    // Page-table lookup for block i of this warp: lane r < 16 resolves token r. It is issued one
    // block ahead of the copies that need it, so its latency hides behind a block's worth of math
    // instead of stalling the (in-order) warp right before every batch of cp.async.
    auto lookup = [&](int i) -> long long {
        long long base = -1;
        if (i < my_blocks && lane < kTok) {
            const int t = (blk0 + warp + i * kDecodeWarps) * kTok + lane;
            if (t < kv_len) {
                const int page = table[t / p.page_size];
                base = static_cast<long long>(page) * p.stride_block + static_cast<long long>(t % p.page_size) * p.stride_token;
            }
        }
        return base;
    };
    auto issue = [&](int i, long long base) {  // i-th block of this warp -> ring slot i % NS
        uint8_t* ks = my_ring + static_cast<size_t>(i % NS) * 2 * TILE;
        uint8_t* vs = ks + TILE;
#pragma unroll
        for (int j = 0; j < (kTok * CH) / 32; ++j) {
            const int c = j * 32 + lane;
            const int row = c / CH, ch = c % CH;
            const long long rb = __shfl_sync(0xffffffffu, base, row);
            const int nbytes = rb >= 0 ? 16 : 0;  // rows past the end are zero-filled
            const long long off = (rb >= 0 ? rb : 0) + ch * 8;
            cp_async16(smem_u32(ks + tile_off<D>(row, ch)), kc + off, nbytes);
            cp_async16(smem_u32(vs + tile_off<D>(row, ch)), vc + off, nbytes);
        }
    };

    float o[NT][4];
#pragma unroll
    for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F}, l_run[2] = {0.f, 0.f};
    const float sl2 = p.scale * 1.4426950408889634f;

    long long base_next = lookup(0);
    for (int i = 0; i < NS - 1; ++i) {
        const long long base = base_next;
        base_next = lookup(i + 1);
        if (i < my_blocks) issue(i, base);
        cp_async_commit();
    }
    for (int i = 0; i < my_blocks; ++i) {
        if (i + NS - 1 < my_blocks) {
            const long long base = base_next;
            base_next = lookup(i + NS);
            issue(i + NS - 1, base);
        }
        cp_async_commit();
        cp_async_wait<NS - 1>();
        __syncwarp();
        const uint8_t* ks = my_ring + static_cast<size_t>(i % NS) * 2 * TILE;
        const uint8_t* vs = ks + TILE;
        const int tok0 = (blk0 + warp + i * kDecodeWarps) * kTok;

        // S = Q K^T for 16 tokens: two n-tiles of 8
        float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int k = 0; k < KS; ++k) {
            uint32_t a[4], bf[4];
            ldmatrix_x4(smem_u32(q_s + tile_off<D>((lane & 7) + ((lane >> 3) & 1) * 8, 2 * k + (lane >> 4))), a);
            ldmatrix_x4(smem_u32(ks + tile_off<D>((lane & 7) + (lane >> 4) * 8, 2 * k + ((lane >> 3) & 1))), bf);
            mma16816<T>(s[0], a, bf[0], bf[1]);
            mma16816<T>(s[1], a, bf[2], bf[3]);
        }
        // scale, soft cap, mask, online softmax (rows lane/4 and lane/4 + 8)
        float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int tok = tok0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                float v = s[nt][e];
                if (p.soft_cap > 0.f) v = p.soft_cap * tanhf(v * p.scale / p.soft_cap) * 1.4426950408889634f;
                else v *= sl2;
                v = tok < kv_len ? v : -CUDART_INF_F;
                s[nt][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        float alpha[2], m_use[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            m_use[r] = m_new == -CUDART_INF_F ? 0.f : m_new;
            alpha[r] = exp2f(m_run[r] - m_use[r]);
            m_run[r] = m_new;
        }
        float rs[2] = {0.f, 0.f};
        uint32_t pa[4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const float p0 = exp2f(s[nt][0] - m_use[0]), p1 = exp2f(s[nt][1] - m_use[0]);
            const float p2 = exp2f(s[nt][2] - m_use[1]), p3 = exp2f(s[nt][3] - m_use[1]);
            rs[0] += p0 + p1;
            rs[1] += p2 + p3;
            pa[nt * 2 + 0] = pack2<T>(p0, p1);
            pa[nt * 2 + 1] = pack2<T>(p2, p3);
        }
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
            rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
            l_run[r] = l_run[r] * alpha[r] + rs[r];
        }
        // O = O * alpha + P V
#pragma unroll
        for (int j = 0; j < NT / 2; ++j) {
            uint32_t bf[4];
            ldmatrix_x4_trans(smem_u32(vs + tile_off<D>((lane & 7) + ((lane >> 3) & 1) * 8, 2 * j + (lane >> 4))), bf);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float (&acc)[4] = o[2 * j + h];
                acc[0] *= alpha[0];
                acc[1] *= alpha[0];
                acc[2] *= alpha[1];
                acc[3] *= alpha[1];
                mma16816<T>(acc, pa, bf[2 * h], bf[2 * h + 1]);
            }
        }
        __syncwarp();
    }
    cp_async_wait<0>();
    __syncthreads();

    // ---- merge the warps through shared memory (the ring is free now)
    float* o_s = reinterpret_cast<float*>(ring);  // [warps][16][D]
    {
        const int r0 = lane >> 2;
        if ((lane & 3) == 0) {
            m_s[warp][r0] = m_run[0];
            m_s[warp][r0 + 8] = m_run[1];
            l_s[warp][r0] = l_run[0];
            l_s[warp][r0 + 8] = l_run[1];
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const int col = nt * 8 + (lane & 3) * 2;
            float* base = o_s + (static_cast<size_t>(warp) * 16) * D;
            *reinterpret_cast<float2*>(base + static_cast<size_t>(r0) * D + col) = make_float2(o[nt][0], o[nt][1]);
            *reinterpret_cast<float2*>(base + static_cast<size_t>(r0 + 8) * D + col) = make_float2(o[nt][2], o[nt][3]);
        }
    }
    __syncthreads();
    const int W2 = D + 2;  // floats per head in the workspace and in the gather buffers: O, LSE, pad
    // cluster merge: the partials of all splits land behind the ring of the cluster's first CTA
    float* part_s = reinterpret_cast<float*>(ring + static_cast<size_t>(kDecodeWarps) * NS * 2 * TILE);
    const uint32_t part_leader = p.cluster_merge ? mapa_u32(smem_u32(part_s), 0) : 0u;
    for (int idx = tid; idx < G * D; idx += kDecodeThreads) {
        const int g = idx / D, c = idx % D;
        float mm = -CUDART_INF_F;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) mm = fmaxf(mm, m_s[w][g]);
        float l = 0.f, acc = 0.f;
        const float mu = mm == -CUDART_INF_F ? 0.f : mm;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) {
            const float f = exp2f(m_s[w][g] - mu);
            l += l_s[w][g] * f;
            acc += o_s[(static_cast<size_t>(w) * 16 + g) * D + c] * f;
        }
        const float val = l > 0.f ? acc / l : 0.f;
        const float lse = l > 0.f ? mm * 0.6931471805599453f + logf(l) : -CUDART_INF_F;
        if (p.cluster_merge) {
            // straight into the leader CTA's shared memory: [G][splits][W2], the layout the merge below reads
            const uint32_t at = part_leader + static_cast<uint32_t>(((g * p.splits + split) * W2 + c) * 4);
            st_shared_cluster_f32(at, val);
            if (c == 0) st_shared_cluster_f32(at + D * 4, lse);
        } else {
            float* dst = p.partial + ((static_cast<size_t>(b) * p.Hq + kvh * G + g) * p.splits + split) * W2;
            dst[c] = val;
            if (c == 0) dst[D] = lse;
        }
    }

    if (p.cluster_merge) {
        // ---- the splits of this (batch, kv head) are one cluster: its first CTA merges them out of its own shared
        // memory once every CTA's stores have arrived (release / acquire at cluster scope); no trip through global
        // memory, no counter
        cluster_arrive();
        cluster_wait();
        if (split != 0) return;
    } else {
        // ---- the last CTA of this (batch, kv head) merges the splits
        __threadfence();
        __syncthreads();
        if (tid == 0) {
            const unsigned old = atomicAdd(p.counters + b * p.Hkv + kvh, 1u);
            last_s = (old == static_cast<unsigned>(p.splits - 1));
            if (last_s) p.counters[b * p.Hkv + kvh] = 0;
        }
        __syncthreads();
        if (!last_s) return;
        __threadfence();
    }

    // A warp per query head: lanes first turn the per-split LSEs into normalised weights (kept in
    // shared memory), then every lane merges 4 output columns with independent 16-byte loads.
    float* merged = o_s;                       // [G][W2] merged O || LSE of this rank (SP mode)
    float* w_s = o_s + 16 * W2;                // [warps][256] split weights
    for (int g = warp; g < G; g += kDecodeWarps) {
        const size_t head = static_cast<size_t>(b) * p.Hq + kvh * G + g;
        const float* src = p.cluster_merge ? part_s + static_cast<size_t>(g) * p.splits * W2 : p.partial + head * p.splits * W2;
        float mm = -CUDART_INF_F;
        for (int sidx = lane; sidx < p.splits; sidx += 32) mm = fmaxf(mm, src[sidx * W2 + D]);
#pragma unroll
        for (int o2 = 16; o2; o2 >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, o2));
        const float mu = mm == -CUDART_INF_F ? 0.f : mm;
        float wsum = 0.f;
        for (int sidx = lane; sidx < p.splits; sidx += 32) {
            const float f = __expf(src[sidx * W2 + D] - mu);
            w_s[warp * 256 + sidx] = f;
            wsum += f;
        }
#pragma unroll
        for (int o2 = 16; o2; o2 >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o2);
        __syncwarp();
        const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
        const float lse = wsum > 0.f ? mm + logf(wsum) : -CUDART_INF_F;
        for (int c = lane * 4; c < D; c += 128) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
            for (int sidx = 0; sidx < p.splits; ++sidx) {
                // rows of the workspace are D + 2 floats: 8-byte aligned, so two float2 loads
                const float2 lo = *reinterpret_cast<const float2*>(src + sidx * W2 + c);
                const float2 hi = *reinterpret_cast<const float2*>(src + sidx * W2 + c + 2);
                const float f = w_s[warp * 256 + sidx];
                acc.x += f * lo.x;
                acc.y += f * lo.y;
                acc.z += f * hi.x;
                acc.w += f * hi.y;
            }
            acc.x *= inv;
            acc.y *= inv;
            acc.z *= inv;
            acc.w *= inv;
            if (p.mode == 0) {
                T* dst = static_cast<T*>(p.out) + head * D + c;
                *reinterpret_cast<uint2*>(dst) = make_uint2(pack2<T>(acc.x, acc.y), pack2<T>(acc.z, acc.w));
            } else if (p.mode == 1) {
                float* dst = static_cast<float*>(p.out) + head * (D + 1) + c;  // rows of D + 1 floats: scalar stores
                dst[0] = acc.x;
                dst[1] = acc.y;
                dst[2] = acc.z;
                dst[3] = acc.w;
            } else {
                *reinterpret_cast<float2*>(merged + g * W2 + c) = make_float2(acc.x, acc.y);
                *reinterpret_cast<float2*>(merged + g * W2 + c + 2) = make_float2(acc.z, acc.w);
            }
        }
        if (lane == 0) {
            if (p.mode == 1) static_cast<float*>(p.out)[head * (D + 1) + D] = lse;
            if (p.mode == 2) {
                merged[g * W2 + D] = lse;
                merged[g * W2 + D + 1] = 0.f;
            }
        }
        __syncwarp();
    }
    if (p.mode != 2) return;
    __syncthreads();

    // ---- sequence-parallel: exchange O||LSE of these G heads with every rank as LL packets
    // Call number and buffer parity: from the arguments, or (replayable launches) from device memory.
    unsigned epoch = p.epoch;
    char* const* ll = p.ll_peer;
    if (p.epoch_ptr != nullptr) {
        epoch = *reinterpret_cast<volatile unsigned*>(p.epoch_ptr) + 1u;
        ll = (epoch & 1u) ? p.ll_peer_alt : p.ll_peer;
    }
    const int npk = G * W2 / 2;                                        // packets of this head group
    const size_t pk0 = (static_cast<size_t>(b) * p.Hq + kvh * G) * W2 / 2;  // first packet in a rank slot
    const size_t slot = static_cast<size_t>(p.B) * p.Hq * W2 / 2;      // packets per source rank
    char* mc = p.ll_mc;
    if (p.epoch_ptr != nullptr && (epoch & 1u)) mc = p.ll_mc_alt;
    for (int i = tid; i < npk; i += kDecodeThreads) {
        const uint64_t payload = *reinterpret_cast<const uint64_t*>(merged + 2 * i);
        if (mc != nullptr) {
            // one store into the NVSwitch multicast alias lands in every rank's buffer (this rank's included). Each
            // 8-byte half of the packet carries its own flag copy, so a packet split on the way is still detected.
            ll_store_multimem(mc + (static_cast<size_t>(p.rank) * slot + pk0 + i) * 16, payload, epoch);
            continue;
        }
        for (int r = 0; r < p.world; ++r) {
            int peer = p.rank + r;
            if (peer >= p.world) peer -= p.world;
            ll_store(ll[peer] + (static_cast<size_t>(p.rank) * slot + pk0 + i) * 16, payload, epoch);
        }
    }
    if (p.push_only) return;
    // gather: lse of every (source, head) first, then the weighted sum
    float* lse_s = reinterpret_cast<float*>(q_s);  // [world][G]  (Q tile is dead)
    const char* mine = ll[p.rank];
    for (int idx = tid; idx < p.world * G; idx += kDecodeThreads) {
        const int r = idx / G, g = idx % G;
        uint64_t v;
        ll_load(mine + (static_cast<size_t>(r) * slot + pk0 + (g * W2 + D) / 2) * 16, epoch, &v, p.wctx, r, g);
        lse_s[idx] = __uint_as_float(static_cast<uint32_t>(v));
    }
    __syncthreads();
    for (int i = tid; i < G * D / 2; i += kDecodeThreads) {
        const int g = i / (D / 2), c = (i % (D / 2)) * 2;
        float mm = -CUDART_INF_F;
        for (int r = 0; r < p.world; ++r) mm = fmaxf(mm, lse_s[r * G + g]);
        const float mu = mm == -CUDART_INF_F ? 0.f : mm;
        float wsum = 0.f, a0 = 0.f, a1 = 0.f;
        for (int r = 0; r < p.world; ++r) {
            const float f = __expf(lse_s[r * G + g] - mu);
            uint64_t v;
            ll_load(mine + (static_cast<size_t>(r) * slot + pk0 + (g * W2 + c) / 2) * 16, epoch, &v, p.wctx, r, i);
            wsum += f;
            a0 += f * __uint_as_float(static_cast<uint32_t>(v));
            a1 += f * __uint_as_float(static_cast<uint32_t>(v >> 32));
        }
        const float inv = wsum > 0.f ? 1.f / wsum : 0.f;
        T* dst = static_cast<T*>(p.out) + (static_cast<size_t>(b) * p.Hq + kvh * G + g) * D + c;
        *reinterpret_cast<uint32_t*>(dst) = pack2<T>(a0 * inv, a1 * inv);
    }
    if (p.epoch_ptr != nullptr) {
        // The last of the B * Hkv exchanging CTAs records the call as done. Every one of them read the number
        // before it got here, and CTAs that merge no head group never read it.
        __syncthreads();
        if (tid == 0) {
            const unsigned old = atomicAdd(p.epoch_done, 1u);
            if (old == static_cast<unsigned>(p.B * p.Hkv - 1)) {
                *p.epoch_done = 0;
                __threadfence();
                *reinterpret_cast<volatile unsigned*>(p.epoch_ptr) = epoch;
            }
        }
    }
}

// Merge per-rank partials [R, B, Hq, D + 1] (O || LSE, fp32) into [B, Hq, D]; ranks whose LSE is
// -inf (no keys) drop out. (reference flash_decode.py:481-532)
template <typename T>
__global__ void lse_combine_kernel(const float* parts, int R, int heads, int D, T* out) {
    const int h = static_cast<int>(blockIdx.x);
    float mm = -CUDART_INF_F;
    for (int r = 0; r < R; ++r) mm = fmaxf(mm, parts[(static_cast<size_t>(r) * heads + h) * (D + 1) + D]);
    const float mu = mm == -CUDART_INF_F ? 0.f : mm;
    for (int c = threadIdx.x; c < D; c += blockDim.x) {
        float wsum = 0.f, acc = 0.f;
        for (int r = 0; r < R; ++r) {
            const float* src = parts + (static_cast<size_t>(r) * heads + h) * (D + 1);
            const float f = __expf(src[D] - mu);
            wsum += f;
            acc += f * src[c];
        }
        out[static_cast<size_t>(h) * D + c] = from_float<T>(wsum > 0.f ? acc / wsum : 0.f);
    }
}

}  // namespace tdist

using namespace tdist;
using tdist_host::fail;

// Largest cluster (splits of one (batch, kv head)) the merge through shared memory is used for, and the bytes it may add
// to a CTA's shared memory. Above either limit the splits meet in global memory (workspace + arrival counter).
// Eight is the portable cluster size; 16-CTA clusters were measured and dropped: with 133 KB of shared memory per CTA
// only some of them are resident at once (batch 1, 8 kv heads, 16384 keys, 16 splits: 37.1 us against 22.6 us through
// global memory). Up to eight splits the cluster form is 5-10 % faster (4096 keys: 14.4 / 20.6 us against 15.4 / 22.6 us
// with 8 / 4 splits).
constexpr int kClusterMergeMaxSplits = 8;
constexpr int kClusterMergeMaxBytes = 48 * 1024;

template <typename T, int D>
static int launch_decode(DecodeParams& p, cudaStream_t stream) {
    constexpr int NS = decode_stages(D);
    constexpr int smem = kTok * D * 2 + kDecodeWarps * NS * 2 * kTok * D * 2;
    static_assert(smem >= kDecodeWarps * 16 * D * 4, "the warp-merge buffer reuses the ring");
    static bool done[64] = {};
    static std::mutex setup_lock;
    static const bool cluster_enabled = [] {
        const char* e = getenv("TDIST_DECODE_CLUSTER_MERGE");
        return e == nullptr || atoi(e) != 0;
    }();
    int dev = 0;
    TDIST_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TDIST_EINVAL, "decode: device ordinal out of range");
    {
        std::lock_guard<std::mutex> guard(setup_lock);
        if (!done[dev]) {
            TDIST_CUDA_OK(cudaFuncSetAttribute(flash_decode_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem + kClusterMergeMaxBytes));
            done[dev] = true;
        }
    }
    const int G = p.Hq / p.Hkv;
    const int part_bytes = G * p.splits * (D + 2) * static_cast<int>(sizeof(float));
    const bool cluster = cluster_enabled && p.splits >= 2 && p.splits <= kClusterMergeMaxSplits && part_bytes <= kClusterMergeMaxBytes;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(static_cast<unsigned>(p.B * p.Hkv * p.splits));
    cfg.blockDim = dim3(kDecodeThreads);
    cfg.stream = stream;
    cfg.dynamicSmemBytes = cluster ? smem + part_bytes : smem;
    cudaLaunchAttribute attr[1];
    if (cluster) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = static_cast<unsigned>(p.splits);
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    p.cluster_merge = cluster ? 1 : 0;
    TDIST_CUDA_OK(cudaLaunchKernelEx(&cfg, flash_decode_kernel<T, D>, p));
    return 0;
}

static int flash_decode_impl(const TdistDecodeArgs* a) {
    if (a->B < 1 || a->Hq < 1 || a->Hkv < 1 || a->Hq % a->Hkv) return fail(TDIST_EINVAL, "decode: bad head counts");
    if (a->Hq / a->Hkv > 16) return fail(TDIST_ELIMIT, "decode: at most 16 query heads per kv head");
    if (a->splits < 1 || a->splits > 256) return fail(TDIST_EINVAL, "decode: splits must be in [1, 256]");
    if (a->head_dim != 64 && a->head_dim != 128 && a->head_dim != 256) return fail(TDIST_EINVAL, "decode: head_dim must be 64, 128 or 256");
    if (a->stride_token % 8 || a->stride_block % 8 || a->stride_head % 8) return fail(TDIST_EINVAL, "decode: cache strides must be multiples of 8 elements");
    if (a->mode < 0 || a->mode > 2) return fail(TDIST_EINVAL, "decode: bad mode");
    if (a->page_size < 1 || a->max_blocks < 1) return fail(TDIST_EINVAL, "decode: page_size and max_blocks must be at least 1");
    if (static_cast<long long>(a->B) * a->Hkv * a->splits > 0x7fffffffLL) return fail(TDIST_ELIMIT, "decode: B * Hkv * splits exceeds the grid limit");
    DecodeParams p;
    memset(&p, 0, sizeof(p));
    p.q = a->q;
    p.k_cache = a->k_cache;
    p.v_cache = a->v_cache;
    p.block_table = static_cast<const int*>(a->block_table);
    p.kv_lens = static_cast<const int*>(a->kv_lens);
    p.partial = static_cast<float*>(a->partial);
    p.counters = static_cast<unsigned*>(a->counters);
    p.out = a->out;
    p.B = a->B;
    p.Hq = a->Hq;
    p.Hkv = a->Hkv;
    p.page_size = a->page_size;
    p.max_blocks = a->max_blocks;
    p.splits = a->splits;
    p.stride_block = a->stride_block;
    p.stride_token = a->stride_token;
    p.stride_head = a->stride_head;
    p.scale = a->scale;
    p.soft_cap = a->soft_cap;
    p.mode = a->mode;
    p.world = a->world;
    p.rank = a->rank;
    p.epoch = a->epoch;
    p.push_only = a->push_only;
    p.wctx.status = static_cast<Status*>(a->status);
    p.wctx.timeout_ns = a->timeout_ns;
    p.wctx.kernel_id = kKernelDecode;
    p.wctx.rank = a->rank;
    if (!p.q || !p.k_cache || !p.v_cache || !p.block_table || !p.kv_lens || !p.partial || !p.counters || !p.out)
        return fail(TDIST_EINVAL, "decode: null pointer");
    if (a->mode == 2) {
        if (a->world < 1 || a->world > TDIST_MAX_RANKS || a->rank < 0 || a->rank >= a->world) return fail(TDIST_EINVAL, "decode: world/rank out of range");
        if (a->epoch == 0 && a->epoch_ptr == nullptr) return fail(TDIST_EINVAL, "decode: the epoch of a sequence-parallel call must be non-zero");
        if (a->epoch_ptr != nullptr && a->epoch_done == nullptr) return fail(TDIST_EINVAL, "decode: epoch_ptr needs epoch_done");
        p.epoch_ptr = static_cast<unsigned*>(a->epoch_ptr);
        p.ll_mc = a->world > 1 ? static_cast<char*>(a->ll_mc) : nullptr;
        p.ll_mc_alt = a->world > 1 ? static_cast<char*>(a->ll_mc_alt) : nullptr;
        if (a->epoch_ptr != nullptr && (p.ll_mc != nullptr) != (p.ll_mc_alt != nullptr))
            return fail(TDIST_EINVAL, "decode: a device-resident call number needs both multicast aliases or none");
        p.epoch_done = static_cast<unsigned*>(a->epoch_done);
        for (int r = 0; r < a->world && a->epoch_ptr != nullptr; ++r) {
            p.ll_peer_alt[r] = static_cast<char*>(a->ll_peer_alt[r]);
            if (!p.ll_peer_alt[r]) return fail(TDIST_EINVAL, "decode: null gather buffer (odd call numbers)");
        }
        for (int r = 0; r < a->world; ++r) {
            p.ll_peer[r] = static_cast<char*>(a->ll_peer[r]);
            if (!p.ll_peer[r]) return fail(TDIST_EINVAL, "decode: null gather buffer");
        }
    }
    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
#define TDIST_DECODE_CASE(TT, DD) return launch_decode<TT, DD>(p, stream)
    if (a->dtype == TDIST_BF16) {
        if (a->head_dim == 64) TDIST_DECODE_CASE(__nv_bfloat16, 64);
        if (a->head_dim == 128) TDIST_DECODE_CASE(__nv_bfloat16, 128);
        TDIST_DECODE_CASE(__nv_bfloat16, 256);
    } else if (a->dtype == TDIST_F16) {
        if (a->head_dim == 64) TDIST_DECODE_CASE(__half, 64);
        if (a->head_dim == 128) TDIST_DECODE_CASE(__half, 128);
        TDIST_DECODE_CASE(__half, 256);
    }
#undef TDIST_DECODE_CASE
    return fail(TDIST_EINVAL, "decode: dtype must be bf16 or fp16");
}

extern "C" int tdist_flash_decode(const TdistDecodeArgs* a) { return flash_decode_impl(a); }

// ---------------------------------------------------------------------------------------------
// Allocation-free variant (contract in ../include/tdist_noalloc.h): the split-merge workspace and
// the arrival counters live in this array instead of caller-provided buffers.
// Layout: [0, counters_bytes) uint32 counters, then fp32 partials. In host code the name below is
// only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_decode_static_scratch[TDIST_DECODE_STATIC_SCRATCH_BYTES];

extern "C" int tdist_flash_decode_static(const TdistDecodeArgs* a) {
    if (a == nullptr) return fail(TDIST_EINVAL, "decode(static): null args");
    if (a->mode != 0 && a->mode != 1)
        return fail(TDIST_EINVAL, "decode(static): only modes 0 and 1 (the sequence-parallel mode needs caller-owned symmetric memory)");
    if (a->B < 1 || a->Hq < 1 || a->Hkv < 1 || a->splits < 1 || a->head_dim < 1)
        return fail(TDIST_EINVAL, "decode(static): bad sizes");
    // the cheap range checks of the regular path come first: nothing is enqueued for a call that will be refused,
    // and the size product below cannot overflow
    if (a->splits > 256) return fail(TDIST_EINVAL, "decode: splits must be in [1, 256]");
    if (a->head_dim != 64 && a->head_dim != 128 && a->head_dim != 256) return fail(TDIST_EINVAL, "decode: head_dim must be 64, 128 or 256");
    if (a->Hq % a->Hkv || a->Hq / a->Hkv > 16) return fail(TDIST_EINVAL, "decode: bad head counts");
    if (a->page_size < 1 || a->max_blocks < 1) return fail(TDIST_EINVAL, "decode: page_size and max_blocks must be at least 1");
    if (static_cast<long long>(a->B) * a->Hq > (1LL << 24)) return fail(TDIST_ELIMIT, "decode(static): B * Hq beyond the built-in scratch");
    const size_t counters_bytes = (static_cast<size_t>(a->B) * a->Hkv * sizeof(unsigned) + 255) / 256 * 256;
    const size_t partial_bytes = static_cast<size_t>(a->B) * a->Hq * a->splits * (a->head_dim + 2) * sizeof(float);
    if (counters_bytes + partial_bytes > TDIST_DECODE_STATIC_SCRATCH_BYTES)
        return fail(TDIST_ELIMIT, "decode(static): B*Hq*splits*(head_dim+2)*4 + counters = " +
                                      std::to_string(counters_bytes + partial_bytes) + " bytes exceeds the built-in scratch of " +
                                      std::to_string(TDIST_DECODE_STATIC_SCRATCH_BYTES) + " bytes; use fewer splits or tdist_flash_decode");
    // once per device, with that device current: resolve the array's device address
    static unsigned char* scratch_of_device[64] = {};
    static std::mutex setup_lock;   // two host threads may make the first call on one device at once
    int dev = 0;
    TDIST_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail(TDIST_EINVAL, "decode(static): device ordinal out of range");
    unsigned char* base = nullptr;
    {
        std::lock_guard<std::mutex> guard(setup_lock);
        if (scratch_of_device[dev] == nullptr) {
            unsigned char* ptr = nullptr;
            TDIST_CUDA_OK(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_decode_static_scratch));
            if (ptr == nullptr) return fail(TDIST_EDRIVER, "decode(static): cudaGetSymbolAddress returned a null address");
            scratch_of_device[dev] = ptr;
        }
        base = scratch_of_device[dev];
    }
    // the counters must start at zero whatever the previous call left behind
    TDIST_CUDA_OK(cudaMemsetAsync(base, 0, counters_bytes, static_cast<cudaStream_t>(a->stream)));
    TdistDecodeArgs b = *a;
    b.counters = base;
    b.partial = base + counters_bytes;
    return flash_decode_impl(&b);
}

extern "C" int tdist_lse_combine(const void* parts, int ranks, int heads, int head_dim, void* out, int dtype, void* stream) {
    if (ranks < 1 || heads < 1 || head_dim < 1) return fail(TDIST_EINVAL, "lse_combine: bad sizes");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int threads = head_dim >= 256 ? 256 : (head_dim >= 128 ? 128 : 64);
    if (dtype == TDIST_BF16)
        lse_combine_kernel<__nv_bfloat16><<<heads, threads, 0, s>>>(static_cast<const float*>(parts), ranks, heads, head_dim, static_cast<__nv_bfloat16*>(out));
    else if (dtype == TDIST_F16)
        lse_combine_kernel<__half><<<heads, threads, 0, s>>>(static_cast<const float*>(parts), ranks, heads, head_dim, static_cast<__half*>(out));
    else
        return fail(TDIST_EINVAL, "lse_combine: dtype must be bf16 or fp16");
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}
