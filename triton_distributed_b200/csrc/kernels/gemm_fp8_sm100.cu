// Block-scaled fp8 (e4m3) GEMM on tcgen05, plain and fused AllGather-GEMM.
//
//   C[m, n] = sum over 128-wide K blocks kb of  SA[m, kb] * SB[n / 128, kb] * (A_kb[m, :] . B_kb[n, :])
//
// A [M, K] and B [N, K] are e4m3 (K contiguous), SA [M, K/128] fp32 holds one scale per row per K block
// (1 x 128), SB [N/128, K/128] fp32 one scale per 128 x 128 block of B, C is bf16. These fp32 scales are
// not what the hardware's block-scaled MMA kinds take (those want ue8m0 per 32 values), so every
// 128-wide K block is multiplied unscaled into a fresh TMEM accumulator (tcgen05.mma kind::f8f6f4,
// M128 N256 K32 x 4) and then *promoted*: eight warps read the block's partial sums out of TMEM
// (tcgen05.ld) and fold them into fp32 register accumulators with the block's scale. Two TMEM buffers
// let the tensor core work on block kb+1 while block kb is promoted.
//
// Warps (320 threads): 0 = TMA producer, 1 = MMA issuer / TMEM owner, 2..9 = promotion + epilogue.
// Promotion warp w reads TMEM lanes 32*(w%4).., i.e. tile rows, and columns 128*((w-2)/4)..: one thread
// owns one row x 128 columns = 128 fp32 accumulators, folded with packed fma.rn.f32x2.
//
// One CTA per 128 x 256 tile, 4 TMA stages of 48 KB. Measured on B200 (m8192 n6144 k12288): 1.8-1.9 PFLOP/s,
// 1.1-1.2x the cuBLAS bf16 rate and about half the dense fp8 rate. The limit is the round trip per K block between
// the MMA issuer and the promotion warps: TMEM (512 columns) holds only two 128 x 256 fp32 accumulators,
// so at most two K blocks of MMA work (~0.5 us) are in flight against a loop of MMA completion latency +
// TMEM read + barrier hand-over of about 1.3 us. A CTA-pair tiling (cta_group::2, 256 x 256) was built and
// measured at half this speed, because the same round trip then crosses two SMs; it was removed.
//
// AG mode is the fp8 twin of gemm_sm100.cu's: pusher CTAs of the same grid stream this rank's rows
// AND their scales into every peer's workspace, one flag per 128-row block.
//
// The reference runs its fp8 GEMMs as plain `tl.dot` on fp8 inputs without block scales
// (reference kernels/nvidia/allgather_group_gemm.py:348); the 1x128 / 128x128 scale layout is the
// DeepSeek-V3 one its tutorial 04 quantises to.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstring>
#include <string>

#include "../device/ptx.cuh"
#include "../device/signal.cuh"
#include "../include/tdist.h"
#include "../runtime/host_common.h"

namespace tdist {
namespace fp8 {

constexpr int BM = 128, BN = 256, BK = 128;   // BK in elements = bytes
constexpr int UMMA_K = 32;
constexpr int A_BYTES = BM * BK;                               // 16 KB
constexpr int EPI_COLS = 64, EPI_BYTES = BM * EPI_COLS * 2;   // 16 KB
constexpr int PIPE_BYTES = 192 * 1024;
constexpr int SMEM_TILES = PIPE_BYTES + 2 * EPI_BYTES;        // 224 KB
constexpr int SMEM_BYTES = SMEM_TILES + 1024 + 256;
constexpr int THREADS = 320;
constexpr int PROMO_WARPS = 8;
constexpr int TMEM_COLS = 512;
constexpr int MAX_STAGES = 4;
constexpr int kKernelGemmFp8 = 7;
constexpr int PUSH_CHUNK = 32768, PUSH_STAGES = 6, PUSH_AHEAD = 4;
static_assert(PUSH_STAGES * PUSH_CHUNK <= SMEM_TILES, "pusher buffers must fit");

constexpr int B_BYTES = BN * BK;                 // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;   // 48 KB
constexpr int STAGES = PIPE_BYTES / STAGE_BYTES; // 4

struct Params {
    CUtensorMap tm_a;       // {K, m_per_rank, world} over A or the gather workspace, box {128, 128, 1}
    CUtensorMap tm_a_own;   // AG: this rank's shard {K, m_per_rank, 1}
    CUtensorMap tm_b;       // {K, N, 1}, box {128, 256, 1}
    CUtensorMap tm_c;       // {N, m_per_rank, world} bf16, box {64, 128, 1}
    const float* sa;        // [world * m_per_rank, KB] (AG: the workspace scales)
    const float* sa_own;    // AG: [m_per_rank, KB]
    const float* sb;        // [ceil(N / 128), KB]
    const char* a_own;
    char* a_ws_peer[kMaxRanks];
    float* sa_ws_peer[kMaxRanks];
    uint32_t* flags;
    uint32_t* flags_peer[kMaxRanks];
    int m_per_rank, n, k, kb_total;
    int world, rank;
    int seg_blocks;         // 128-row blocks per segment (one flag and one tile row each)
    int n_tiles, num_tiles, num_comm, mode;
    uint32_t epoch;
    WaitCtx wctx;
};

struct TileCoord {
    int seg, m_in_seg, n_tile;
};
__device__ __forceinline__ TileCoord decode_tile(int t, int first_seg, int world, int seg_m_tiles, int n_tiles) {
    const int per_seg = seg_m_tiles * n_tiles;
    const int si = t / per_seg;
    int r = t - si * per_seg;
    TileCoord c;
    c.seg = first_seg + si;
    if (c.seg >= world) c.seg -= world;
    const int group_span = 8 * n_tiles;
    const int g = r / group_span;
    r -= g * group_span;
    const int first_m = g * 8;
    const int gsize = min(8, seg_m_tiles - first_m);
    c.n_tile = r / gsize;
    c.m_in_seg = first_m + (r - c.n_tile * gsize);
    return c;
}

// acc2[0..N/2) (pairs of fp32) += r[0..N) * scale, two lanes per fma.rn.f32x2.
template <int N>
__device__ __forceinline__ void fold(unsigned long long* acc2, const uint32_t (&r)[N], unsigned long long s2) {
#pragma unroll
    for (int i = 0; i < N / 2; ++i) {
        unsigned long long v;
        asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "r"(r[2 * i]), "r"(r[2 * i + 1]));
        asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc2[i]) : "l"(v), "l"(s2));
    }
}
template <int N>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t (&r)[N]) {
    if constexpr (N == 8) tmem_ld_32x8(taddr, r);
    else tmem_ld_32x16(taddr, r);
}

// Pusher CTA: for each (destination, 128-row block) item all threads store the rows' scales into the
// destination (4-byte stores: a slab of scales starts and ends on no 16-byte boundary in general, so the
// bulk engine cannot move it), then thread 0 streams the rows through shared memory with bulk copies
// and raises the block's flag on the destination.
__device__ void pusher(const Params& p, uint8_t* smem, uint64_t* bars) {
    const int nitems = (p.world - 1) * p.seg_blocks;
    const size_t row_bytes = static_cast<size_t>(p.k);
    uint32_t it_load = 0, it_store = 0;
    auto stream = [&](const char* src, char* out, size_t bytes) {
        const int nchunks = static_cast<int>((bytes + PUSH_CHUNK - 1) / PUSH_CHUNK);
        for (int c = 0; c < nchunks + PUSH_AHEAD; ++c) {
            if (c < nchunks) {
                const uint32_t s = it_load % PUSH_STAGES;
                if (it_load >= PUSH_STAGES) bulk_wait_read<PUSH_STAGES - PUSH_AHEAD - 1>();
                const size_t off = static_cast<size_t>(c) * PUSH_CHUNK;
                const uint32_t sz = static_cast<uint32_t>(min(static_cast<size_t>(PUSH_CHUNK), bytes - off));
                mbar_expect_tx(smem_u32(&bars[s]), sz);
                bulk_load(smem_u32(smem + s * PUSH_CHUNK), src + off, sz, smem_u32(&bars[s]));
                ++it_load;
            }
            if (c >= PUSH_AHEAD) {
                const int cs = c - PUSH_AHEAD;
                const uint32_t s = it_store % PUSH_STAGES;
                mbar_wait(smem_u32(&bars[s]), (it_store / PUSH_STAGES) & 1u, p.wctx, 10);
                const size_t off = static_cast<size_t>(cs) * PUSH_CHUNK;
                const uint32_t sz = static_cast<uint32_t>(min(static_cast<size_t>(PUSH_CHUNK), bytes - off));
                bulk_store(out + off, smem_u32(smem + s * PUSH_CHUNK), sz);
                bulk_commit();
                ++it_store;
            }
        }
    };
    for (int item = static_cast<int>(blockIdx.x); item < nitems; item += p.num_comm) {
        const int hop = item / p.seg_blocks + 1;
        const int mb = item - (hop - 1) * p.seg_blocks;
        int dst = p.rank - hop;
        if (dst < 0) dst += p.world;
        const int rows = min(BM, p.m_per_rank - mb * BM);
        const size_t row0 = static_cast<size_t>(mb) * BM;
        const size_t dst_row0 = static_cast<size_t>(p.rank) * p.m_per_rank + row0;
        {
            const float* ssrc = p.sa_own + row0 * p.kb_total;
            float* sdst = p.sa_ws_peer[dst] + dst_row0 * p.kb_total;
            const int nsc = rows * p.kb_total;
            for (int i = static_cast<int>(threadIdx.x); i < nsc; i += 4 * THREADS) {
                float v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) v[u] = i + u * THREADS < nsc ? ssrc[i + u * THREADS] : 0.f;
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    if (i + u * THREADS < nsc) sdst[i + u * THREADS] = v[u];
            }
        }
        __syncthreads();  // the scale stores of every thread happen before thread 0's fence below
        if (threadIdx.x == 0) {
            stream(p.a_own + row0 * row_bytes, p.a_ws_peer[dst] + dst_row0 * row_bytes, rows * row_bytes);
            bulk_wait<0>();
            fence_proxy_async();
            fence_acq_rel_sys();
            st_release_sys_u32(p.flags_peer[dst] + p.rank * p.seg_blocks + mb, p.epoch);
        }
    }
}

template <int STG>
__global__ void __launch_bounds__(THREADS, 1) gemm_fp8_kernel(const __grid_constant__ Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_TILES);
    // slots: [0,S) full, [S,2S) empty, [2S,2S+2) tmem_full, [2S+2,2S+4) tmem_empty with S = MAX_STAGES
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 4);
    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const int lane = static_cast<int>(threadIdx.x) & 31;

    // pusher CTAs
    if (p.mode == TDIST_GEMM_AG && static_cast<int>(blockIdx.x) < p.num_comm) {
        if (threadIdx.x == 0) {
            for (int s = 0; s < PUSH_STAGES; ++s) mbar_init(smem_u32(&bars[s]), 1);
            fence_mbar_init();
        }
        __syncthreads();
        pusher(p, smem, bars);
        return;
    }
    const int cta = static_cast<int>(blockIdx.x) - p.num_comm;
    const int num_cta = static_cast<int>(gridDim.x) - p.num_comm;
    const int unit = cta, num_units = num_cta;
    const uint32_t bars_u32 = smem_u32(bars);
    auto bar_full = [&](int s) { return bars_u32 + 8u * s; };
    auto bar_empty = [&](int s) { return bars_u32 + 8u * (MAX_STAGES + s); };
    auto bar_tfull = [&](int b) { return bars_u32 + 8u * (2 * MAX_STAGES + b); };
    auto bar_tempty = [&](int b) { return bars_u32 + 8u * (2 * MAX_STAGES + 2 + b); };

    if (threadIdx.x == 0) {
        prefetch_tensormap(&p.tm_a);
        prefetch_tensormap(&p.tm_b);
        prefetch_tensormap(&p.tm_c);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_tfull(b), 1);
            mbar_init(bar_tempty(b), PROMO_WARPS);  // one arrival per promotion warp
        }
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish<1>();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
    const int first_seg = p.rank;

    if (warp == 0) {
        // ===================== TMA producer =====================
        if (lane == 0) {
            uint32_t it = 0;
            for (int t = unit; t < p.num_tiles; t += num_units) {
                const TileCoord tc = decode_tile(t, first_seg, p.world, p.seg_blocks, p.n_tiles);
                const int block = tc.m_in_seg;
                const CUtensorMap* am = &p.tm_a;
                int az = tc.seg;
                if (p.mode == TDIST_GEMM_AG) {
                    if (tc.seg == p.rank) {
                        am = &p.tm_a_own;
                        az = 0;
                    } else if (block < p.seg_blocks) {
                        wait_flag_ge_sys(p.flags + tc.seg * p.seg_blocks + block, p.epoch, p.wctx, tc.seg, block, 1);
                        fence_proxy_async();
                    }
                }
                const int row = block * BM;
                const int col = tc.n_tile * BN;
                for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    mbar_wait(bar_empty(s), ((it / STAGES) & 1u) ^ 1u, p.wctx, 2);
                    const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                    mbar_expect_tx(bar_full(s), STAGE_BYTES);
                    tma_load_3d(sa, am, bar_full(s), kb * BK, row, az);
                    tma_load_3d(sa + A_BYTES, &p.tm_b, bar_full(s), kb * BK, col, 0);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ===================== MMA issuer =====================
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(0u, 0u, BM, BN);  // e4m3 x e4m3 -> f32
            uint32_t it = 0;
            for (int t = unit; t < p.num_tiles; t += num_units) {
                for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
                    const uint32_t s = it % STAGES, buf = it & 1u;
                    mbar_wait(bar_tempty(buf), ((it >> 1) & 1u) ^ 1u, p.wctx, 3);
                    mbar_wait(bar_full(s), (it / STAGES) & 1u, p.wctx, 4);
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t adesc = umma_desc_k_sw128(sa);
                    const uint64_t bdesc = umma_desc_k_sw128(sa + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)  // 32 bytes of K per MMA = 2 descriptor units
                        umma_fp8<1>(tmem_base + buf * BN, adesc + 2 * k, bdesc + 2 * k, idesc, k != 0 ? 1u : 0u);
                    umma_commit(bar_empty(s));
                    umma_commit(bar_tfull(buf));
                }
            }
        }
        __syncwarp();
    } else {
        // ===================== promotion + epilogue (warps 2..9) =====================
        const int q = warp & 3;                  // TMEM lane quadrant
        const int half = (warp - 2) >> 2;        // which 128 columns
        const int row_in_tile = q * 32 + lane;
        const bool issuer = (warp == 2 && lane == 0);
        uint8_t* cstage = smem + PIPE_BYTES;
        uint32_t it = 0;
        for (int t = unit; t < p.num_tiles; t += num_units) {
            const TileCoord tc = decode_tile(t, first_seg, p.world, p.seg_blocks, p.n_tiles);
            const int block = tc.m_in_seg;
            const int row = block * BM + row_in_tile;                   // row inside the segment
            const bool own = p.mode == TDIST_GEMM_AG && tc.seg == p.rank;
            const int row_c = min(row, p.m_per_rank - 1);               // padding rows read a valid scale
            const float* sa_row = own ? p.sa_own + static_cast<size_t>(row_c) * p.kb_total
                                      : p.sa + (static_cast<size_t>(tc.seg) * p.m_per_rank + row_c) * p.kb_total;
            const int nblk = min((tc.n_tile * BN + half * 128) / 128, (p.n + 127) / 128 - 1);
            const float* sb_row = p.sb + static_cast<size_t>(nblk) * p.kb_total;
            if (p.mode == TDIST_GEMM_AG && !own && block < p.seg_blocks && lane == 0)
                wait_flag_ge_sys(p.flags + tc.seg * p.seg_blocks + block, p.epoch, p.wctx, tc.seg, block, 7);
            __syncwarp();
            unsigned long long acc[64];  // 128 fp32 accumulators as pairs
#pragma unroll
            for (int i = 0; i < 64; ++i) acc[i] = 0ull;
            float scale_next = sa_row[0] * sb_row[0];
            for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
                unsigned long long scale;
                asm("mov.b64 %0, {%1, %1};" : "=l"(scale) : "r"(__float_as_uint(scale_next)));
                if (kb + 1 < p.kb_total) scale_next = sa_row[kb + 1] * sb_row[kb + 1];
                const uint32_t buf = it & 1u;
                mbar_wait(bar_tfull(buf), (it >> 1) & 1u, p.wctx, 5);
                tc_fence_after();
                const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN + half * 128;
                // Two STG-register staging buffers (the load of chunk c+1 is in flight while chunk c is folded in):
                // with 128 accumulators per thread wider ones do not fit the 168 registers a 10-warp CTA gets,
                // and spills inside this loop cost more than the wider loads gain.
                constexpr int NCH = 128 / STG;
                uint32_t r0[STG], r1[STG];
                tmem_ld_cols<STG>(taddr, r0);
#pragma unroll
                for (int c = 0; c < NCH; c += 2) {
                    tmem_ld_wait();
                    tmem_ld_cols<STG>(taddr + STG * (c + 1), r1);
                    fold<STG>(acc + (STG / 2) * c, r0, scale);
                    tmem_ld_wait();
                    if (c + 2 < NCH) {
                        tmem_ld_cols<STG>(taddr + STG * (c + 2), r0);
                    } else {
                        // the block's partial sums are in registers: hand the TMEM buffer back to the MMA issuer
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_tempty(buf));
                    }
                    fold<STG>(acc + (STG / 2) * (c + 1), r1, scale);
                }
            }
            // ---- epilogue: this warp's 128 columns in two passes of 64, one staging buffer per column half
            const int col = tc.n_tile * BN;
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
                named_barrier(1, PROMO_WARPS * 32);  // the stores that last read the buffers have drained
                uint8_t* rowp = cstage + half * EPI_BYTES + row_in_tile * 128;
                const int sw = row_in_tile & 7;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    uint4 v;
                    const unsigned long long* a4 = acc + pass * 32 + j * 4;
                    v.x = pack_bf16x2(__uint_as_float(static_cast<uint32_t>(a4[0])), __uint_as_float(static_cast<uint32_t>(a4[0] >> 32)));
                    v.y = pack_bf16x2(__uint_as_float(static_cast<uint32_t>(a4[1])), __uint_as_float(static_cast<uint32_t>(a4[1] >> 32)));
                    v.z = pack_bf16x2(__uint_as_float(static_cast<uint32_t>(a4[2])), __uint_as_float(static_cast<uint32_t>(a4[2] >> 32)));
                    v.w = pack_bf16x2(__uint_as_float(static_cast<uint32_t>(a4[3])), __uint_as_float(static_cast<uint32_t>(a4[3] >> 32)));
                    *reinterpret_cast<uint4*>(rowp + ((j ^ sw) << 4)) = v;
                }
                fence_proxy_async_smem();
                named_barrier(1, PROMO_WARPS * 32);
                if (issuer) {
                    if (block < p.seg_blocks) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const int c0 = col + (h * 2 + pass) * EPI_COLS;
                            if (c0 < p.n) tma_store_3d(&p.tm_c, smem_u32(cstage + h * EPI_BYTES), c0, block * BM, tc.seg);
                        }
                    }
                    bulk_commit();
                    bulk_wait_read<0>();
                }
            }
        }
        if (issuer) bulk_wait<0>();
        __syncwarp();
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc<1>(tmem_base, TMEM_COLS);
}

}  // namespace fp8
}  // namespace tdist

using namespace tdist;
using tdist_host::fail;

namespace {

// CTAs of the kernel that can be resident at once (pusher and GEMM CTAs wait on one another through
// flags across ranks, so the grid never exceeds this). Cached per device.
int fp8_resident_ctas() {
    using namespace fp8;
    static int cache[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return tdist_host::sm_count();
    if (cache[dev] > 0) return cache[dev];
    int result = 0, per_sm = 0;
    if (cudaFuncSetAttribute(gemm_fp8_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) == cudaSuccess &&
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, gemm_fp8_kernel<16>, THREADS, SMEM_BYTES) == cudaSuccess && per_sm > 0)
        result = per_sm * tdist_host::sm_count();
    cudaGetLastError();
    if (result <= 0) result = tdist_host::sm_count();
    cache[dev] = result;
    return result;
}

}  // namespace

extern "C" int tdist_gemm_fp8_run(const TdistGemmFp8Args* a) {
    using namespace tdist::fp8;
    if (a == nullptr) return fail(TDIST_EINVAL, "null args");
    if (a->world < 1 || a->world > TDIST_MAX_RANKS || a->rank < 0 || a->rank >= a->world) return fail(TDIST_EINVAL, "fp8 gemm: world/rank out of range");
    if (a->mode != TDIST_GEMM_PLAIN && a->mode != TDIST_GEMM_AG) return fail(TDIST_EINVAL, "fp8 gemm: mode must be PLAIN or AG");
    if (a->m_per_rank < 1 || a->n < 1 || a->k < 1) return fail(TDIST_EINVAL, "fp8 gemm: empty problem");
    if (a->k % 128 != 0) return fail(TDIST_EINVAL, "fp8 gemm: K must be a multiple of 128 (one scale per 128 values)");
    if (a->n % 8 != 0) return fail(TDIST_EINVAL, "fp8 gemm: N must be a multiple of 8");
    if (!a->a || !a->b || !a->c || !a->sa || !a->sb) return fail(TDIST_EINVAL, "fp8 gemm: null operand");
    Params p;
    memset(&p, 0, sizeof(p));
    const uint64_t K = a->k, N = a->n, MPR = a->m_per_rank, W = a->world;
    const bool ag = a->mode == TDIST_GEMM_AG && a->world > 1;
    int rc;
    {
        const void* base = ag ? a->a_ws : a->a;
        if (base == nullptr) return fail(TDIST_EINVAL, "fp8 gemm: workspace pointer is null");
        uint64_t dims[3] = {K, MPR, (a->mode == TDIST_GEMM_AG && !ag) ? 1 : W};
        uint64_t strides[2] = {K, MPR * K};
        uint32_t box[3] = {BK, BM, 1};
        if ((rc = tdist_host::encode_tmap(&p.tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 3, base, dims, strides, box, tdist_host::Swizzle::B128))) return rc;
        uint64_t dims1[3] = {K, MPR, 1};
        if ((rc = tdist_host::encode_tmap(&p.tm_a_own, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 3, a->a, dims1, strides, box, tdist_host::Swizzle::B128))) return rc;
    }
    {
        uint64_t dims[3] = {K, N, 1};
        uint64_t strides[2] = {K, N * K};
        uint32_t box[3] = {BK, BN, 1};
        if ((rc = tdist_host::encode_tmap(&p.tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, 3, a->b, dims, strides, box, tdist_host::Swizzle::B128))) return rc;
    }
    {
        uint64_t dims[3] = {N, MPR, W};
        uint64_t strides[2] = {N * 2, MPR * N * 2};
        uint32_t box[3] = {EPI_COLS, BM, 1};
        if ((rc = tdist_host::encode_tmap(&p.tm_c, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, 3, a->c, dims, strides, box, tdist_host::Swizzle::B128))) return rc;
    }
    p.sa = static_cast<const float*>(ag ? a->sa_ws : a->sa);
    p.sa_own = static_cast<const float*>(a->sa);
    p.sb = static_cast<const float*>(a->sb);
    p.a_own = static_cast<const char*>(a->a);
    for (int r = 0; r < a->world; ++r) {
        p.a_ws_peer[r] = static_cast<char*>(a->a_ws_peer[r]);
        p.sa_ws_peer[r] = static_cast<float*>(a->sa_ws_peer[r]);
        p.flags_peer[r] = static_cast<uint32_t*>(a->flags_peer[r]);
        if (ag && (!p.a_ws_peer[r] || !p.sa_ws_peer[r] || !p.flags_peer[r])) return fail(TDIST_EINVAL, "fp8 AG gemm: null peer pointer");
    }
    if (ag && (!a->flags || !a->sa_ws)) return fail(TDIST_EINVAL, "fp8 AG gemm: null flags / scale workspace");
    p.flags = static_cast<uint32_t*>(a->flags);
    p.m_per_rank = a->m_per_rank;
    p.n = a->n;
    p.k = a->k;
    p.kb_total = a->k / 128;
    p.world = a->world;
    p.rank = a->rank;
    p.mode = a->mode;  // world 1 in AG mode: only the "own" path is used, no pushers
    p.seg_blocks = (a->m_per_rank + BM - 1) / BM;
    p.n_tiles = (a->n + BN - 1) / BN;
    p.num_tiles = p.seg_blocks * p.n_tiles * a->world;
    p.epoch = a->epoch;
    p.wctx.status = static_cast<Status*>(a->status);
    p.wctx.timeout_ns = a->timeout_ns;
    p.wctx.kernel_id = kKernelGemmFp8;
    p.wctx.rank = a->rank;
    const int capacity = fp8_resident_ctas();
    int sms = a->num_sms > 0 ? a->num_sms : capacity;
    if (sms > capacity) sms = capacity;
    if (sms < 1) sms = 1;
    p.num_comm = 0;
    if (ag) {
        p.num_comm = a->num_comm_sms > 0 ? a->num_comm_sms : 8;
        if (p.num_comm > sms - 1) p.num_comm = sms - 1;
        if (p.num_comm < 1) return fail(TDIST_EINVAL, "fp8 AG gemm: needs room for at least one pusher and one GEMM CTA");
    }
    int gemm_ctas = sms - p.num_comm;
    if (gemm_ctas > p.num_tiles) gemm_ctas = p.num_tiles;
    void* kargs[] = {&p};
    const void* fn = reinterpret_cast<const void*>(&gemm_fp8_kernel<16>);  // 8-column staging measured the same
    TDIST_CUDA_OK(cudaLaunchKernel(fn, dim3(gemm_ctas + p.num_comm), dim3(THREADS), kargs,
                                   SMEM_BYTES, static_cast<cudaStream_t>(a->stream)));
    return 0;
}
