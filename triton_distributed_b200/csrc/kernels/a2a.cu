// Low-latency MoE all-to-all (expert-parallel dispatch and combine) over peer memory.
//
// One launch moves every row to the rank that owns its expert: CTA group g of the grid serves
// destination (rank + g) % world, a warp per row, 16-byte vector stores straight into the
// destination's receive slot for this source, then the per-expert counts, then one release flag
// per (source, destination) carrying the call number. Receive buffers are double-buffered by call
// parity, so no reset pass and no barrier are needed between calls.
//
//   DISPATCH  rows of `send` (optionally gathered through `src_index`, optionally quantised on
//             the fly to fp8 e4m3 with one fp32 scale per 128 values) go to the expert ranks.
//   COMBINE   rows of the expert ranks' receive-layout buffer go back to their source ranks; with
//             `reduce` set the kernel then waits for all returns and computes
//             out[t] = sum_k w[t,k] * returned_row(t,k) in fp32.
//
// Reference counterparts: kernels/nvidia/low_latency_all_to_all.py:35-118 (`all_to_all_kernel`, one
// CTA per destination, NVSHMEM putmem_nbi_block + signal) and the quantising variant of
// tutorials/04-deepseek-infer-all2all.py:150-201,308-368.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../device/shmem.cuh"
#include "../include/tdist.h"
#include "../runtime/host_common.h"

namespace tdist {

constexpr int kKernelA2A = 3;
constexpr int kA2AThreads = 512;

struct A2AParams {
    const char* send;              // DISPATCH: [rows, row_bytes_in]; COMBINE: receive-layout [world*max_m, row_bytes_in]
    const int* src_index;          // DISPATCH, optional: source row of sorted row i
    const int* counts;             // DISPATCH: cumsum [G+1]; COMBINE: received splits [world*epr]
    const float* send_scale;       // optional [rows, scale_cols] (copied along, not used with quant)
    char* recv_peer[kMaxRanks];    // this call's parity: [world(src)][max_m][row_bytes_out]
    float* scale_peer[kMaxRanks];  // [world(src)][max_m][scale_cols]
    int* splits_peer[kMaxRanks];   // [world(src)][epr]
    uint64_t* sig_peer[kMaxRanks]; // [world]
    uint32_t* counters;            // local [world]
    // fused reduction (COMBINE only)
    const int* slot_of;            // [ntok*topk]: position of (t,k) in this rank's sorted send order
    const int* cumsum;             // [G+1] of this rank's dispatch
    const int* topk_ids;           // [ntok*topk]
    const float* topk_w;           // [ntok*topk]
    __nv_bfloat16* out;            // [ntok, hidden]
    int ntok, topk;
    int row_bytes_in, row_bytes_out, scale_cols, hidden;
    int max_m, epr, world, rank;
    int mode, quant, reduce, phase, ctas_per_peer;
    uint64_t epoch;
    WaitCtx wctx;
};

// Work is dealt to warps in (row, segment) items so that a 128-row message still occupies every
// warp of the grid and each item costs about one memory round trip.
constexpr int kSegLoads = 8;                      // 16-byte loads in flight per lane
constexpr int kSegBytes = kSegLoads * 512;        // plain copy: bytes per item
constexpr int kSegGroups = kSegLoads * 2;         // quantising copy: groups of 128 values per item

__device__ __forceinline__ void copy_seg_warp(char* dst, const char* src, int bytes, int seg, int lane) {
    const int b0 = seg * kSegBytes;
    const int b1 = min(bytes, b0 + kSegBytes);
    uint4 q[kSegLoads];
#pragma unroll
    for (int u = 0; u < kSegLoads; ++u) {
        const int i = b0 + u * 512 + lane * 16;
        if (i < b1) q[u] = ld_nc_v4(src + i);
    }
#pragma unroll
    for (int u = 0; u < kSegLoads; ++u) {
        const int i = b0 + u * 512 + lane * 16;
        if (i < b1) st_v4(dst + i, q[u]);
    }
}

// bf16 -> fp8 e4m3 with one fp32 scale per 128 values (scale = amax / 448) for groups
// [16*seg, 16*seg + 16) of one row. A half-warp (16 lanes x 8 values) owns a group; the eight groups
// of each half-warp are loaded before any is processed.
__device__ __forceinline__ void quant_seg_warp(char* dst, float* dst_scale, const char* src, int hidden, int seg, int lane) {
    const int groups = hidden / 128;
    const int half = lane >> 4, sub = lane & 15;
    const int g0 = seg * kSegGroups;
    uint4 q[kSegLoads];
#pragma unroll
    for (int u = 0; u < kSegLoads; ++u) {
        const int g = g0 + 2 * u + half;
        q[u] = g < groups ? ld_nc_v4(src + (static_cast<size_t>(g) * 128 + sub * 8) * 2) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < kSegLoads; ++u) {
        const int g = g0 + 2 * u + half;
        const bool active = g < groups;
        const uint32_t w[4] = {q[u].x, q[u].y, q[u].z, q[u].w};
        float v[8];
        float amax = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
            amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
        }
#pragma unroll
        for (int o = 8; o >= 1; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (active) {
            const float scale = fmaxf(amax, 1e-10f) / 448.f;
            const float inv = 1.f / scale;
            // packed conversion: one cvt.rn.satfinite.e4m3x2.f32 per pair of values (.x lands in the low byte)
            uint32_t lo = 0, hi = 0;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t b0 = __nv_cvt_float2_to_fp8x2(make_float2(v[2 * i] * inv, v[2 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
                const uint32_t b1 = __nv_cvt_float2_to_fp8x2(make_float2(v[4 + 2 * i] * inv, v[5 + 2 * i] * inv), __NV_SATFINITE, __NV_E4M3);
                lo |= b0 << (16 * i);
                hi |= b1 << (16 * i);
            }
            *reinterpret_cast<uint2*>(dst + static_cast<size_t>(g) * 128 + sub * 8) = make_uint2(lo, hi);
            if (sub == 0) dst_scale[g] = scale;
        }
    }
}

__global__ void __launch_bounds__(kA2AThreads, 2) a2a_kernel(const A2AParams p) {
    const int g = static_cast<int>(blockIdx.x) / p.ctas_per_peer;
    const int slice = static_cast<int>(blockIdx.x) % p.ctas_per_peer;
    const int dest = (p.rank + g) % p.world;
    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const int lane = static_cast<int>(threadIdx.x) & 31;
    const int warps = static_cast<int>(blockDim.x) >> 5;

    if (p.phase & 1) {
        int first, count;
        if (p.mode == TDIST_A2A_DISPATCH) {
            first = p.counts[dest * p.epr];
            count = p.counts[(dest + 1) * p.epr] - first;
        } else {
            first = dest * p.max_m;
            count = 0;
            for (int e = 0; e < p.epr; ++e) count += p.counts[dest * p.epr + e];
        }
        if (count > p.max_m) {
            // A destination's slot for this source holds max_m rows: the surplus is not sent, the splits published
            // below are clamped to what was sent, and the host learns of it through the status block.
            if (slice == 0 && threadIdx.x == 0) report_timeout(p.wctx, kStatusBadArgument, dest, p.max_m, p.max_m, count, 3);
            count = p.max_m;
        }
        char* rbase = p.recv_peer[dest] + static_cast<size_t>(p.rank) * p.max_m * p.row_bytes_out;
        float* sbase = p.scale_peer[dest] ? p.scale_peer[dest] + static_cast<size_t>(p.rank) * p.max_m * p.scale_cols : nullptr;
        const int segs = p.quant ? (p.hidden / 128 + kSegGroups - 1) / kSegGroups : (p.row_bytes_in + kSegBytes - 1) / kSegBytes;
        for (int item = slice * warps + warp; item < count * segs; item += p.ctas_per_peer * warps) {
            const int i = item / segs, seg = item - i * segs;
            int srow = first + i;
            if (p.src_index != nullptr) srow = p.src_index[srow];
            const char* src = p.send + static_cast<size_t>(srow) * p.row_bytes_in;
            char* dst = rbase + static_cast<size_t>(i) * p.row_bytes_out;
            if (p.quant) {
                quant_seg_warp(dst, sbase + static_cast<size_t>(i) * p.scale_cols, src, p.hidden, seg, lane);
            } else {
                copy_seg_warp(dst, src, p.row_bytes_in, seg, lane);
                if (seg == 0 && sbase != nullptr && p.send_scale != nullptr)
                    for (int c = lane; c < p.scale_cols; c += 32)
                        sbase[static_cast<size_t>(i) * p.scale_cols + c] = p.send_scale[static_cast<size_t>(srow) * p.scale_cols + c];
            }
        }
        if (p.mode == TDIST_A2A_DISPATCH && slice == 0 && static_cast<int>(threadIdx.x) < p.epr) {
            const int e = dest * p.epr + threadIdx.x;
            const int lo = min(p.counts[e] - first, p.max_m), hi = min(p.counts[e + 1] - first, p.max_m);
            p.splits_peer[dest][p.rank * p.epr + threadIdx.x] = hi - lo;   // rows of this expert that were sent
        }
        // Publish: the last CTA of the group raises this source's flag on the destination. Only one
        // thread per CTA fences: the CTA barrier orders every thread's stores before thread 0's
        // release (gpu scope, chained through the counter), and the last CTA's system-scope fence +
        // release store makes all of them visible to the destination before the flag. A system
        // fence in every one of the grid's ~70K threads costs tens of microseconds.
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t old = atom_add_acq_rel_gpu_u32(p.counters + dest, 1);
            if (old == static_cast<uint32_t>(p.ctas_per_peer - 1)) {
                p.counters[dest] = 0;
                fence_acq_rel_sys();
                st_release_sys_u64(p.sig_peer[dest] + p.rank, p.epoch);
            }
        }
    }
    if (!(p.phase & 2)) return;

    if (!p.reduce) {
        // each group's first CTA waits for the flag of the rank it just served
        if (slice == 0 && threadIdx.x == 0)
            signal_wait_until(p.sig_peer[p.rank] + dest, kCmpGe, p.epoch, p.wctx, dest, 1);
        return;
    }
    // ---- fused combine reduction: every CTA waits for all returns, then a warp per token
    if (static_cast<int>(threadIdx.x) < p.world)
        signal_wait_until(p.sig_peer[p.rank] + threadIdx.x, kCmpGe, p.epoch, p.wctx, threadIdx.x, 2);
    __syncthreads();
    const char* rlocal = p.recv_peer[p.rank];
    const int gw = static_cast<int>(blockIdx.x) * warps + warp;
    const int nw = static_cast<int>(gridDim.x) * warps;
    const int chunks = (p.hidden + 255) / 256;  // a warp covers 256 columns (8 per lane) per item
    for (int item = gw; item < p.ntok * chunks; item += nw) {
        const int t = item / chunks;
        const int c0 = (item - t * chunks) * 256 + lane * 8;
        if (c0 >= p.hidden) continue;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int k0 = 0; k0 < p.topk; k0 += 8) {
            uint4 q[8];
            float w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int k = k0 + j;
                w[j] = 0.f;
                q[j] = make_uint4(0, 0, 0, 0);
                if (k < p.topk) {
                    const int pair = t * p.topk + k;
                    const int er = p.topk_ids[pair] / p.epr;
                    const int row = er * p.max_m + (p.slot_of[pair] - p.cumsum[er * p.epr]);
                    w[j] = p.topk_w[pair];
                    q[j] = ld_nc_v4(rlocal + static_cast<size_t>(row) * p.row_bytes_out + static_cast<size_t>(c0) * 2);
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
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        st_v4(reinterpret_cast<char*>(p.out) + (static_cast<size_t>(t) * p.hidden + c0) * 2, o);
    }
}

// fp8 e4m3 rows + per-128 scales -> bf16 rows (expert-side dequantisation; reference
// tutorials/04-deepseek-infer-all2all.py `_dequant_kernel`).
__global__ void dequant_fp8_kernel(const uint8_t* x, const float* scale, __nv_bfloat16* out, int rows, int hidden) {
    const int groups = hidden / 128;
    const size_t total = static_cast<size_t>(rows) * hidden / 8;
    for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t e0 = i * 8;
        const size_t r = e0 / hidden;
        const int c = static_cast<int>(e0 - r * hidden);
        const float s = scale[r * groups + c / 128];
        const uint2 q = *reinterpret_cast<const uint2*>(x + e0);
        float v[8];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const float2 a = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>((q.x >> (16 * j)) & 0xffff), __NV_E4M3)));
            const float2 b = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(static_cast<__nv_fp8x2_storage_t>((q.y >> (16 * j)) & 0xffff), __NV_E4M3)));
            v[2 * j] = a.x * s;
            v[2 * j + 1] = a.y * s;
            v[4 + 2 * j] = b.x * s;
            v[5 + 2 * j] = b.y * s;
        }
        uint4 o;
        o.x = pack_bf16x2(v[0], v[1]);
        o.y = pack_bf16x2(v[2], v[3]);
        o.z = pack_bf16x2(v[4], v[5]);
        o.w = pack_bf16x2(v[6], v[7]);
        *reinterpret_cast<uint4*>(out + e0) = o;
    }
}

}  // namespace tdist

using namespace tdist;
using tdist_host::fail;

extern "C" int tdist_a2a(const TdistA2AArgs* a) {
    if (a->world < 1 || a->world > TDIST_MAX_RANKS || a->rank < 0 || a->rank >= a->world)
        return fail(TDIST_EINVAL, "a2a: world/rank out of range");
    if (a->epr < 1 || a->epr > kA2AThreads) return fail(TDIST_EINVAL, "a2a: experts per rank must be in [1, 512]");
    if (a->row_bytes_in % 16 || a->row_bytes_out % 16) return fail(TDIST_EINVAL, "a2a: row sizes must be multiples of 16 bytes");
    if (a->quant && (a->hidden % 128 || a->row_bytes_in != a->hidden * 2 || a->row_bytes_out != a->hidden || a->scale_cols != a->hidden / 128))
        return fail(TDIST_EINVAL, "a2a: fp8 quantisation needs bf16 rows with hidden % 128 == 0 and scale_cols == hidden / 128");
    if (a->reduce && (a->mode != TDIST_A2A_COMBINE || a->hidden % 8 || a->row_bytes_out != a->hidden * 2))
        return fail(TDIST_EINVAL, "a2a: the fused reduction is for bf16 combine");
    A2AParams p;
    memset(&p, 0, sizeof(p));
    p.send = static_cast<const char*>(a->send);
    p.src_index = static_cast<const int*>(a->src_index);
    p.counts = static_cast<const int*>(a->counts);
    p.send_scale = static_cast<const float*>(a->send_scale);
    for (int r = 0; r < a->world; ++r) {
        p.recv_peer[r] = static_cast<char*>(a->recv_peer[r]);
        p.scale_peer[r] = static_cast<float*>(a->scale_peer[r]);
        p.splits_peer[r] = static_cast<int*>(a->splits_peer[r]);
        p.sig_peer[r] = static_cast<uint64_t*>(a->sig_peer[r]);
        if (!p.recv_peer[r] || !p.sig_peer[r] || (a->mode == TDIST_A2A_DISPATCH && !p.splits_peer[r]))
            return fail(TDIST_EINVAL, "a2a: null peer pointer");
        if (a->quant && !p.scale_peer[r]) return fail(TDIST_EINVAL, "a2a: quantisation needs the scale buffers");
    }
    p.counters = static_cast<uint32_t*>(a->counters);
    p.slot_of = static_cast<const int*>(a->slot_of);
    p.cumsum = static_cast<const int*>(a->cumsum);
    p.topk_ids = static_cast<const int*>(a->topk_ids);
    p.topk_w = static_cast<const float*>(a->topk_w);
    p.out = static_cast<__nv_bfloat16*>(a->out);
    p.ntok = a->ntok;
    p.topk = a->topk;
    p.row_bytes_in = a->row_bytes_in;
    p.row_bytes_out = a->row_bytes_out;
    p.scale_cols = a->scale_cols;
    p.hidden = a->hidden;
    p.max_m = a->max_m;
    p.epr = a->epr;
    p.world = a->world;
    p.rank = a->rank;
    p.mode = a->mode;
    p.quant = a->quant;
    p.reduce = a->reduce;
    p.phase = a->phase ? a->phase : 3;
    // about one CTA per SM in total: the rows of a small message are spread over the whole machine
    p.ctas_per_peer = a->ctas_per_peer > 0 ? a->ctas_per_peer : 288 / a->world;  // two 512-thread CTAs per SM
    if (p.ctas_per_peer > 144) p.ctas_per_peer = 144;
    if (p.ctas_per_peer < 1) p.ctas_per_peer = 1;
    p.epoch = a->epoch;
    p.wctx.status = static_cast<Status*>(a->status);
    p.wctx.timeout_ns = a->timeout_ns;
    p.wctx.kernel_id = kKernelA2A;
    p.wctx.rank = a->rank;
    if (!p.send || !p.counts || !p.counters) return fail(TDIST_EINVAL, "a2a: null send/counts/counters");
    if (a->reduce && (!p.slot_of || !p.cumsum || !p.topk_ids || !p.topk_w || !p.out))
        return fail(TDIST_EINVAL, "a2a: the fused reduction needs slot_of, cumsum, topk_ids, topk_w and out");
    a2a_kernel<<<a->world * p.ctas_per_peer, kA2AThreads, 0, static_cast<cudaStream_t>(a->stream)>>>(p);
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}

extern "C" int tdist_dequant_fp8(const void* x, const void* scale, void* out, int rows, int hidden, void* stream) {
    if (hidden % 128) return fail(TDIST_EINVAL, "dequant: hidden must be a multiple of 128");
    if (rows <= 0) return 0;
    const size_t total = static_cast<size_t>(rows) * hidden / 8;
    const int blocks = static_cast<int>(min(static_cast<size_t>(592), (total + 255) / 256));
    dequant_fp8_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint8_t*>(x), static_cast<const float*>(scale), static_cast<__nv_bfloat16*>(out), rows, hidden);
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}
