// Expert-parallel MoE dispatch and combine over peer memory, one launch each, no host round trip.
//
//   DISPATCH  every CTA first routes in place: histogram of the (token, k) pairs by expert, exclusive scan, stable
//             counting sort, so that each pair knows the row it takes in its destination's receive buffer. Then a
//             warp per (token, 1024-value segment) loads the segment ONCE, optionally quantises it to fp8 e4m3 with
//             one fp32 scale per 128 values, and stores it straight into the receive buffers of the up to `topk`
//             ranks that own the token's experts (16-byte stores over NVLink). The last CTA to finish raises one
//             release flag per destination carrying the call number. Two receive layouts:
//               slots    source s owns rows [s * max_m, (s + 1) * max_m) of every receiver, sorted by local expert
//                        (what the low-latency all-to-all of the reference uses; no exchange before the rows move);
//               compact  rows grouped by (local expert, source rank) back to back, the layout an expert GEMM wants.
//                        The ranks first exchange their per-expert counts (one small put + flag each), every rank
//                        derives the start row of each (expert, source) group from the gathered counts, and the rows
//                        go straight to their final place.
//   COMBINE   pull: every rank announces that its expert outputs are in place, waits for the same announcement of the
//             others, then a warp per (token, 256-column chunk) reads the up to `topk` rows of the token from the
//             owning ranks' buffers through peer pointers, accumulates them in fp32 (optionally weighted) and writes
//             the token once. Nothing is staged and no second pass runs.
//
// Reference counterparts: kernels/nvidia/ep_a2a.py:35-147 (`kernel_dispatch_token`), :150-239 (`kernel_combine_token`),
// :242-306 (`kernel_get_ag_splits_and_recv_offset`), :309-321 (`kernel_bincount`) and the quantising dispatch of
// tutorials/04-deepseek-infer-all2all.py:150-201. There the counts travel through pinned host memory that the CPU
// polls; here they stay on the device.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../device/moe_sort.cuh"
#include "../device/shmem.cuh"
#include "../include/tdist.h"
#include "../runtime/host_common.h"

namespace tdist {

constexpr int kKernelMoeEp = 7;
constexpr int kEpSegLoads = 4;                       // 16-byte loads in flight per lane and item
constexpr int kEpSegValues = kEpSegLoads * 32 * 8;   // bf16 values per (token, segment) item: 1024

struct DispatchParams {
    const char* x;                  // [ntok, hidden] bf16
    const int* topk_ids;            // [ntok * topk]
    const int* slot_in;             // optional pre-computed routing (large token counts): sorted position of each pair
    const int* cumsum_in;           // ... and the exclusive prefix sum of the per-expert counts [E + 1]
    char* recv_peer[kMaxRanks];
    float* scale_peer[kMaxRanks];
    int* counts_peer[kMaxRanks];    // [world][E]
    uint64_t* sig_peer[kMaxRanks];  // [2 * world]: data flags, then count flags
    uint32_t* counters;             // local, [2]
    int* pair_row;                  // [ntok * topk]
    int* send_splits;               // [E]
    int* recv_splits;               // [world, epr]
    int* recv_offset;               // [epr, world] (compact)
    int* num_recv;                  // [1]
    int* block_expert;              // optional (compact): local expert of every `align`-row block of the receive buffer
    int* num_blocks;                // optional (compact): [1] live blocks
    int ntok, topk, hidden, E, epr, world, rank;
    int max_m, quant, compact, phase, align;
    uint64_t epoch;
    WaitCtx wctx;
};

// Exclusive scan of hist[0, E) into out[0, E] by warp 0 (a contiguous run of experts per lane).
__device__ __forceinline__ void scan_by_warp0(const int* hist, int E, int* out) {
    if (threadIdx.x < 32) {
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
            out[e] = acc;
            acc += hist[e];
        }
        if (lane == 31) out[E] = incl;
    }
}

// One segment of one token, quantised: lanes [0,16) and [16,32) each own a group of 128 values per load.
struct QuantSeg {
    uint2 q[kEpSegLoads];
    float scale[kEpSegLoads];
};

// The raw 16-byte loads of one (token, segment) item: issued early (before the routing, which does not need them) and
// consumed by quantise_segment / the plain copy afterwards.
__device__ __forceinline__ void load_segment(const char* src, int hidden, int seg, int lane, bool quant, uint4 (&raw)[kEpSegLoads]) {
    if (quant) {
        const int groups = hidden / 128;
        const int half = lane >> 4, sub = lane & 15;
        const int g0 = seg * (kEpSegLoads * 2);
#pragma unroll
        for (int u = 0; u < kEpSegLoads; ++u) {
            const int g = g0 + 2 * u + half;
            raw[u] = g < groups ? ld_nc_v4(src + (static_cast<size_t>(g) * 128 + sub * 8) * 2) : make_uint4(0, 0, 0, 0);
        }
    } else {
        const int b0 = seg * kEpSegValues * 2;
        const int b1 = min(hidden * 2, b0 + kEpSegValues * 2);
#pragma unroll
        for (int u = 0; u < kEpSegLoads; ++u) {
            const int off = b0 + u * 512 + lane * 16;
            raw[u] = off < b1 ? ld_nc_v4(src + off) : make_uint4(0, 0, 0, 0);
        }
    }
}

__device__ __forceinline__ void quantise_segment(const uint4 (&raw)[kEpSegLoads], QuantSeg& out) {
#pragma unroll
    for (int u = 0; u < kEpSegLoads; ++u) {
        const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
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
        const float scale = fmaxf(amax, 1e-10f) / 448.f;
        const float inv = 1.f / scale;
        uint32_t lo = 0, hi = 0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const uint32_t b0 = __nv_cvt_float2_to_fp8x2(make_float2(v[2 * i] * inv, v[2 * i + 1] * inv), __NV_SATFINITE, __NV_E4M3);
            const uint32_t b1 = __nv_cvt_float2_to_fp8x2(make_float2(v[4 + 2 * i] * inv, v[5 + 2 * i] * inv), __NV_SATFINITE, __NV_E4M3);
            lo |= b0 << (16 * i);
            hi |= b1 << (16 * i);
        }
        out.q[u] = make_uint2(lo, hi);
        out.scale[u] = scale;
    }
}

__global__ void __launch_bounds__(kMoeThreads, 1) moe_dispatch_kernel(const __grid_constant__ DispatchParams p) {
    extern __shared__ int sm[];
    const int E = p.E;
    const int n = p.ntok * p.topk;
    // shared memory: hist[E] | cum[E + 1] | base[E] | running[E] | cnt[kMoeWarps * E] | row[n] (routing in place only)
    int* hist = sm;
    int* cum = hist + E;
    int* base = cum + E + 1;
    int* running = base + E;
    int* cnt = running + E;
    int* row_s = cnt + kMoeWarps * E;
    const bool in_place = p.slot_in == nullptr;
    const int tid = static_cast<int>(threadIdx.x);
    const int warp = tid >> 5, lane = tid & 31;
    const bool first_cta = blockIdx.x == 0;

    // The rows do not depend on the routing: this warp's first (token, segment) item is loaded now, so that its
    // memory round trip runs under the sort below.
    const int segs = (p.hidden + kEpSegValues - 1) / kEpSegValues;
    const int gw = static_cast<int>(blockIdx.x) * kMoeWarps + warp;
    const int nw = static_cast<int>(gridDim.x) * kMoeWarps;
    uint4 raw[kEpSegLoads];
    if ((p.phase & 2) && gw < p.ntok * segs)
        load_segment(p.x + static_cast<size_t>(gw / segs) * p.hidden * 2, p.hidden, gw % segs, lane, p.quant != 0, raw);

    if (p.phase & 3) {
        // ---------------------------------------------------------------- per-expert counts of this rank
        if (in_place) {
            histogram(p.topk_ids, n, E, hist, p.wctx);
            scan_by_warp0(hist, E, cum);
        } else {
            for (int e = tid; e <= E; e += kMoeThreads) cum[e] = p.cumsum_in[e];
            __syncthreads();
            for (int e = tid; e < E; e += kMoeThreads) hist[e] = cum[e + 1] - cum[e];
        }
        __syncthreads();
    }

    if ((p.phase & 1) && p.compact && first_cta) {
        // ---------------------------------------------------------------- compact layout: publish the counts first
        for (int i = tid; i < p.world * E; i += kMoeThreads) {
            const int d = i / E, e = i - d * E;
            p.counts_peer[d][p.rank * E + e] = hist[e];
        }
        __syncthreads();
        if (tid < p.world) {
            fence_acq_rel_sys();
            st_release_sys_u64(p.sig_peer[tid] + p.world + p.rank, p.epoch);
        }
    }

    if (p.phase & 2) {
        // ---------------------------------------------------------------- start row of each expert's group at its owner
        if (p.compact) {
            if (tid < p.world) signal_wait_until(p.sig_peer[p.rank] + p.world + tid, kCmpGe, p.epoch, p.wctx, tid, 1);
            __syncthreads();
            const int* counts = p.counts_peer[p.rank];   // [world][E], complete after the waits above
            // running[e] = rows of expert e over all sources; cnt[e] (scratch) = rows of expert e from lower ranks
            for (int e = tid; e < E; e += kMoeThreads) {
                int tot = 0, before = 0;
                for (int s = 0; s < p.world; ++s) {
                    const int c = ld_relaxed_sys_u32(reinterpret_cast<const uint32_t*>(counts + s * E + e));
                    tot += c;
                    before += s < p.rank ? c : 0;
                }
                running[e] = tot;
                cnt[e] = before;
            }
            __syncthreads();
            // every expert's group starts on a multiple of `align` rows (128 = ready for the grouped GEMM, 1 = dense)
            const int al = p.align;
            for (int e = tid; e < E; e += kMoeThreads) {
                int b = cnt[e];
                for (int f = (e / p.epr) * p.epr; f < e; ++f) b += (running[f] + al - 1) / al * al;
                base[e] = b;
            }
            if (first_cta) {
                // what this rank receives: splits [src, le], start rows [le, src], total
                for (int i = tid; i < p.world * p.epr; i += kMoeThreads) {
                    const int s = i / p.epr, le = i - s * p.epr;
                    p.recv_splits[i] = ld_relaxed_sys_u32(reinterpret_cast<const uint32_t*>(counts + s * E + p.rank * p.epr + le));
                }
                for (int i = tid; i < p.epr * p.world; i += kMoeThreads) {
                    const int le = i / p.world, s = i - le * p.world;
                    int off = 0;
                    for (int f = 0; f < le; ++f) off += (running[p.rank * p.epr + f] + al - 1) / al * al;
                    if (s == 0 && p.block_expert != nullptr) {
                        const int nb = (running[p.rank * p.epr + le] + al - 1) / al;
                        for (int b = 0; b < nb; ++b)
                            if ((off / al + b + 1) * al <= p.max_m) p.block_expert[off / al + b] = le;
                    }
                    for (int q = 0; q < s; ++q) off += ld_relaxed_sys_u32(reinterpret_cast<const uint32_t*>(counts + q * E + p.rank * p.epr + le));
                    p.recv_offset[i] = off;
                }
                if (tid == 0) {
                    int tot = 0, padded = 0;
                    for (int le = 0; le < p.epr; ++le) {
                        tot += running[p.rank * p.epr + le];
                        padded += (running[p.rank * p.epr + le] + al - 1) / al * al;
                    }
                    *p.num_recv = tot;
                    if (p.num_blocks != nullptr) *p.num_blocks = min(padded, p.max_m) / al;
                    if (padded > p.max_m) report_timeout(p.wctx, kStatusBadArgument, -1, p.max_m, p.max_m, padded, 4);
                }
            }
            __syncthreads();
        } else {
            for (int e = tid; e < E; e += kMoeThreads) base[e] = p.rank * p.max_m + cum[e] - cum[(e / p.epr) * p.epr];
            __syncthreads();
        }
        // rows one receiver accepts from this rank (slots) or holds in all (compact)
        const int row_limit = p.compact ? p.max_m : (p.rank + 1) * p.max_m;

        // ---------------------------------------------------------------- row of every pair
        if (in_place) {
            for (int e = tid; e < E; e += kMoeThreads) running[e] = 0;   // position inside the expert's group
            __syncthreads();
            stable_positions(p.topk_ids, n, E, running, cnt, p.wctx, [&](int i, int pos) {
                int r = -1;
                if (pos >= 0) {
                    r = base[p.topk_ids[i]] + pos;
                    if (r >= row_limit) {
                        report_timeout(p.wctx, kStatusBadArgument, p.topk_ids[i] / p.epr, i, row_limit, r, 5);
                        r = -1;   // the destination has no room for this row: it is dropped, and reported
                    }
                }
                row_s[i] = r;
                if (first_cta) p.pair_row[i] = r;
            });
        } else if (first_cta) {
            for (int i = tid; i < n; i += kMoeThreads) {
                const int e = p.topk_ids[i];
                int r = -1;
                if (expert_in_range(e, E) && p.slot_in[i] >= 0) {
                    r = base[e] + p.slot_in[i] - cum[e];
                    if (r >= row_limit) {
                        report_timeout(p.wctx, kStatusBadArgument, e / p.epr, i, row_limit, r, 5);
                        r = -1;
                    }
                }
                p.pair_row[i] = r;
            }
        }
        if (first_cta) {
            for (int e = tid; e < E; e += kMoeThreads) p.send_splits[e] = hist[e];
            if (!p.compact) {
                // slots: the counts travel with the rows, clamped to the rows the slot can take
                for (int i = tid; i < p.world * E; i += kMoeThreads) {
                    const int d = i / E, e = i - d * E;
                    const int first = cum[(e / p.epr) * p.epr];
                    p.counts_peer[d][p.rank * E + e] = min(cum[e + 1] - first, p.max_m) - min(cum[e] - first, p.max_m);
                }
            }
        }
        __syncthreads();

        // ---------------------------------------------------------------- rows: load once, store to every owner
        const int row_bytes_out = p.quant ? p.hidden : p.hidden * 2;
        const int scale_cols = p.hidden / 128;
        for (int item = gw; item < p.ntok * segs; item += nw) {
            const int t = item / segs, seg = item - t * segs;
            if (item != gw) load_segment(p.x + static_cast<size_t>(t) * p.hidden * 2, p.hidden, seg, lane, p.quant != 0, raw);
            QuantSeg qs;
            if (p.quant) quantise_segment(raw, qs);
            const int half = lane >> 4, sub = lane & 15;
            const int b0 = seg * kEpSegValues * 2;
            const int b1 = min(p.hidden * 2, b0 + kEpSegValues * 2);
            for (int k = 0; k < p.topk; ++k) {
                const int i = t * p.topk + k;
                int r;
                if (in_place) {
                    r = row_s[i];
                } else {
                    const int e = p.topk_ids[i];
                    r = expert_in_range(e, E) && p.slot_in[i] >= 0 ? base[e] + p.slot_in[i] - cum[e] : -1;
                    if (r >= row_limit) r = -1;
                }
                if (r < 0) continue;
                const int d = p.topk_ids[i] / p.epr;
                char* dst = p.recv_peer[d] + static_cast<size_t>(r) * row_bytes_out;
                if (p.quant) {
                    float* dsc = p.scale_peer[d] + static_cast<size_t>(r) * scale_cols;
#pragma unroll
                    for (int u = 0; u < kEpSegLoads; ++u) {
                        const int g = seg * (kEpSegLoads * 2) + 2 * u + half;
                        if (g < scale_cols) {
                            *reinterpret_cast<uint2*>(dst + static_cast<size_t>(g) * 128 + sub * 8) = qs.q[u];
                            if (sub == 0) dsc[g] = qs.scale[u];
                        }
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < kEpSegLoads; ++u) {
                        const int off = b0 + u * 512 + lane * 16;
                        if (off < b1) st_v4(dst + off, raw[u]);
                    }
                }
            }
        }

        // ---------------------------------------------------------------- publish
        // One thread per CTA joins the arrival counter after the CTA barrier (gpu scope, acq_rel: every CTA's stores
        // happen before the last arrival); the last CTA fences at system scope and raises this source's flag on
        // every destination.
        __syncthreads();
        __shared__ int last_s;
        if (tid == 0) {
            const uint32_t old = atom_add_acq_rel_gpu_u32(p.counters, 1);
            last_s = old == gridDim.x - 1;
            if (last_s) p.counters[0] = 0;
        }
        __syncthreads();
        if (last_s && tid < p.world) {
            fence_acq_rel_sys();
            st_release_sys_u64(p.sig_peer[tid] + p.rank, p.epoch);
        }
    }

    if ((p.phase & 4) && first_cta) {
        // ---------------------------------------------------------------- every source's rows have landed here
        if (tid < p.world) signal_wait_until(p.sig_peer[p.rank] + tid, kCmpGe, p.epoch, p.wctx, tid, 2);
        __syncthreads();
        if (!p.compact) {
            const int* counts = p.counts_peer[p.rank];
            int part = 0;
            for (int i = tid; i < p.world * p.epr; i += kMoeThreads) {
                const int s = i / p.epr, le = i - s * p.epr;
                const int c = ld_relaxed_sys_u32(reinterpret_cast<const uint32_t*>(counts + s * E + p.rank * p.epr + le));
                p.recv_splits[i] = c;
                part += c;
            }
            // total rows received: block sum through shared memory
            __shared__ int total_s;
            if (tid == 0) total_s = 0;
            __syncthreads();
            if (part) atomicAdd(&total_s, part);
            __syncthreads();
            if (tid == 0) *p.num_recv = total_s;
        }
    }
}

// ------------------------------------------------------------------------------------------------ combine (pull)
struct CombineParams {
    const char* buf_peer[kMaxRanks];   // expert outputs [rows, hidden] bf16 of every rank as mapped here
    uint64_t* sig_peer[kMaxRanks];     // [world] "my outputs are in place" flags
    const int* topk_ids;
    const float* topk_w;               // nullptr = plain sum
    const int* pair_row;
    __nv_bfloat16* out;
    int ntok, topk, hidden, epr, world, rank, phase;
    uint64_t epoch;
    WaitCtx wctx;
};

__global__ void __launch_bounds__(kMoeThreads, 2) moe_combine_kernel(const __grid_constant__ CombineParams p) {
    const int tid = static_cast<int>(threadIdx.x);
    const int warp = tid >> 5, lane = tid & 31;
    if ((p.phase & 1) && blockIdx.x == 0 && tid < p.world) {
        // the expert outputs were written by earlier work of this stream: complete and visible to peer reads
        fence_acq_rel_sys();
        st_release_sys_u64(p.sig_peer[tid] + p.rank, p.epoch);
    }
    if (!(p.phase & 2)) return;
    if (tid < p.world) signal_wait_until(p.sig_peer[p.rank] + tid, kCmpGe, p.epoch, p.wctx, tid, 1);
    __syncthreads();
    const int gw = static_cast<int>(blockIdx.x) * kMoeWarps + warp;
    const int nw = static_cast<int>(gridDim.x) * kMoeWarps;
    const int chunks = (p.hidden + 255) / 256;   // a warp covers 256 columns (8 per lane) per item
    const size_t row_bytes = static_cast<size_t>(p.hidden) * 2;
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
                    const int r = p.pair_row[pair];
                    if (r >= 0) {
                        w[j] = p.topk_w ? p.topk_w[pair] : 1.f;
                        q[j] = ld_nc_v4(p.buf_peer[p.topk_ids[pair] / p.epr] + static_cast<size_t>(r) * row_bytes + static_cast<size_t>(c0) * 2);
                    }
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

}  // namespace tdist

using namespace tdist;
using tdist_host::fail;

static int dispatch_smem_bytes(int E, int n, bool in_place) {
    return (4 * E + 1 + kMoeWarps * E + (in_place ? n : 0)) * static_cast<int>(sizeof(int));
}

extern "C" int tdist_moe_dispatch(const TdistMoeDispatchArgs* a) {
    if (a == nullptr) return fail(TDIST_EINVAL, "moe_dispatch: null args");
    if (a->world < 1 || a->world > TDIST_MAX_RANKS || a->rank < 0 || a->rank >= a->world)
        return fail(TDIST_EINVAL, "moe_dispatch: world/rank out of range");
    if (a->num_experts < a->world || a->num_experts % a->world || a->num_experts > 1024)
        return fail(TDIST_EINVAL, "moe_dispatch: the expert count must be a multiple of the world size, at most 1024");
    if (a->ntok < 0 || a->topk < 1 || a->topk > 64 || a->hidden < 8 || a->hidden % 8)
        return fail(TDIST_EINVAL, "moe_dispatch: bad sizes (hidden must be a multiple of 8)");
    if (a->quant && a->hidden % 128) return fail(TDIST_EINVAL, "moe_dispatch: fp8 rows need hidden % 128 == 0");
    if (a->max_m < 1) return fail(TDIST_EINVAL, "moe_dispatch: max_m must be positive");
    const long long n = static_cast<long long>(a->ntok) * a->topk;
    const bool in_place = a->slot_of == nullptr;
    if (in_place && n > TDIST_MOE_ROUTE_IN_PLACE_MAX)
        return fail(TDIST_ELIMIT, "moe_dispatch: more pairs than the in-place routing takes; pass slot_of and cumsum");
    if (!in_place && a->cumsum == nullptr) return fail(TDIST_EINVAL, "moe_dispatch: slot_of needs cumsum");
    DispatchParams p;
    memset(&p, 0, sizeof(p));
    p.x = static_cast<const char*>(a->x);
    p.topk_ids = static_cast<const int*>(a->topk_ids);
    p.slot_in = static_cast<const int*>(a->slot_of);
    p.cumsum_in = static_cast<const int*>(a->cumsum);
    for (int r = 0; r < a->world; ++r) {
        p.recv_peer[r] = static_cast<char*>(a->recv_peer[r]);
        p.scale_peer[r] = static_cast<float*>(a->scale_peer[r]);
        p.counts_peer[r] = static_cast<int*>(a->counts_peer[r]);
        p.sig_peer[r] = static_cast<uint64_t*>(a->sig_peer[r]);
        if (!p.recv_peer[r] || !p.counts_peer[r] || !p.sig_peer[r]) return fail(TDIST_EINVAL, "moe_dispatch: null peer pointer");
        if (a->quant && !p.scale_peer[r]) return fail(TDIST_EINVAL, "moe_dispatch: fp8 rows need the scale buffers");
    }
    p.counters = static_cast<uint32_t*>(a->counters);
    p.pair_row = static_cast<int*>(a->pair_row);
    p.send_splits = static_cast<int*>(a->send_splits);
    p.recv_splits = static_cast<int*>(a->recv_splits);
    p.recv_offset = static_cast<int*>(a->recv_offset);
    p.num_recv = static_cast<int*>(a->num_recv);
    p.block_expert = static_cast<int*>(a->block_expert);
    p.num_blocks = static_cast<int*>(a->num_blocks);
    p.align = a->align > 0 ? a->align : 1;
    if (!p.x || !p.topk_ids || !p.counters || !p.pair_row || !p.send_splits || !p.recv_splits || !p.num_recv)
        return fail(TDIST_EINVAL, "moe_dispatch: null pointer");
    if (a->compact && !p.recv_offset) return fail(TDIST_EINVAL, "moe_dispatch: the compact layout needs recv_offset");
    p.ntok = a->ntok;
    p.topk = a->topk;
    p.hidden = a->hidden;
    p.E = a->num_experts;
    p.epr = a->num_experts / a->world;
    p.world = a->world;
    p.rank = a->rank;
    p.max_m = a->max_m;
    p.quant = a->quant;
    p.compact = a->compact;
    p.phase = a->phase ? a->phase : 7;
    p.epoch = a->epoch;
    p.wctx.status = static_cast<Status*>(a->status);
    p.wctx.timeout_ns = a->timeout_ns;
    p.wctx.kernel_id = kKernelMoeEp;
    p.wctx.rank = a->rank;
    const int smem = dispatch_smem_bytes(p.E, static_cast<int>(n), in_place);
    static bool attr_set[64] = {};
    int dev = 0;
    TDIST_CUDA_OK(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        TDIST_CUDA_OK(cudaFuncSetAttribute(moe_dispatch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
        attr_set[dev] = true;
    }
    if (smem > 160 * 1024) return fail(TDIST_ELIMIT, "moe_dispatch: routing tables exceed shared memory");
    // one CTA per SM at most (every CTA routes for itself), and no more CTAs than there are warps' worth of items
    const int segs = (a->hidden + kEpSegValues - 1) / kEpSegValues;
    int ctas = a->num_ctas > 0 ? a->num_ctas : (a->ntok * segs + kMoeWarps - 1) / kMoeWarps;
    const int sms = tdist_host::sm_count();
    if (ctas > sms) ctas = sms;
    if (ctas < 1 || !(p.phase & 2)) ctas = 1;   // counts-only and wait-only launches need one CTA
    moe_dispatch_kernel<<<ctas, kMoeThreads, smem, static_cast<cudaStream_t>(a->stream)>>>(p);
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}

extern "C" int tdist_moe_combine(const TdistMoeCombineArgs* a) {
    if (a == nullptr) return fail(TDIST_EINVAL, "moe_combine: null args");
    if (a->world < 1 || a->world > TDIST_MAX_RANKS || a->rank < 0 || a->rank >= a->world)
        return fail(TDIST_EINVAL, "moe_combine: world/rank out of range");
    if (a->ntok < 0 || a->topk < 1 || a->hidden < 8 || a->hidden % 8 || a->epr < 1)
        return fail(TDIST_EINVAL, "moe_combine: bad sizes (hidden must be a multiple of 8)");
    CombineParams p;
    memset(&p, 0, sizeof(p));
    for (int r = 0; r < a->world; ++r) {
        p.buf_peer[r] = static_cast<const char*>(a->buf_peer[r]);
        p.sig_peer[r] = static_cast<uint64_t*>(a->sig_peer[r]);
        if (!p.buf_peer[r] || !p.sig_peer[r]) return fail(TDIST_EINVAL, "moe_combine: null peer pointer");
    }
    p.topk_ids = static_cast<const int*>(a->topk_ids);
    p.topk_w = static_cast<const float*>(a->topk_w);
    p.pair_row = static_cast<const int*>(a->pair_row);
    p.out = static_cast<__nv_bfloat16*>(a->out);
    if (!p.topk_ids || !p.pair_row || !p.out) return fail(TDIST_EINVAL, "moe_combine: null pointer");
    p.ntok = a->ntok;
    p.topk = a->topk;
    p.hidden = a->hidden;
    p.epr = a->epr;
    p.world = a->world;
    p.rank = a->rank;
    p.phase = a->phase ? a->phase : 3;
    p.epoch = a->epoch;
    p.wctx.status = static_cast<Status*>(a->status);
    p.wctx.timeout_ns = a->timeout_ns;
    p.wctx.kernel_id = kKernelMoeEp;
    p.wctx.rank = a->rank;
    const int chunks = (a->hidden + 255) / 256;
    int ctas = a->num_ctas > 0 ? a->num_ctas : (a->ntok * chunks + kMoeWarps - 1) / kMoeWarps;
    const int cap = 2 * tdist_host::sm_count();
    if (ctas > cap) ctas = cap;
    if (ctas < 1 || !(p.phase & 2)) ctas = 1;
    moe_combine_kernel<<<ctas, kMoeThreads, 0, static_cast<cudaStream_t>(a->stream)>>>(p);
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}
