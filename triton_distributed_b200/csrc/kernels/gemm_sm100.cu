// Persistent warp-specialised tcgen05 GEMM for sm_100a and its two fused forms.
//
//   PLAIN  C[M,N] = A[M,K] * B[N,K]^T
//   AG     AllGather-GEMM (tensor-parallel column-parallel linear). Each rank holds a row shard
//          of A; dedicated pusher CTAs of the SAME kernel copy the shard into every peer's
//          gather workspace 128 rows at a time (bulk-async copies over NVLink) and publish one
//          flag per 128-row block; the MMA side consumes its own rows first, then the peers'
//          blocks in arrival order, waiting per block. Plays the role of the reference's
//          `ag_gemm_intra_node` (python/triton_dist/kernels/nvidia/allgather_gemm.py:131-252,
//          835-882), where the gather is a copy-engine stream and the wait is per rank.
//   RS     GEMM-ReduceScatter (row-parallel linear). The epilogue TMA-stores each partial tile
//          straight into the owning rank's staging slot over NVLink and raises that tile's flag;
//          this rank's own rows come last, and the epilogue of such a tile adds the other ranks'
//          partials of it (in fp32) and stores the finished rows, so no reduce pass follows the
//          GEMM. Plays the role of the reference's `gemm_rs`
//          (python/triton_dist/kernels/nvidia/gemm_reduce_scatter.py:104-232,482-538 and
//          reduce_scatter.py:527-685), where scatter and reduction are separate streams.
//
// Three tilings of the same kernel body:
//   CTAS = 1        one CTA computes a 128 x 256 tile (tcgen05.mma cta_group::1), 4 TMA stages of 48 KB.
//   CTAS = 2        a cluster of two CTAs computes a 256 x 256 tile (cta_group::2): each CTA loads its own
//                   128 rows of A and its own half (128 rows) of the B tile, the leader CTA issues the MMAs
//                   for both, 6 stages of 32 KB per CTA. B is read from L2 once per pair.
//   CTAS = 2, WIDE  the pair computes a 256 x 512 tile as two 256 x 256 halves that share the A rows: per
//                   K block each CTA loads 16 KB of A and 2 x 16 KB of B (4 stages of 48 KB) for twice the
//                   MMA work, so a quarter less operand traffic from L2 into shared memory per FLOP and a
//                   quarter less shared-memory write bandwidth beside the tensor core's own operand reads.
//                   The two halves fill all 512 TMEM columns: the epilogue of a tile overlaps the next main
//                   loop only half by half (each half has its own full / empty barrier), which long-K
//                   problems do not notice. When the last round of tiles would leave at least half of the
//                   CTA pairs idle, its tiles are split into their 256 x 256 halves.
// No TMA load here uses cluster multicast. K advances 64 elements per stage; the fp32 accumulators live in two
// TMEM slots of 256 columns: narrow tiles alternate between them so that the epilogue of tile i overlaps the
// main loop of tile i+1, a wide tile takes both.
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer and TMEM owner,
// warps 2..5 = epilogue (TMEM -> registers -> swizzled smem -> TMA store).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <string>

#include "../device/ptx.cuh"
#include "../device/signal.cuh"
#include "../include/tdist.h"
#include "../runtime/host_common.h"

namespace tdist {

constexpr int BM = 128;   // rows per CTA
constexpr int BN = 256;   // columns per tile
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int EPI_COLS = 64;                    // columns per epilogue store
constexpr int EPI_BYTES = BM * EPI_COLS * 2;    // 16 KB
constexpr int PIPE_BYTES = 192 * 1024;          // operand stages (either tiling)
constexpr int SMEM_TILES = PIPE_BYTES + 2 * EPI_BYTES;
constexpr int SMEM_BYTES = SMEM_TILES + 1024 /*alignment slack*/ + 256 /*barriers*/;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int DEFAULT_GROUP_M = 8;
constexpr int MAX_STAGES = 6;

template <int CTAS, bool WIDE = false>
struct Tiling {
    static_assert(!WIDE || CTAS == 2, "the wide tiling is a CTA-pair tiling");
    static constexpr int HALVES = WIDE ? 2 : 1;           // 256-column halves of a tile
    static constexpr int B_ROWS = BN / CTAS;              // rows of one half of the B tile this CTA loads
    static constexpr int B_BYTES = B_ROWS * BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + HALVES * B_BYTES;
    static constexpr int STAGES = PIPE_BYTES / STAGE_BYTES;  // 4, 6 or 4
    static_assert(STAGES <= MAX_STAGES, "barrier area too small");
};

// Pusher pipeline (AG): PUSH_STAGES buffers of PUSH_CHUNK bytes, loads run PUSH_AHEAD chunks
// ahead of the stores.
constexpr int PUSH_CHUNK = 32768;
constexpr int PUSH_STAGES = 7;
constexpr int PUSH_AHEAD = 5;
static_assert(PUSH_STAGES * PUSH_CHUNK <= SMEM_TILES, "pusher buffers must fit the tile area");

constexpr int kKernelGemm = 1;

struct GemmParams {
    CUtensorMap tm_a;       // PLAIN/RS: A as {K, m_per_rank, world}; AG: the gather workspace
    CUtensorMap tm_a_own;   // AG: this rank's shard as {K, m_per_rank, 1}
    CUtensorMap tm_b;       // {K, N, 1}
    CUtensorMap tm_c[kMaxRanks];  // PLAIN/AG: [0] = C as {N, m_per_rank, world}; RS: per owner
    const char* a_own;            // AG pusher source
    char* a_ws_peer[kMaxRanks];
    const char* stage_local;      // RS reduce source [world][m_per_rank][N]
    char* a_ws_mc;                // AG: multicast alias of the gather workspace (NVLS pusher), or nullptr
    void* rs_out;
    int rs_fused;                 // RS: the epilogue of this rank's own tiles adds the peers' partials and writes rs_out itself
    uint32_t* flags;
    uint32_t* flags_peer[kMaxRanks];
    int m_per_rank, n, k;
    int world, rank;
    int seg_m_tiles, n_tiles, k_blocks;
    int seg_blocks;  // 128-row blocks per segment (flag granularity)
    int num_tiles;   // work items of the schedule: 256-column tiles, or 512-column tiles (wide tiling)
    int split_first; // wide tiling, AG: own items cut into halves in round 0 (see get_work)
    int n_pairs;     // wide tiling: 512-column tiles per row of tiles = ceil(n_tiles / 2)
    int num_comm;
    int push_ahead;             // chunks the pusher's loads run ahead of its stores (1..PUSH_AHEAD)
    int push_parts;             // row slices a 128-row block is pushed in (AG, unicast pushers)
    uint32_t* push_count;       // [(world - 1) * seg_blocks] slice arrivals per (hop, block), zero between launches
    int group_m;
    int is_f16;
    uint32_t epoch;
    int debug_delay_ns;
    unsigned long long* trace;  // optional timeline (see tdist.h), nullptr = off
    const int* expert_ids;      // grouped GEMM: expert (slice of B) of every 128-row block, nullptr = plain
    const int* num_m_blocks;    // grouped GEMM: device count of live 128-row blocks (rest is padding)
    // Row-gathering A operand (PLAIN, one CTA per tile): row r of the logical A is row a_gather[r] of the matrix
    // at a_raw ([a_gather_rows, K], K contiguous); indices >= a_gather_rows read as zeros. With block_src set,
    // the rows of 128-row block b come from rank block_src[b]'s segment of an all-gather in flight: the
    // producer waits until src_flags[block_src[b]] >= src_epoch before it loads them.
    const int* a_gather;
    const char* a_raw;
    int a_gather_rows;
    const int* block_src;
    const uint64_t* src_flags;
    uint64_t src_epoch;
    int src_rank, src_world;    // this rank and the size of the all-gather's group
    // Staged row gather (PLAIN): the rows of block b are copied into gather_dst (the matrix tm_a describes) by the
    // CTAs' own warps, block_ready[b] = epoch says they are complete; the TMA producers wait per block.
    char* gather_dst;
    uint32_t* block_ready;
    uint32_t* gather_counter;   // 4 + blocks words, zero between launches: prologue arrivals, claim cursor, exits, per-block arrivals
    int gather_pro_blocks;      // blocks the prologue stages
    const int* block_rot;       // device scalar: block the schedule starts at (cyclic), nullptr = 0
    // Scattering epilogue (PLAIN, one CTA per tile): row r of the product goes to row c_scatter[r] of c_out.
    const int* c_scatter;
    char* c_out;
    int c_rows;
    WaitCtx wctx;
};

// Block the schedule visits i-th when it starts at block `rot` and wraps around after `live` blocks.
__device__ __forceinline__ int rotate_block(int i, int rot, int live) {
    int b = i + rot;
    return b >= live ? b - live : b;
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

struct TileCoord {
    int seg, m_in_seg, n_tile;
};

// Tiles are ordered segment by segment (a segment = the rows one rank owns), starting at
// `first_seg`; inside a segment, groups of GROUP_M row-tiles sweep all column-tiles so that
// concurrently running CTAs share A rows and B columns in L2.
__host__ __device__ __forceinline__ TileCoord decode_tile(int t, int first_seg, int world, int seg_m_tiles,
                                                 int n_tiles, int GROUP_M) {
    const int per_seg = seg_m_tiles * n_tiles;
    const int si = t / per_seg;
    int r = t - si * per_seg;
    TileCoord c;
    c.seg = first_seg + si;
    if (c.seg >= world) c.seg -= world;
    const int group_span = GROUP_M * n_tiles;
    const int g = r / group_span;
    r -= g * group_span;
    const int first_m = g * GROUP_M;
    const int gsize = min(GROUP_M, seg_m_tiles - first_m);
    c.n_tile = r / gsize;
    c.m_in_seg = first_m + (r - c.n_tile * gsize);
    return c;
}

// One unit of work of a CTA (CTAS == 1) or a CTA pair: `halves` neighbouring 256-column tiles of one row of tiles.
struct Work {
    int seg, m_in_seg, n_tile, halves;
};

// Static schedule: unit u of num_units takes item u + round * num_units. Narrow tilings: an item is one 256-column
// tile. Wide tiling: an item is a pair of neighbouring 256-column tiles (the odd last tile of a row stands alone), and
// two rounds may be cut into halves (single 256-column tiles, half as long):
//  * the last, partial round, when that shortens it (the units that are free first take whole items, the others halves);
//  * the first round of the AG mode when this rank's own segment has fewer items than there are units (`split_first` of
//    them, S = units - own items): instead of sending S units to a peer's segment, whose rows have not arrived yet, the
//    last S own items are cut in two, so that 2 S "early" units finish round 0 in half the time, by when the first
//    remote segment is here. From then on the early units come first in every round.
// Returns false once the unit has nothing left; an item with halves == 0 means "nothing in this round".
template <bool WIDE>
__host__ __device__ __forceinline__ bool get_work(const GemmParams& p, int unit, int num_units, int round, int first_seg, Work& w) {
    if (!WIDE) {
        const int t = unit + round * num_units;
        if (t >= p.num_tiles) return false;
        const TileCoord tc = decode_tile(t, first_seg, p.world, p.seg_m_tiles, p.n_tiles, p.group_m);
        w.seg = tc.seg;
        w.m_in_seg = tc.m_in_seg;
        w.n_tile = tc.n_tile;
        w.halves = 1;
        return true;
    }
    const int S = p.split_first;             // own items cut in two in round 0
    const int E = 2 * S, L = num_units - E;  // early units (a half in round 0) and late units (a whole item)
    int t, half = -1;
    if (S > 0 && round == 0) {
        if (unit < L) {
            t = unit;
        } else {
            t = L + ((unit - L) >> 1);
            half = (unit - L) & 1;
        }
    } else {
        const int base = S > 0 ? L + S : 0;                                  // items taken by round 0
        const int r = S > 0 ? round - 1 : round;
        const int pos = S > 0 ? (unit >= L ? unit - L : E + unit) : unit;    // early units first
        const int rest = p.num_tiles - base;
        const int full_rounds = rest / num_units;
        const int rem = rest - full_rounds * num_units;
        if (r < full_rounds) {
            t = base + r * num_units + pos;
        } else if (r > full_rounds || rem == 0) {
            return false;
        } else if (2 * rem <= E) {
            // the early units alone finish the rest as halves
            if (pos >= 2 * rem) return false;
            t = base + full_rounds * num_units + (pos >> 1);
            half = pos & 1;
        } else if (2 * (rem - E) <= L) {
            // early units take whole items, late units (half an item behind) halves: both end together
            if (pos < E) {
                if (pos >= rem) return false;
                t = base + full_rounds * num_units + pos;
            } else {
                const int j = pos - E;
                if (j >= 2 * (rem - E)) return false;
                t = base + full_rounds * num_units + E + (j >> 1);
                half = j & 1;
            }
        } else {
            if (pos >= rem) return false;
            t = base + full_rounds * num_units + pos;
        }
    }
    const TileCoord tc = decode_tile(t, first_seg, p.world, p.seg_m_tiles, p.n_pairs, p.group_m);
    w.seg = tc.seg;
    w.m_in_seg = tc.m_in_seg;
    w.n_tile = 2 * tc.n_tile;
    w.halves = (w.n_tile + 1 < p.n_tiles) ? 2 : 1;
    if (half >= 0) {
        if (half >= w.halves) {
            w.halves = 0;   // the second half of a row's odd last tile: nothing to do in this round
            return true;
        }
        w.n_tile += half;
        w.halves = 1;
    }
    return true;
}

// TMEM slot (256 accumulator columns) of half `h` of a work item: a wide item takes both slots, narrow items alternate.
__device__ __forceinline__ uint32_t slot_of_half(const Work& w, int h, uint32_t next_narrow) {
    return w.halves == 2 ? static_cast<uint32_t>(h) : next_narrow;
}

// ------------------------------------------------------------------------------------------
// AG pusher: one thread per pusher CTA streams this rank's shard to the peers.
// Work items are (destination, 128-row block, part) triples ordered by how soon the destination's MMA side reaches
// this rank's rows (rank-1 first), dealt round-robin to the pusher CTAs. A block is cut into `push_parts` row slices
// that different pushers send at the same time, so that the first blocks of a segment reach their destination a
// pusher-count sooner than whole blocks would (the GEMM CTAs that have no local tile in the first wave wait for
// exactly those); the pusher whose slice completes a block raises the block's flag at the destination.
// The chunks of consecutive items form ONE stream through the ring (loads PUSH_AHEAD chunks ahead of the stores): an
// item's flag is raised a few chunks into the next item, when waiting for its stores costs nothing.
// ------------------------------------------------------------------------------------------
struct PushItem {
    const char* src;
    char* dst;
    size_t bytes;
    int nchunks;
    int dest, mb, hop;
};
// Item `j` of this pusher (items blockIdx.x + j * num_comm of the global order). False past the end.
__device__ __forceinline__ bool push_item(const GemmParams& p, int j, PushItem& it) {
    const int parts = p.push_parts;
    const int item = static_cast<int>(blockIdx.x) + j * p.num_comm;
    if (item >= (p.world - 1) * p.seg_blocks * parts) return false;
    const int part = item % parts;
    const int mb = (item / parts) % p.seg_blocks;
    const int hop = item / (parts * p.seg_blocks) + 1;
    int dst = p.rank - hop;
    if (dst < 0) dst += p.world;
    const size_t row_bytes = static_cast<size_t>(p.k) * 2;
    const int rows = min(BM, p.m_per_rank - mb * BM);
    const int per = BM / parts;
    const int r0 = min(part * per, rows), r1 = min(r0 + per, rows);
    it.bytes = static_cast<size_t>(r1 - r0) * row_bytes;
    it.src = p.a_own + (static_cast<size_t>(mb) * BM + r0) * row_bytes;
    it.dst = p.a_ws_peer[dst] + (static_cast<size_t>(p.rank) * p.m_per_rank + static_cast<size_t>(mb) * BM + r0) * row_bytes;
    it.nchunks = static_cast<int>((it.bytes + PUSH_CHUNK - 1) / PUSH_CHUNK);
    it.dest = dst;
    it.mb = mb;
    it.hop = hop;
    return true;
}
// The item's rows are complete at the destination (the caller has waited for the stores): order them (async proxy)
// before the release of the flag (generic proxy). With several parts per block the pushers meet on a local counter
// and the last one raises the flag.
__device__ __forceinline__ void push_publish(const GemmParams& p, const PushItem& it) {
    fence_proxy_async();
    uint32_t* flag = p.flags_peer[it.dest] + p.rank * p.seg_blocks + it.mb;
    if (p.push_parts == 1) {
        fence_acq_rel_sys();
        st_release_sys_u32(flag, p.epoch);
        return;
    }
    // gpu scope is enough between the pushers of this GPU (the release half of the add orders this slice's completed
    // writes before it); the pusher that completes the block then releases at system scope on behalf of all of them
    uint32_t* cnt = p.push_count + (it.hop - 1) * p.seg_blocks + it.mb;
    if (atom_add_acq_rel_gpu_u32(cnt, 1) == static_cast<uint32_t>(p.push_parts - 1)) {
        *cnt = 0;   // for the next launch
        fence_acq_rel_sys();
        st_release_sys_u32(flag, p.epoch);
    }
}
__device__ void ag_pusher(const GemmParams& p, uint8_t* smem, uint64_t* bars) {
    if (threadIdx.x != 0) return;
    // An item's flag is raised once FLAG_LAG younger chunks have been stored: a remote bulk store takes several
    // microseconds to complete, and waiting for it any sooner stalls the stream (8 slices per block with a lag of 4
    // chunks ran at 19 GB/s per pusher instead of 36). Up to PENDING finished items wait for their flags.
    constexpr int FLAG_LAG = 12;
    constexpr int PENDING = 4;
    uint32_t full[PUSH_STAGES];
    for (int s = 0; s < PUSH_STAGES; ++s) full[s] = smem_u32(&bars[s]);
    uint32_t it_load = 0, it_store = 0;  // running chunk counters (stage = counter % PUSH_STAGES)
    unsigned long long* tr = (p.trace != nullptr && blockIdx.x < 16) ? p.trace + blockIdx.x * 40 : nullptr;
    int tr_item = 0;
    unsigned long long t_wait = 0, t_publish = 0;   // timeline only: time in completion waits and in flag publication
    if (tr) tr[0] = globaltimer_ns();
    if (p.debug_delay_ns > 0) __nanosleep(p.debug_delay_ns);

    PushItem ld, st;
    PushItem pend[PENDING];       // ring of finished items, oldest at pend_head
    uint32_t pend_at[PENDING];    // it_store right after the item's last store
    int pend_head = 0, pend_n = 0;
    int ld_j = 0, ld_c = 0, st_j = 0, st_c = 0;
    bool ld_ok = push_item(p, 0, ld), st_ok = push_item(p, 0, st);
    while (st_ok) {
        // loads: up to push_ahead chunks ahead of the stores, across item boundaries
        while (ld_ok && it_load - it_store < static_cast<uint32_t>(p.push_ahead)) {
            if (ld_c >= ld.nchunks) {
                ld_ok = push_item(p, ++ld_j, ld);
                ld_c = 0;
                continue;
            }
            const uint32_t s = it_load % PUSH_STAGES;
            // The store that last used this buffer was issued PUSH_STAGES chunks ago; at most
            // PUSH_STAGES - push_ahead - 1 younger stores may still be reading smem.
            if (it_load >= PUSH_STAGES) {
                switch (p.push_ahead) {
                    case 1: bulk_wait_read<PUSH_STAGES - 2>(); break;
                    case 2: bulk_wait_read<PUSH_STAGES - 3>(); break;
                    case 3: bulk_wait_read<PUSH_STAGES - 4>(); break;
                    case 4: bulk_wait_read<PUSH_STAGES - 5>(); break;
                    default: bulk_wait_read<PUSH_STAGES - PUSH_AHEAD - 1>(); break;
                }
            }
            const size_t off = static_cast<size_t>(ld_c) * PUSH_CHUNK;
            const uint32_t sz = static_cast<uint32_t>(min(static_cast<size_t>(PUSH_CHUNK), ld.bytes - off));
            mbar_expect_tx(full[s], sz);
            bulk_load(smem_u32(smem + s * PUSH_CHUNK), ld.src + off, sz, full[s]);
            ++it_load;
            ++ld_c;
        }
        if (st_c < st.nchunks) {
            if (tr && st_c == 0 && tr_item < 18) tr[2 + 2 * tr_item] = globaltimer_ns();
            const uint32_t s = it_store % PUSH_STAGES;
            mbar_wait(full[s], (it_store / PUSH_STAGES) & 1u, p.wctx, 10);
            const size_t off = static_cast<size_t>(st_c) * PUSH_CHUNK;
            const uint32_t sz = static_cast<uint32_t>(min(static_cast<size_t>(PUSH_CHUNK), st.bytes - off));
            bulk_store(st.dst + off, smem_u32(smem + s * PUSH_CHUNK), sz);
            bulk_commit();
            ++it_store;
            ++st_c;
        }
        if (pend_n > 0 && it_store - pend_at[pend_head] >= static_cast<uint32_t>(FLAG_LAG)) {
            // everything but the newest FLAG_LAG groups is complete: so are the stores of every pending item that old
            const unsigned long long w0 = tr ? globaltimer_ns() : 0;
            bulk_wait<FLAG_LAG>();
            const unsigned long long w1 = tr ? globaltimer_ns() : 0;
            while (pend_n > 0 && it_store - pend_at[pend_head] >= static_cast<uint32_t>(FLAG_LAG)) {
                push_publish(p, pend[pend_head]);
                pend_head = (pend_head + 1) % PENDING;
                --pend_n;
            }
            if (tr) {
                t_wait += w1 - w0;
                t_publish += globaltimer_ns() - w1;
            }
        }
        if (st_c >= st.nchunks) {
            // the item's last store is issued (or it had none: a slice past the end of a ragged block)
            if (pend_n == PENDING) {
                bulk_wait<0>();
                while (pend_n > 0) {
                    push_publish(p, pend[pend_head]);
                    pend_head = (pend_head + 1) % PENDING;
                    --pend_n;
                }
            }
            if (tr && tr_item < 18) tr[3 + 2 * tr_item] = globaltimer_ns();
            ++tr_item;
            const int slot = (pend_head + pend_n) % PENDING;
            pend[slot] = st;
            pend_at[slot] = it_store;
            ++pend_n;
            st_ok = push_item(p, ++st_j, st);
            st_c = 0;
        }
    }
    if (pend_n > 0) {
        bulk_wait<0>();
        while (pend_n > 0) {
            push_publish(p, pend[pend_head]);
            pend_head = (pend_head + 1) % PENDING;
            --pend_n;
        }
    }
    if (tr) {
        tr[1] = globaltimer_ns();
        tr[38] = t_wait;
        tr[39] = t_publish;
    }
}

// ------------------------------------------------------------------------------------------
// AG pusher through the NVSwitch multicast engine: the workspace is bound to a multicast object, so ONE
// multimem.st per 16 bytes lands in every rank's workspace. A pusher CTA owns whole 128-row blocks: thread
// 0 streams the block into shared memory with bulk loads, all threads replay it from shared memory as
// multimem.st, then one flag per peer is raised. A seventh of the stores of the unicast pusher, hence
// far fewer CTAs taken from the GEMM.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void multimem_st_v4(char* mc_addr, const uint4& v) {
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}
__device__ void ag_pusher_nvls(const GemmParams& p, uint8_t* smem, uint64_t* bars) {
    const int tid = static_cast<int>(threadIdx.x);
    const size_t row_bytes = static_cast<size_t>(p.k) * 2;
    uint32_t it_load = 0, it_use = 0;  // running chunk counters, the same in every thread
    for (int mb = static_cast<int>(blockIdx.x); mb < p.seg_blocks; mb += p.num_comm) {
        const int rows = min(BM, p.m_per_rank - mb * BM);
        const size_t bytes = static_cast<size_t>(rows) * row_bytes;
        const char* src = p.a_own + static_cast<size_t>(mb) * BM * row_bytes;
        char* out = p.a_ws_mc + (static_cast<size_t>(p.rank) * p.m_per_rank + static_cast<size_t>(mb) * BM) * row_bytes;
        const int nchunks = static_cast<int>((bytes + PUSH_CHUNK - 1) / PUSH_CHUNK);
        if (p.debug_delay_ns > 0) __nanosleep(p.debug_delay_ns);
        for (int c = 0; c < nchunks + PUSH_AHEAD; ++c) {
            if (c < nchunks) {
                // slot it_load % PUSH_STAGES was last read as chunk it_load - PUSH_STAGES, i.e. before the
                // __syncthreads of an earlier iteration (PUSH_STAGES - 1 >= PUSH_AHEAD)
                if (tid == 0) {
                    const uint32_t s = it_load % PUSH_STAGES;
                    const size_t off = static_cast<size_t>(c) * PUSH_CHUNK;
                    const uint32_t sz = static_cast<uint32_t>(min(static_cast<size_t>(PUSH_CHUNK), bytes - off));
                    mbar_expect_tx(smem_u32(&bars[s]), sz);
                    bulk_load(smem_u32(smem + s * PUSH_CHUNK), src + off, sz, smem_u32(&bars[s]));
                }
                ++it_load;
            }
            if (c >= PUSH_AHEAD) {
                const int cs = c - PUSH_AHEAD;
                const uint32_t s = it_use % PUSH_STAGES;
                mbar_wait(smem_u32(&bars[s]), (it_use / PUSH_STAGES) & 1u, p.wctx, 11);
                const size_t off = static_cast<size_t>(cs) * PUSH_CHUNK;
                const uint32_t sz = static_cast<uint32_t>(min(static_cast<size_t>(PUSH_CHUNK), bytes - off));
                const uint8_t* buf = smem + s * PUSH_CHUNK;
                for (uint32_t i = static_cast<uint32_t>(tid) * 16u; i < sz; i += THREADS * 16u)
                    multimem_st_v4(out + off + i, *reinterpret_cast<const uint4*>(buf + i));
                ++it_use;
                __syncthreads();  // the slot is fully replayed before thread 0 may refill it
            }
        }
        // every thread's stores were issued before the barrier above; thread 0's fence orders them
        // (cumulatively) before the flags
        if (tid == 0) {
            fence_acq_rel_sys();
            for (int r = 0; r < p.world; ++r)
                if (r != p.rank) st_release_sys_u32(p.flags_peer[r] + p.rank * p.seg_blocks + mb, p.epoch);
        }
    }
}

// ------------------------------------------------------------------------------------------
// Staged row gather (grouped GEMM over rows picked by index): the rows of one 128-row block after the other are copied
// into the staging matrix the TMA producers read, in the order the GEMM visits the blocks, with one flag per block.
// The first wave's blocks are copied by all threads of the grid before the roles split; the others by the epilogue
// warps while they wait for accumulators. With block_src the rows of a block come from another rank's segment of an
// all-gather that may still be in flight: a group is copied only once that rank's arrival flag is up, so the MMAs of
// the blocks that are already here run while the later segments are still on the wire. Plays the role of the
// reference's `kernel_consumer_m_parallel_scatter_group_gemm` gathering A rows by `sorted_token_ids` behind a per-rank
// barrier (kernels/nvidia/allgather_group_gemm.py:229-314).
// ------------------------------------------------------------------------------------------
// words of the gather_counter array
enum : int { kGatherPrologue = 0, kGatherCursor = 1, kGatherExits = 2, kGatherArrive = 4 };
// Blocks (in schedule order) that every CTA of the grid helps to stage before the MMAs start: what the first wave of
// tiles touches, cut short at the first block whose rows belong to another rank's segment (those may not be here yet).
__device__ __forceinline__ int gather_prologue_blocks(const GemmParams& p, int live, int rot) {
    int pro = min(live, p.gather_pro_blocks);
    if (p.block_src != nullptr) {
        for (int i = 0; i < pro; ++i) {
            const int src = p.block_src[rotate_block(i, rot, live)];
            if (src != p.src_rank && src >= 0 && src < p.src_world) return i;
        }
    }
    return pro;
}

// All CTAs, all threads: copy the rows of the first `pro` blocks (a warp per row, rows dealt round-robin over the grid);
// the last CTA to finish publishes their flags.
__device__ void gather_prologue(const GemmParams& p, int pro, int live, int rot) {
    const int tid = static_cast<int>(threadIdx.x);
    const int warp = tid >> 5, lane = tid & 31;
    const int nwarps = static_cast<int>(blockDim.x) >> 5;
    const size_t row_bytes = static_cast<size_t>(p.k) * 2;
    for (int g = static_cast<int>(blockIdx.x) * nwarps + warp; g < pro * BM; g += static_cast<int>(gridDim.x) * nwarps) {
        const int row = rotate_block(g / BM, rot, live) * BM + (g % BM);
        if (row >= p.m_per_rank) continue;
        const int idx = p.a_gather[row];
        if (idx < 0 || idx >= p.a_gather_rows) continue;   // padding row: its product is never used
        const char* src = p.a_raw + static_cast<size_t>(idx) * row_bytes;
        char* dst = p.gather_dst + static_cast<size_t>(row) * row_bytes;
        for (size_t off = static_cast<size_t>(lane) * 16; off < row_bytes; off += 8 * 512) {
            uint4 q[8];
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (off + u * 512 < row_bytes) q[u] = *reinterpret_cast<const uint4*>(src + off + u * 512);
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (off + u * 512 < row_bytes) *reinterpret_cast<uint4*>(dst + off + u * 512) = q[u];
        }
    }
    // the CTA barrier orders every thread's stores before thread 0's arrival (gpu scope, acq_rel): the last CTA to
    // arrive has every CTA's rows behind it when it raises the flags
    __syncthreads();
    if (tid == 0) {
        const uint32_t old = atom_add_acq_rel_gpu_u32(p.gather_counter + kGatherPrologue, 1);
        if (old == gridDim.x - 1) {
            p.gather_counter[kGatherPrologue] = 0;
            fence_acq_rel_gpu();
            for (int i = 0; i < pro; ++i) st_release_gpu_u32(p.block_ready + rotate_block(i, rot, live), p.epoch);
        }
    }
}

// The remaining blocks are staged by the epilogue warps of the GEMM CTAs in the time they would otherwise spend waiting
// for an accumulator: a warp claims the next 16-row group (in the order the GEMM visits the blocks) from a grid-wide
// cursor, copies it one row per step, looking at its accumulator barrier between rows, and the warp that completes a
// block's last group raises the block's flag. No CTA is taken away from the MMAs and the copy bandwidth grows with the
// grid (4 warps x 148 CTAs).
constexpr int GATHER_SUB = 16;              // rows per claimed item
constexpr int GATHER_SUBS = BM / GATHER_SUB;
struct GatherCursor {
    int item;   // claimed group in schedule order (-1: none claimed yet)
    int row;    // next row of the group
};

// One step of a warp's share: claim a group if it holds none, then copy at most one row. False once the cursor has run
// past the last block (nothing left for this warp). A group whose rows belong to an all-gather segment that has not
// arrived yet is kept and retried on the next step.
__device__ __forceinline__ bool gather_step(const GemmParams& p, GatherCursor& g, int pro, int live, int rot, int lane) {
    if (g.item < 0) {
        int it = 0;
        if (lane == 0) it = static_cast<int>(atomicAdd(p.gather_counter + kGatherCursor, 1u)) + pro * GATHER_SUBS;
        g.item = __shfl_sync(0xffffffffu, it, 0);
        g.row = 0;
    }
    if (g.item >= live * GATHER_SUBS) return false;
    const int b = rotate_block(g.item / GATHER_SUBS, rot, live);
    if (g.row == 0 && p.block_src != nullptr) {
        const int srcr = p.block_src[b];
        if (srcr != p.src_rank && srcr >= 0 && srcr < p.src_world) {
            // every lane acquires: its own loads below are ordered after the segment's arrival
            const bool here = static_cast<long long>(ld_acquire_sys_u64(p.src_flags + srcr)) >= static_cast<long long>(p.src_epoch);
            if (!__all_sync(0xffffffffu, here)) return true;
        }
    }
    const int row = b * BM + (g.item % GATHER_SUBS) * GATHER_SUB + g.row;
    if (row < p.m_per_rank) {
        const int idx = p.a_gather[row];
        if (idx >= 0 && idx < p.a_gather_rows) {   // else a padding row: its product is never used
            const size_t row_bytes = static_cast<size_t>(p.k) * 2;
            const char* src = p.a_raw + static_cast<size_t>(idx) * row_bytes;
            char* dst = p.gather_dst + static_cast<size_t>(row) * row_bytes;
            for (size_t off = static_cast<size_t>(lane) * 16; off < row_bytes; off += 8 * 512) {
                uint4 q[8];
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (off + u * 512 < row_bytes) q[u] = *reinterpret_cast<const uint4*>(src + off + u * 512);
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (off + u * 512 < row_bytes) *reinterpret_cast<uint4*>(dst + off + u * 512) = q[u];
            }
        }
    }
    if (++g.row == GATHER_SUB) {
        // the warp barrier orders every lane's stores before lane 0's arrival (gpu scope, acq_rel); the warp that brings
        // the block's count to GATHER_SUBS therefore has all of the block's rows behind it when it raises the flag
        __syncwarp();
        if (lane == 0) {
            fence_acq_rel_gpu();
            const uint32_t old = atom_add_acq_rel_gpu_u32(p.gather_counter + kGatherArrive + b, 1);
            if (old == GATHER_SUBS - 1) {
                p.gather_counter[kGatherArrive + b] = 0;
                st_release_gpu_u32(p.block_ready + b, p.epoch);
            }
        }
        g.item = -1;
    }
    return true;
}

// The epilogue's wait for an accumulator, spent on the row staging while there is any.
__device__ __forceinline__ void gather_while_waiting(const GemmParams& p, GatherCursor& g, int pro, int live, int rot, int lane,
                                                     uint32_t bar, uint32_t parity, int where) {
    uint64_t t0 = 0;
    uint32_t spins = 0;
    const uint64_t limit = p.wctx.timeout_ns ? p.wctx.timeout_ns : kDefaultTimeoutNs;
    while (true) {
        // all lanes take the same branch: the barrier's state is read by lane 0 only
        const bool done = __shfl_sync(0xffffffffu, lane == 0 ? mbar_test_wait(bar, parity) : false, 0);
        if (done) break;
        if (!gather_step(p, g, pro, live, rot, lane)) break;
        if ((++spins & 63u) == 0) {
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit || aborted(p.wctx)) break;   // the bounded wait below reports it
        }
    }
    mbar_wait(bar, parity, p.wctx, where);
}

// A warp leaves the tile loop: the group it still holds is finished first (a producer may be waiting for it).
__device__ __forceinline__ void gather_finish(const GemmParams& p, GatherCursor& g, int pro, int live, int rot, int lane) {
    if (g.item < 0) return;
    const uint64_t limit = p.wctx.timeout_ns ? p.wctx.timeout_ns : kDefaultTimeoutNs;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (g.item >= 0 && g.item < live * GATHER_SUBS) {
        gather_step(p, g, pro, live, rot, lane);
        if ((++spins & 63u) == 0 && (aborted(p.wctx) || globaltimer_ns() - t0 > limit)) {
            if (lane == 0) report_timeout(p.wctx, kStatusFlagTimeout, -1, g.item, p.src_epoch, -1, 8);
            return;
        }
    }
}

// ------------------------------------------------------------------------------------------
// RS reduce: sum the `world` partial copies of one owned tile in fp32, write bf16/f16.
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void rs_reduce_tile(const GemmParams& p, int block, int n_tile) {
    const int row0 = block * BM;
    const int col0 = n_tile * BN;
    const int rows = min(BM, p.m_per_rank - row0);
    const int cols = min(BN, p.n - col0);
    const int vec_per_row = cols / 8;  // N % 8 == 0 is checked on the host
    const int nvec = rows * vec_per_row;
    const size_t slot = static_cast<size_t>(p.m_per_rank) * p.n;  // elements per source slot
    for (int v = static_cast<int>(threadIdx.x); v < nvec; v += THREADS) {
        const int r = v / vec_per_row;
        const int cv = v - r * vec_per_row;
        const size_t off = static_cast<size_t>(row0 + r) * p.n + col0 + cv * 8;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        // all sources' loads are issued before the first add: one dependent load per source would leave
        // the tail latency-bound (it reads world x the output's size)
        uint4 qs[kMaxRanks];
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s)
            if (s < p.world) qs[s] = *reinterpret_cast<const uint4*>(p.stage_local + (s * slot + off) * 2);
#pragma unroll
        for (int s = 0; s < kMaxRanks; ++s) {
            if (s >= p.world) break;
            const uint4 q = qs[s];
            const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (p.is_f16) {
                    const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
                    const float2 f = __half22float2(h);
                    acc[2 * i] += f.x;
                    acc[2 * i + 1] += f.y;
                } else {
                    acc[2 * i] += __uint_as_float(w[i] << 16);
                    acc[2 * i + 1] += __uint_as_float(w[i] & 0xffff0000u);
                }
            }
        }
        uint4 o;
        uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (p.is_f16) {
                const __half2 h = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
                ow[i] = *reinterpret_cast<const uint32_t*>(&h);
            } else {
                ow[i] = pack_bf16x2(acc[2 * i], acc[2 * i + 1]);
            }
        }
        *reinterpret_cast<uint4*>(static_cast<char*>(p.rs_out) + off * 2) = o;
    }
}

// GATHER (PLAIN, one CTA per tile): four extra warps (threads 192..319) copy the A rows by index with cp.async,
// warp 0 then only issues the TMA loads of B.
constexpr int GATHER_THREADS = THREADS + 128;
template <int MODE, int CTAS, bool GATHER = false, bool WIDE = false>
__global__ void __launch_bounds__(GATHER ? GATHER_THREADS : THREADS, 1) gemm_sm100_kernel(const __grid_constant__ GemmParams p) {
    using T = Tiling<CTAS, WIDE>;
    static_assert(!(GATHER && WIDE), "the row-gathering producer feeds narrow tiles");
    constexpr int STAGES = T::STAGES;
    constexpr int STAGE_BYTES = T::STAGE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_TILES);
    // barrier slots: [0,S) full, [S,2S) empty, [2S,2S+2) tmem_full, [2S+2,2S+4) tmem_empty
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * MAX_STAGES + 4);

    const int warp = static_cast<int>(threadIdx.x) >> 5;
    const int lane = static_cast<int>(threadIdx.x) & 31;

    // ---------------- pusher CTAs (AG only; whole clusters when CTAS == 2) ----------------
    if (MODE == TDIST_GEMM_AG && static_cast<int>(blockIdx.x) < p.num_comm) {
        if (threadIdx.x == 0) {
            for (int s = 0; s < PUSH_STAGES; ++s) mbar_init(smem_u32(&bars[s]), 1);
            fence_mbar_init();
        }
        __syncthreads();
        if (p.a_ws_mc != nullptr) ag_pusher_nvls(p, smem, bars);
        else ag_pusher(p, smem, bars);
        return;
    }

    // ---------------- staged row gather (grouped GEMM): every CTA copies its share of the first wave's rows ----------------
    constexpr bool STAGED = MODE == TDIST_GEMM_PLAIN && CTAS == 1 && !GATHER;
    int gather_live = 0, gather_rot = 0, gather_pro = 0;
    if (STAGED && p.gather_dst != nullptr) {
        gather_live = min(p.seg_blocks, p.num_m_blocks ? *p.num_m_blocks : p.seg_blocks);
        gather_rot = p.block_rot ? min(max(*p.block_rot, 0), max(gather_live - 1, 0)) : 0;
        gather_pro = gather_prologue_blocks(p, gather_live, gather_rot);
        if (gather_pro > 0) gather_prologue(p, gather_pro, gather_live, gather_rot);
    }

    // `unit` = the CTA (CTAS == 1) or the CTA pair (CTAS == 2) that owns a tile.
    const int cta = static_cast<int>(blockIdx.x) - p.num_comm;
    const int num_cta = static_cast<int>(gridDim.x) - p.num_comm;
    const int unit = cta / CTAS;
    const int num_units = num_cta / CTAS;
    const int cta_rank = (CTAS == 2) ? static_cast<int>(cluster_ctarank()) : 0;
    const int first_seg = (MODE == TDIST_GEMM_RS) ? (p.rank + 1) % p.world : p.rank;

    // shared-memory addresses of the barriers (computed, not tabulated, to stay in registers)
    const uint32_t bars_u32 = smem_u32(bars);
    struct {
        uint32_t base;
        __device__ uint32_t operator()(int slot) const { return base + static_cast<uint32_t>(slot) * 8u; }
    } bar{bars_u32};
#define bar_full(s) bar(s)
#define bar_empty(s) bar(MAX_STAGES + (s))
#define bar_tfull(b) bar(2 * MAX_STAGES + (b))
#define bar_tempty(b) bar(2 * MAX_STAGES + 2 + (b))

    if (threadIdx.x == 0) {
        prefetch_tensormap(&p.tm_a);
        prefetch_tensormap(&p.tm_b);
        if (MODE == TDIST_GEMM_AG) prefetch_tensormap(&p.tm_a_own);
        for (int s = 0; s < STAGES; ++s) {
            // gather mode: the 128 producer threads each arrive once their cp.async rows have landed, plus warp 0's expect_tx
            mbar_init(bar_full(s), GATHER ? 129 : 1);
            mbar_init(bar_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_tfull(b), 1);
            mbar_init(bar_tempty(b), 4 * CTAS);  // one arrival per epilogue warp of every CTA
        }
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc<CTAS>(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish<CTAS>();
    }
    tc_fence_before();
    if (CTAS == 2) {
        // the peer CTA signals this CTA's barriers: they must exist cluster-wide before any use
        cluster_arrive();
        cluster_wait();
    } else {
        __syncthreads();
    }
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    if (GATHER && warp >= THREADS / 32) {
        // ===================== gathering producers: A rows by index with cp.async ==========
        // Eight consecutive threads copy the eight 16-byte chunks of one row and K block (one full 128-byte line per
        // row, four rows per warp instruction); thread t does chunk t % 8 of rows t / 8 + 16 j, j < 8, written in the
        // 128-byte-swizzled layout the MMA descriptors expect. Completion is lagged: before a thread waits for the next free slot it
        // makes the arrivals of every stage that is more than LAG copy groups old (cp.async.wait_group), after a proxy
        // fence that makes the generic-proxy writes visible to the tensor core's async-proxy reads. The arrival of
        // stage i therefore never waits for the MMA of stage i - 1 to retire: the MMA queue stays one stage ahead.
        constexpr int LAG = 2;
        const int r = static_cast<int>(threadIdx.x) - THREADS;
        uint32_t it = 0, signaled = 0;
        const int live_blocks = p.num_m_blocks ? *p.num_m_blocks : 0x7fffffff;
        auto drain = [&]() {
            cp_async_wait<0>();
            fence_proxy_async();
            while (signaled < it) {
                mbar_arrive(bar_full(signaled % STAGES));
                ++signaled;
            }
        };
        for (int t = unit; t < p.num_tiles; t += num_units) {
            const TileCoord tc = decode_tile(t, first_seg, p.world, p.seg_m_tiles, p.n_tiles, p.group_m);
            const int block = tc.m_in_seg;
            if (block >= live_blocks) continue;
            if (p.block_src != nullptr) {
                const int src = p.block_src[block];
                if (src != p.src_rank && src >= 0 && src < p.src_world) {
                    drain();  // do not leave the MMA side waiting for stages that are already in shared memory
                    if (lane == 0) signal_wait_until(p.src_flags + src, kCmpGe, p.src_epoch, p.wctx, src, 8);
                    __syncwarp();
                }
            }
            const int c = r & 7, r0 = r >> 3;
            const char* rowp[8];
            unsigned valid = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int row = block * BM + r0 + 16 * j;
                const int idx = row < p.m_per_rank ? p.a_gather[row] : p.a_gather_rows;
                const bool ok = idx >= 0 && idx < p.a_gather_rows;
                valid |= ok ? (1u << j) : 0u;
                rowp[j] = p.a_raw + (ok ? static_cast<size_t>(idx) * p.k * 2 : 0) + c * 16;
            }
            for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                const uint32_t s = it % STAGES;
                while (it - signaled > LAG) {   // `it` groups issued so far: all but the newest LAG have landed after this wait
                    cp_async_wait<LAG>();
                    fence_proxy_async();
                    mbar_arrive(bar_full(signaled % STAGES));
                    ++signaled;
                }
                mbar_wait(bar_empty(s), ((it / STAGES) & 1u) ^ 1u, p.wctx, 2);
                const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                const bool in_k = kb * BK + c * 8 < p.k;  // K % 8 == 0: a chunk is whole or absent
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int rr = r0 + 16 * j;
                    const int nbytes = (in_k && ((valid >> j) & 1u)) ? 16 : 0;
                    cp_async16(sa + rr * 128 + ((c ^ (rr & 7)) << 4), rowp[j] + (nbytes ? static_cast<size_t>(kb) * BK * 2 : 0), nbytes);
                }
                cp_async_commit();
            }
        }
        drain();
        __syncwarp();
    } else if (GATHER && warp == 0) {
        // ===================== B-only TMA producer of the gather variant ==========
        if (lane == 0) {
            uint32_t it = 0;
            const int live_blocks = p.num_m_blocks ? *p.num_m_blocks : 0x7fffffff;
            for (int t = unit; t < p.num_tiles; t += num_units) {
                const TileCoord tc = decode_tile(t, first_seg, p.world, p.seg_m_tiles, p.n_tiles, p.group_m);
                const int block = tc.m_in_seg;
                if (block >= live_blocks) continue;
                const int bz = p.expert_ids ? p.expert_ids[block] : 0;
                const int col = tc.n_tile * BN;
                for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    mbar_wait(bar_empty(s), ((it / STAGES) & 1u) ^ 1u, p.wctx, 2);
                    mbar_expect_tx(bar_full(s), T::B_BYTES);
                    tma_load_3d(smem_u32(smem + s * STAGE_BYTES) + A_BYTES, &p.tm_b, bar_full(s), kb * BK, col, bz);
                }
            }
        }
        __syncwarp();
    } else if (warp == 0) {
        // ===================== TMA producer (every CTA loads its own A rows and B rows) ==========
        if (lane == 0) {
            uint32_t it = 0;
            unsigned long long* tr = (p.trace != nullptr && cta < 64) ? p.trace + 1024 + cta * 4 : nullptr;
            unsigned long long waited = 0, blocked = 0;
            if (tr) tr[0] = globaltimer_ns();
            const int live_blocks = p.num_m_blocks ? *p.num_m_blocks : 0x7fffffff;
            const int block_rot = p.block_rot ? min(max(*p.block_rot, 0), max(min(live_blocks, p.seg_m_tiles) - 1, 0)) : 0;
            Work tc;
            for (int round = 0; get_work<WIDE>(p, unit, num_units, round, first_seg, tc); ++round) {
                if (tc.halves == 0 || tc.m_in_seg * CTAS >= live_blocks) continue;  // padding tile of a grouped GEMM: every role skips it
                int block = tc.m_in_seg * CTAS + cta_rank;  // 128-row block inside the segment
                if (MODE == TDIST_GEMM_PLAIN && CTAS == 1 && p.block_rot != nullptr)
                    block = rotate_block(block, block_rot, min(live_blocks, p.seg_m_tiles));
                const int bz = p.expert_ids ? p.expert_ids[block] : 0;
                const CUtensorMap* am = &p.tm_a;
                int az = tc.seg;
                if (MODE == TDIST_GEMM_PLAIN && CTAS == 1 && p.block_ready != nullptr) {
                    // this block's rows have been staged (generic-proxy stores, read next by TMA)
                    wait_flag_ge_gpu(p.block_ready + block, p.epoch, p.wctx, -1, block, 7);
                    fence_proxy_async();
                }
                if (MODE == TDIST_GEMM_AG) {
                    if (tc.seg == p.rank) {
                        am = &p.tm_a_own;
                        az = 0;
                    } else if (block < p.seg_blocks) {
                        const unsigned long long w0 = tr ? globaltimer_ns() : 0;
                        wait_flag_ge_sys(p.flags + tc.seg * p.seg_blocks + block, p.epoch, p.wctx, tc.seg, block, 1);
                        fence_proxy_async();
                        if (tr) {
                            const unsigned long long dt = globaltimer_ns() - w0;
                            waited += dt;
                            blocked += dt > 2000 ? 1 : 0;
                        }
                    }
                }
                const int row = block * BM;
                const int col = tc.n_tile * BN + cta_rank * T::B_ROWS;
                const uint32_t stage_tx = A_BYTES + tc.halves * T::B_BYTES;
                for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    mbar_wait(bar_empty(s), ((it / STAGES) & 1u) ^ 1u, p.wctx, 2);
                    const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                    if (CTAS == 1) {
                        mbar_expect_tx(bar_full(s), STAGE_BYTES);
                        tma_load_3d(sa, am, bar_full(s), kb * BK, row, az);
                        tma_load_3d(sa + A_BYTES, &p.tm_b, bar_full(s), kb * BK, col, bz);
                    } else {
                        // both CTAs' bytes are counted on the leader's barrier
                        if (cta_rank == 0) mbar_expect_tx(bar_full(s), 2 * stage_tx);
                        const uint32_t leader_full = mapa_u32(bar_full(s), 0);
                        tma_load_3d_pair(sa, am, leader_full, kb * BK, row, az);
                        tma_load_3d_pair(sa + A_BYTES, &p.tm_b, leader_full, kb * BK, col, bz);
                        if (WIDE && tc.halves == 2)
                            tma_load_3d_pair(sa + A_BYTES + T::B_BYTES, &p.tm_b, leader_full, kb * BK, col + BN, bz);
                    }
                }
            }
            if (tr) {
                tr[1] = globaltimer_ns();
                tr[2] = waited;
                tr[3] = blocked;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ===================== MMA issuer (leader CTA only when CTAS == 2) =====================
        if (lane == 0 && cta_rank == 0) {
            const uint32_t idesc = umma_idesc(p.is_f16 ? 0u : 1u, p.is_f16 ? 0u : 1u, BM * CTAS, BN);
            uint32_t it = 0;
            uint32_t uses0 = 0, uses1 = 0, next_narrow = 0;   // per-slot use counts give the barrier phases
            const int live_blocks = p.num_m_blocks ? *p.num_m_blocks : 0x7fffffff;
            // optional timeline of the issuing thread: cycles in all, cycles waiting for operands, cycles waiting for the
            // epilogue to hand a TMEM slot back, tiles
            unsigned long long* mtr = (p.trace != nullptr && unit < 64) ? p.trace + 1536 + unit * 4 : nullptr;
            long long t_begin = mtr ? clock64() : 0, t_full = 0, t_tempty = 0, n_tiles_done = 0;
            Work tc;
            for (int round = 0; get_work<WIDE>(p, unit, num_units, round, first_seg, tc); ++round) {
                if (tc.halves == 0 || tc.m_in_seg * CTAS >= live_blocks) continue;
                ++n_tiles_done;
                // the four MMAs of one 256-column half over one K block (stage `s`, K block `kb` of the tile)
                auto issue_half = [&](int h, int kb, uint32_t s) {
                    const uint32_t slot = slot_of_half(tc, h, next_narrow);
                    if (kb == 0) {
                        // the epilogue has drained this slot's previous accumulator
                        const long long w0 = mtr ? clock64() : 0;
                        mbar_wait(bar_tempty(slot), ((slot ? uses1 : uses0) & 1u) ^ 1u, p.wctx, 3);
                        if (mtr) t_tempty += clock64() - w0;
                        tc_fence_after();
                    }
                    const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                    const uint32_t d_tmem = tmem_base + slot * BN;
                    const uint64_t adesc = umma_desc_k_sw128(sa);
                    const uint64_t bdesc = umma_desc_k_sw128(sa + A_BYTES + h * T::B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // 16 elements of K = 32 bytes = 2 descriptor address units
                        umma_bf16<CTAS>(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    }
                };
                auto release_stage = [&](uint32_t s) {
                    // frees the smem stage (in both CTAs) when the MMAs retire
                    if (CTAS == 1) umma_commit(bar_empty(s));
                    else umma_commit_pair(bar_empty(s), 3);
                };
                for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
                    const uint32_t s = it % STAGES;
                    const long long w0 = mtr ? clock64() : 0;
                    mbar_wait(bar_full(s), (it / STAGES) & 1u, p.wctx, 4);
                    if (mtr) t_full += clock64() - w0;
                    tc_fence_after();
                    if (WIDE && CTAS == 2 && tc.halves == 2 && kb > 0) {
                        // Both halves multiply the same A rows: issue them pairwise per 16-wide K step, the first
                        // filling the A collector, the second reading A from it, so that A crosses the shared-memory
                        // port once per step. (The first K block of a tile keeps the half-by-half order: its second
                        // half may still have to wait for the epilogue.)
                        const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
                        const uint64_t adesc = umma_desc_k_sw128(sa);
                        const uint64_t bdesc0 = umma_desc_k_sw128(sa + A_BYTES);
                        const uint64_t bdesc1 = umma_desc_k_sw128(sa + A_BYTES + T::B_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            umma_bf16_pair_collect<kCollectorFill>(tmem_base, adesc + 2 * k, bdesc0 + 2 * k, idesc, 1u);
                            umma_bf16_pair_collect<kCollectorLastUse>(tmem_base + BN, adesc + 2 * k, bdesc1 + 2 * k, idesc, 1u);
                        }
                    } else {
                        for (int h = 0; h < tc.halves; ++h) issue_half(h, kb, s);
                    }
                    release_stage(s);
                }
                for (int h = 0; h < tc.halves; ++h) {
                    const uint32_t slot = slot_of_half(tc, h, next_narrow);
                    if (CTAS == 1) umma_commit(bar_tfull(slot));  // accumulator ready
                    else umma_commit_pair(bar_tfull(slot), 3);
                    if (slot) ++uses1;
                    else ++uses0;
                }
                if (tc.halves == 1) next_narrow ^= 1u;
            }
            if (mtr) {
                mtr[0] = static_cast<unsigned long long>(clock64() - t_begin);
                mtr[1] = static_cast<unsigned long long>(t_full);
                mtr[2] = static_cast<unsigned long long>(t_tempty);
                mtr[3] = static_cast<unsigned long long>(n_tiles_done);
            }
        }
        __syncwarp();
    } else {
        // ===================== epilogue (warps 2..5) =====================
        const int q = warp & 3;                 // TMEM lane quadrant this warp may read
        const int row_in_tile = q * 32 + lane;
        const bool issuer = (warp == 2 && lane == 0);
        uint8_t* cstage = smem + PIPE_BYTES;
        uint32_t uses0 = 0, uses1 = 0, next_narrow = 0;   // same slot bookkeeping as the MMA issuer
        // RS: the flag of a 256-column partial tile may only be raised once its stores have completed at the owner.
        // Waiting for that right after issuing them would stall the epilogue for an NVLink round trip per tile, so
        // the flag of a tile is published two tiles later, when `cp.async.bulk.wait_group 8` (all but the newest
        // eight groups, i.e. the two younger tiles' four chunks each, are complete) costs nothing.
        uint32_t* pend0 = nullptr;   // older
        uint32_t* pend1 = nullptr;   // younger
        const int live_blocks = p.num_m_blocks ? *p.num_m_blocks : 0x7fffffff;
        const int block_rot = p.block_rot ? min(max(*p.block_rot, 0), max(min(live_blocks, p.seg_m_tiles) - 1, 0)) : 0;
        const bool scatter = MODE == TDIST_GEMM_PLAIN && CTAS == 1 && p.c_scatter != nullptr;
        GatherCursor gcur{-1, 0};
        Work tc;
        for (int round = 0; get_work<WIDE>(p, unit, num_units, round, first_seg, tc); ++round) {
            if (tc.halves == 0 || tc.m_in_seg * CTAS >= live_blocks) continue;
            const CUtensorMap* cm = (MODE == TDIST_GEMM_RS) ? &p.tm_c[tc.seg] : &p.tm_c[0];
            const int cz = (MODE == TDIST_GEMM_RS) ? p.rank : tc.seg;
            int block = tc.m_in_seg * CTAS + cta_rank;
            if (MODE == TDIST_GEMM_PLAIN && CTAS == 1 && p.block_rot != nullptr)
                block = rotate_block(block, block_rot, min(live_blocks, p.seg_m_tiles));
            const int row = block * BM;
            // scattering epilogue: the output row of this thread's row of the tile (-1 = padding, dropped)
            int out_row = -1;
            if (scatter && row + row_in_tile < p.m_per_rank) {
                out_row = p.c_scatter[row + row_in_tile];
                if (out_row >= p.c_rows) out_row = -1;
            }
            for (int h = 0; h < tc.halves; ++h) {
                const uint32_t buf = slot_of_half(tc, h, next_narrow);
                if (STAGED && p.gather_dst != nullptr)
                    gather_while_waiting(p, gcur, gather_pro, gather_live, gather_rot, lane, bar_tfull(buf), (buf ? uses1 : uses0) & 1u, 5);
                else
                    mbar_wait(bar_tfull(buf), (buf ? uses1 : uses0) & 1u, p.wctx, 5);
                tc_fence_after();
                if (buf) ++uses1;
                else ++uses0;
                const int col = (tc.n_tile + h) * BN;
                // RS, this rank's own rows: the other ranks' partials of this tile are added here, so wait for them first
                // (they were computed one segment-time ago or earlier; only the MMAs of the next tile run meanwhile)
                const bool reduce_here = MODE == TDIST_GEMM_RS && p.rs_fused && tc.seg == p.rank;
                if (reduce_here && issuer && (pend0 != nullptr || pend1 != nullptr)) {
                    // the last remote tiles' flags must not wait for this rank's own tiles (which store nothing over
                    // NVLink): their owners are about to add them
                    bulk_wait<0>();
                    fence_proxy_async();
                    fence_acq_rel_sys();
                    if (pend0 != nullptr) st_release_sys_u32(pend0, p.epoch);
                    if (pend1 != nullptr) st_release_sys_u32(pend1, p.epoch);
                    pend0 = pend1 = nullptr;
                }
                if (reduce_here && lane < p.world && lane != p.rank && block < p.seg_blocks)
                    wait_flag_ge_sys(p.flags + (block * p.n_tiles + tc.n_tile + h) * p.world + lane, p.epoch, p.wctx, lane, block, 6);
                if (reduce_here) __syncwarp();
#pragma unroll 1
                for (int c = 0; c < BN / EPI_COLS; ++c) {
                    uint32_t r0[32], r1[32];
                    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * BN + c * EPI_COLS;
                    tmem_ld_32x32(taddr, r0);
                    tmem_ld_32x32(taddr + 32, r1);
                    tmem_ld_wait();
                    if (c == BN / EPI_COLS - 1) {
                        // accumulator fully read: hand the TMEM slot back to the MMA issuer
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if (CTAS == 1) mbar_arrive(bar_tempty(buf));
                            else mbar_arrive_cluster(bar_tempty(buf), 0);
                        }
                    }
                    if (reduce_here) {
                        // every thread owns one row of the tile: add the 64 columns of every other rank's partial (fp32)
                        // and store the finished 128 bytes of the output row
                        const int grow = row + row_in_tile;
                        if (grow < p.m_per_rank) {
                            const size_t slot_elems = static_cast<size_t>(p.m_per_rank) * p.n;
                            const size_t off = static_cast<size_t>(grow) * p.n + col + c * EPI_COLS;
                            for (int src = 0; src < p.world; ++src) {
                                if (src == p.rank) continue;
                                const char* sp = p.stage_local + (src * slot_elems + off) * 2;
                                uint4 q[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    if (col + c * EPI_COLS + j * 8 < p.n) q[j] = *reinterpret_cast<const uint4*>(sp + j * 16);
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    if (col + c * EPI_COLS + j * 8 >= p.n) continue;
                                    uint32_t* r = j < 4 ? r0 + 8 * j : r1 + 8 * (j - 4);
                                    const uint32_t w[4] = {q[j].x, q[j].y, q[j].z, q[j].w};
#pragma unroll
                                    for (int i = 0; i < 4; ++i) {
                                        float lo, hi;
                                        if (p.is_f16) {
                                            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
                                            lo = f.x;
                                            hi = f.y;
                                        } else {
                                            lo = __uint_as_float(w[i] << 16);
                                            hi = __uint_as_float(w[i] & 0xffff0000u);
                                        }
                                        r[2 * i] = __float_as_uint(__uint_as_float(r[2 * i]) + lo);
                                        r[2 * i + 1] = __float_as_uint(__uint_as_float(r[2 * i + 1]) + hi);
                                    }
                                }
                            }
                            char* orow = static_cast<char*>(p.rs_out) + off * 2;
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const uint32_t* r = j < 4 ? r0 + 8 * j : r1 + 8 * (j - 4);
                                if (col + c * EPI_COLS + j * 8 < p.n) {
                                    uint4 v;
                                    if (p.is_f16) {
                                        v.x = pack_f16x2(__uint_as_float(r[0]), __uint_as_float(r[1]));
                                        v.y = pack_f16x2(__uint_as_float(r[2]), __uint_as_float(r[3]));
                                        v.z = pack_f16x2(__uint_as_float(r[4]), __uint_as_float(r[5]));
                                        v.w = pack_f16x2(__uint_as_float(r[6]), __uint_as_float(r[7]));
                                    } else {
                                        v.x = pack_bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1]));
                                        v.y = pack_bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3]));
                                        v.z = pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5]));
                                        v.w = pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7]));
                                    }
                                    *reinterpret_cast<uint4*>(orow + j * 16) = v;
                                }
                            }
                        }
                        continue;
                    }
                    if (scatter) {
                        // every thread owns one row of the tile: 64 columns = 128 contiguous bytes of its output row
                        if (out_row >= 0) {
                            char* orow = p.c_out + (static_cast<size_t>(out_row) * p.n + col + c * EPI_COLS) * 2;
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const uint32_t* r = j < 4 ? r0 + 8 * j : r1 + 8 * (j - 4);
                                if (col + c * EPI_COLS + j * 8 < p.n) {
                                    uint4 v;
                                    if (p.is_f16) {
                                        v.x = pack_f16x2(__uint_as_float(r[0]), __uint_as_float(r[1]));
                                        v.y = pack_f16x2(__uint_as_float(r[2]), __uint_as_float(r[3]));
                                        v.z = pack_f16x2(__uint_as_float(r[4]), __uint_as_float(r[5]));
                                        v.w = pack_f16x2(__uint_as_float(r[6]), __uint_as_float(r[7]));
                                    } else {
                                        v.x = pack_bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1]));
                                        v.y = pack_bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3]));
                                        v.z = pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5]));
                                        v.w = pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7]));
                                    }
                                    *reinterpret_cast<uint4*>(orow + j * 16) = v;
                                }
                            }
                        }
                        continue;
                    }
                    uint8_t* cs = cstage + (c & 1) * EPI_BYTES;
                    named_barrier(1, 128);  // the store that last read this buffer has drained
                    uint8_t* rowp = cs + row_in_tile * 128;
                    const int sw = row_in_tile & 7;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint4 v0, v1;
                        if (p.is_f16) {
                            v0.x = pack_f16x2(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
                            v0.y = pack_f16x2(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
                            v0.z = pack_f16x2(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
                            v0.w = pack_f16x2(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
                            v1.x = pack_f16x2(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
                            v1.y = pack_f16x2(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
                            v1.z = pack_f16x2(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
                            v1.w = pack_f16x2(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
                        } else {
                            v0.x = pack_bf16x2(__uint_as_float(r0[8 * j + 0]), __uint_as_float(r0[8 * j + 1]));
                            v0.y = pack_bf16x2(__uint_as_float(r0[8 * j + 2]), __uint_as_float(r0[8 * j + 3]));
                            v0.z = pack_bf16x2(__uint_as_float(r0[8 * j + 4]), __uint_as_float(r0[8 * j + 5]));
                            v0.w = pack_bf16x2(__uint_as_float(r0[8 * j + 6]), __uint_as_float(r0[8 * j + 7]));
                            v1.x = pack_bf16x2(__uint_as_float(r1[8 * j + 0]), __uint_as_float(r1[8 * j + 1]));
                            v1.y = pack_bf16x2(__uint_as_float(r1[8 * j + 2]), __uint_as_float(r1[8 * j + 3]));
                            v1.z = pack_bf16x2(__uint_as_float(r1[8 * j + 4]), __uint_as_float(r1[8 * j + 5]));
                            v1.w = pack_bf16x2(__uint_as_float(r1[8 * j + 6]), __uint_as_float(r1[8 * j + 7]));
                        }
                        // 16-byte chunk index inside the 128-byte row, XOR-swizzled with the row
                        *reinterpret_cast<uint4*>(rowp + ((j ^ sw) << 4)) = v0;
                        *reinterpret_cast<uint4*>(rowp + (((4 + j) ^ sw) << 4)) = v1;
                    }
                    fence_proxy_async_smem();
                    named_barrier(1, 128);  // the staging buffer is complete
                    if (issuer) {
                        if (col + c * EPI_COLS < p.n && row < p.m_per_rank)
                            tma_store_3d(cm, smem_u32(cs), col + c * EPI_COLS, row, cz);
                        // One group per chunk even when the chunk lies outside the matrix and stores
                        // nothing: "at most one group pending" below then always means that the store
                        // which last read the OTHER staging buffer (two chunks back) has drained, and the
                        // flag scheme below can count four groups per 256-column tile.
                        bulk_commit();
                        bulk_wait_read<1>();
                    }
                }
                if (MODE == TDIST_GEMM_RS && issuer && !reduce_here) {
                    if (pend0 != nullptr) {
                        // the tile two back is complete at its owner: order its (async-proxy) writes before the
                        // system-scope release store of its flag
                        bulk_wait<2 * (BN / EPI_COLS)>();
                        fence_proxy_async();
                        fence_acq_rel_sys();
                        st_release_sys_u32(pend0, p.epoch);
                    }
                    pend0 = pend1;
                    pend1 = p.flags_peer[tc.seg] + (block * p.n_tiles + tc.n_tile + h) * p.world + p.rank;
                }
            }
            if (tc.halves == 1) next_narrow ^= 1u;
        }
        if (MODE == TDIST_GEMM_RS && issuer && (pend0 != nullptr || pend1 != nullptr)) {
            bulk_wait<0>();
            fence_proxy_async();
            fence_acq_rel_sys();
            if (pend0 != nullptr) st_release_sys_u32(pend0, p.epoch);
            if (pend1 != nullptr) st_release_sys_u32(pend1, p.epoch);
        }
        if (issuer) bulk_wait<0>();
        __syncwarp();
        if (STAGED && p.gather_dst != nullptr) gather_finish(p, gcur, gather_pro, gather_live, gather_rot, lane);
    }

    tc_fence_before();
    if (CTAS == 2) {
        // neither CTA may free TMEM or exit while its partner can still touch its TMEM, smem or barriers
        cluster_arrive();
        cluster_wait();
    } else {
        __syncthreads();
    }
    if (warp == 1) tmem_dealloc<CTAS>(tmem_base, TMEM_COLS);
    if (STAGED && p.gather_dst != nullptr && threadIdx.x == 0) {
        // every warp of this CTA is past its last claim: the last CTA to leave rewinds the cursor for the next launch
        const uint32_t old = atom_add_acq_rel_gpu_u32(p.gather_counter + kGatherExits, 1);
        if (old == gridDim.x - 1) {
            p.gather_counter[kGatherCursor] = 0;
            p.gather_counter[kGatherExits] = 0;
        }
    }

    if (MODE == TDIST_GEMM_RS && !p.rs_fused) {
        // ===================== reduce the 128-row blocks this rank owns =====================
        const int own_units = p.seg_blocks * p.n_tiles;
        for (int u = cta; u < own_units; u += num_cta) {
            if (warp == 0) {
                if (lane < p.world)
                    wait_flag_ge_sys(p.flags + u * p.world + lane, p.epoch, p.wctx, lane, u, 6);
            }
            __syncthreads();
            rs_reduce_tile(p, u / p.n_tiles, u % p.n_tiles);
        }
    }
}
#undef bar_full
#undef bar_empty
#undef bar_tfull
#undef bar_tempty

}  // namespace tdist

// ============================================================================================
// host side
// ============================================================================================
using namespace tdist;
using tdist_host::fail;

static bool use_pair(const TdistGemmArgs* a) {
    if (a->expert_ids != nullptr || a->a_gather != nullptr || a->c_scatter != nullptr || a->block_rot != nullptr)
        return false;  // one expert / one source / one output row per 128-row block and thread
    if (a->cta_pair == 0) return false;
    if (a->cta_pair > 0) return true;
    return a->m_per_rank > BM;  // a second CTA would only compute padding otherwise
}

// The wide tiling pays when the main loop of a 256 x 512 tile is long against its epilogue, which only
// overlaps the next tile half by half: from K = 4096 on, and only where a row of tiles has a pair to form.
static bool use_wide(const TdistGemmArgs* a) {
    if (!use_pair(a)) return false;
    if (a->cta_pair == 2) return true;
    if (a->cta_pair == 1) return false;
    // RS: the epilogue of a wide tile stores 128 KB per CTA over NVLink with the MMAs of the next tile held up, so the
    // main loop has to be longer still before the wide tile wins
    return a->k >= (a->mode == TDIST_GEMM_RS && a->world > 1 ? 8192 : 4096) && a->n > BN;
}

struct GridPlan {
    int ctas_per_tile, wide, num_comm, num_tiles, grid;
};

template <int CTAS, bool WIDE>
static const void* kernel_for(int mode) {
    switch (mode) {
        case TDIST_GEMM_PLAIN: return reinterpret_cast<const void*>(&gemm_sm100_kernel<TDIST_GEMM_PLAIN, CTAS, false, WIDE>);
        case TDIST_GEMM_AG: return reinterpret_cast<const void*>(&gemm_sm100_kernel<TDIST_GEMM_AG, CTAS, false, WIDE>);
        default: return reinterpret_cast<const void*>(&gemm_sm100_kernel<TDIST_GEMM_RS, CTAS, false, WIDE>);
    }
}
static const void* kernel_of(int ctas, int wide, int mode) {
    if (ctas == 1) return kernel_for<1, false>(mode);
    return wide ? kernel_for<2, true>(mode) : kernel_for<2, false>(mode);
}

// CTAs of this kernel that can be resident at once on the current device (all of them wait on
// one another through flags, so the grid must never exceed this). Cached per device/variant.
static int resident_ctas(int ctas, int wide, int mode) {
    static int cache[64][3][3] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return tdist_host::sm_count();
    int& slot = cache[dev][ctas - 1 + wide][mode];
    if (slot > 0) return slot;
    const void* fn = kernel_of(ctas, wide, mode);
    int result = 0;
    if (cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) == cudaSuccess) {
        if (ctas == 2) {
            cudaLaunchConfig_t cfg;
            memset(&cfg, 0, sizeof(cfg));
            cfg.gridDim = dim3(tdist_host::sm_count() & ~1);
            cfg.blockDim = dim3(THREADS);
            cfg.dynamicSmemBytes = SMEM_BYTES;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, fn, &cfg) == cudaSuccess && clusters > 0) result = clusters * 2;
        } else {
            int per_sm = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, THREADS, SMEM_BYTES) == cudaSuccess && per_sm > 0)
                result = per_sm * tdist_host::sm_count();
        }
    }
    cudaGetLastError();
    if (result <= 0) result = tdist_host::sm_count() & ~(ctas - 1);
    slot = result;
    return result;
}

// Length of the schedule in rounds of 256-column tiles (a round of wide items counts two): what get_work() deals out.
static int schedule_cost(int items, int units, int wide) {
    if (!wide) return (items + units - 1) / units;
    const int full = items / units, rem = items - full * units;
    return 2 * full + (rem == 0 ? 0 : (2 * rem <= units ? 1 : 2));
}

// AG mode, several ranks: how many pusher CTAs and which pair tiling. A model of the run, not a table:
//   the GEMM side needs  t_gemm = (schedule length in 256-column tiles) x (time of such a tile on a CTA pair);
//   the pushers need     t_push = bytes / min(pushers x 34 GB/s, 600 GB/s)   (one unicast pusher CTA moves 36-40 GB/s
//                        alone and a little less beside a running GEMM; NVLink saturates near 600 GB/s of payload);
//   after the last rows arrive the tiles of one segment are still to do: t_tail = their rounds x tile time;
//   the run takes max(t_gemm, t_push + t_tail).
// Long-K problems are bound by t_gemm and want few pushers and the wide tiling (3 % faster per FLOP at K = 12288);
// short-K problems are bound by the all-gather and want many pushers and small tiles, which shorten the tail.
// Measured on 8 x B200, m8192 n49152 k12288: wide 4/6/8/10 pushers 1.72/1.19/0.97/1.02 ms (model 8), 256 x 256 tiles
// 1.29/1.09/1.00/1.24 ms; on 4 x B200, m8192 n11008 k4096: 16 pushers 158 (256 x 256) / 171 us (wide), 8 pushers
// 226 / 223 us, 24 pushers 190 / 206 us.
static void plan_ag(const TdistGemmArgs* a, int sms, int n_tiles, GridPlan& g) {
    const bool nvls = a->a_ws_mc != nullptr;
    const double push_bytes = static_cast<double>(nvls ? 1 : a->world - 1) * a->m_per_rank * a->k * 2.0;
    const double per_pusher = nvls ? 33e9 : 34e9, link_cap = 600e9;
    const int step = g.ctas_per_tile;
    const int seg_m_tiles = (a->m_per_rank + BM * g.ctas_per_tile - 1) / (BM * g.ctas_per_tile);
    const int nc_lo = a->num_comm_sms > 0 ? a->num_comm_sms : step;
    // never more pushers than there are (destination, 128-row block) items to push
    const int seg_blocks = (a->m_per_rank + BM - 1) / BM;
    int nc_cap = (a->world - 1) * seg_blocks;
    nc_cap = (nc_cap + step - 1) / step * step;
    const int nc_hi = a->num_comm_sms > 0 ? a->num_comm_sms : (nc_cap < 18 ? (nc_cap < step ? step : nc_cap) : 18);
    const bool may_wide = g.ctas_per_tile == 2 && a->cta_pair != 1 && a->k >= 4096 && a->n > BN;
    const bool may_narrow = !(g.ctas_per_tile == 2 && a->cta_pair == 2 && may_wide);
    double best_t = 1e30;
    int best_nc = nc_lo, best_wide = may_narrow ? 0 : 1;
    for (int wide = 0; wide <= 1; ++wide) {
        if ((wide && !may_wide) || (!wide && !may_narrow)) continue;
        const int seg_items = seg_m_tiles * (wide ? (n_tiles + 1) / 2 : n_tiles);
        // a 256-column tile (or half of a wide item) on one CTA pair / CTA: the wide tiling runs ~4 % more FLOP/s but
        // pays ~1.5 us more per half for an epilogue that overlaps the next main loop only half by half
        const double rows = BM * g.ctas_per_tile;
        const double tile_s = 2.0 * rows * BN * a->k / ((wide ? 19.0e12 : 18.2e12) * g.ctas_per_tile / 2.0) + (wide ? 1.5e-6 : 0.5e-6);
        for (int nc = nc_lo; nc <= nc_hi; nc += step) {
            const int units = (sms - nc) / g.ctas_per_tile;
            if (units < 1) break;
            const double t_gemm = schedule_cost(seg_items * a->world, units, wide) * tile_s;
            const double rate = nc * per_pusher < link_cap ? nc * per_pusher : link_cap;
            const double t_push = push_bytes / rate;
            const double t_tail = schedule_cost(seg_items, units, wide) * tile_s;
            double t = t_gemm > t_push + t_tail ? t_gemm : t_push + t_tail;
            if (!wide) t *= 0.98;   // on a tie the smaller tiles: their tail is finer
            if (t < best_t * 0.999) {
                best_t = t;
                best_nc = nc;
                best_wide = wide;
            }
        }
    }
    g.num_comm = best_nc;
    g.wide = best_wide;
    g.num_tiles = seg_m_tiles * (g.wide ? (n_tiles + 1) / 2 : n_tiles) * a->world;
}

static GridPlan plan_grid(const TdistGemmArgs* a) {
    GridPlan g;
    g.ctas_per_tile = use_pair(a) ? 2 : 1;
    g.wide = use_wide(a) ? 1 : 0;
    const int seg_m_tiles = (a->m_per_rank + BM * g.ctas_per_tile - 1) / (BM * g.ctas_per_tile);
    const int n_tiles = (a->n + BN - 1) / BN;
    g.num_tiles = seg_m_tiles * (g.wide ? (n_tiles + 1) / 2 : n_tiles) * a->world;
    int capacity = resident_ctas(g.ctas_per_tile, g.wide, a->mode);
    if (a->mode == TDIST_GEMM_AG && a->world > 1 && g.ctas_per_tile == 2) {
        // either pair tiling may be chosen below: the grid has to fit both
        const int other = resident_ctas(2, g.wide ? 0 : 1, a->mode);
        if (other < capacity) capacity = other;
    }
    int sms = a->num_sms > 0 ? a->num_sms : capacity;
    if (sms > capacity) sms = capacity;
    if (g.ctas_per_tile == 2) sms &= ~1;
    if (sms < g.ctas_per_tile) sms = g.ctas_per_tile;
    g.num_comm = 0;
    if (a->mode == TDIST_GEMM_AG && a->world > 1) {
        plan_ag(a, sms, n_tiles, g);
        if (g.ctas_per_tile == 2) g.num_comm = (g.num_comm + 1) & ~1;
        if (g.num_comm > sms - g.ctas_per_tile) g.num_comm = sms - g.ctas_per_tile;
        if (g.num_comm < g.ctas_per_tile) g.num_comm = g.ctas_per_tile;
    }
    int units = (sms - g.num_comm) / g.ctas_per_tile;
    // a wide schedule may split its last round in two: allow up to twice the items
    const int most = g.wide ? 2 * g.num_tiles : g.num_tiles;
    if (units > most) units = most;
    if (units < 1) units = 1;
    g.grid = units * g.ctas_per_tile + g.num_comm;
    return g;
}

extern "C" int tdist_gemm_grid(const TdistGemmArgs* a) { return plan_grid(a).grid; }

extern "C" int tdist_gemm_plan(const TdistGemmArgs* a, int* out4) {
    if (a == nullptr || out4 == nullptr) return fail(TDIST_EINVAL, "null args");
    const GridPlan g = plan_grid(a);
    out4[0] = g.ctas_per_tile;
    out4[1] = g.wide;
    out4[2] = g.num_comm;
    out4[3] = g.grid;
    return 0;
}

// Runs the static schedule on the host: every 256-column tile of the problem must be given to exactly one unit, a
// wide item's halves to the same unit in the same round. Returns 0 and the longest unit's length in half items, or the
// number of the first check that failed.
extern "C" int tdist_gemm_schedule_check(int wide, int num_units, int world, int rank, int seg_m_tiles, int n_tiles,
                                         int group_m, int split_first, int* makespan_halves, int* first_remote_half) {
    if (num_units < 1 || world < 1 || seg_m_tiles < 1 || n_tiles < 1 || rank < 0 || rank >= world) return -1;
    GemmParams* p = new GemmParams;
    memset(p, 0, sizeof(*p));
    p->world = world;
    p->rank = rank;
    p->seg_m_tiles = seg_m_tiles;
    p->n_tiles = n_tiles;
    p->n_pairs = (n_tiles + 1) / 2;
    p->group_m = group_m > 0 ? group_m : DEFAULT_GROUP_M;
    p->num_tiles = seg_m_tiles * (wide ? p->n_pairs : n_tiles) * world;
    p->split_first = split_first;
    std::string seen(static_cast<size_t>(world) * seg_m_tiles * n_tiles, 0);
    int rc = 0, longest = 0, first_remote = 1 << 30;
    for (int u = 0; u < num_units && rc == 0; ++u) {
        Work w;
        int len = 0;
        for (int round = 0; rc == 0; ++round) {
            const bool more = wide ? get_work<true>(*p, u, num_units, round, rank, w) : get_work<false>(*p, u, num_units, round, rank, w);
            if (!more) break;
            if (round > 4 * (p->num_tiles / num_units + 2)) rc = 1;   // the schedule must end
            if (w.halves == 0) continue;
            if (w.halves < 0 || w.halves > 2 || w.seg < 0 || w.seg >= world || w.m_in_seg < 0 || w.m_in_seg >= seg_m_tiles) rc = 2;
            for (int h = 0; h < w.halves && rc == 0; ++h) {
                if (w.n_tile + h >= n_tiles) rc = 3;
                else {
                    char& c = seen[(static_cast<size_t>(w.seg) * seg_m_tiles + w.m_in_seg) * n_tiles + w.n_tile + h];
                    if (c) rc = 4;
                    c = 1;
                }
            }
            if (w.seg != rank && len < first_remote) first_remote = len;
            len += w.halves;
        }
        if (len > longest) longest = len;
    }
    if (rc == 0)
        for (char c : seen)
            if (!c) rc = 5;
    if (makespan_halves) *makespan_halves = longest;
    if (first_remote_half) *first_remote_half = first_remote;
    delete p;
    return rc;
}

extern "C" int tdist_gemm_run(const TdistGemmArgs* a) {
    if (a == nullptr) return fail(TDIST_EINVAL, "null args");
    if (a->world < 1 || a->world > TDIST_MAX_RANKS || a->rank < 0 || a->rank >= a->world)
        return fail(TDIST_EINVAL, "world/rank out of range (at most 8 ranks)");
    if (a->m_per_rank < 1 || a->n < 1 || a->k < 1) return fail(TDIST_EINVAL, "empty problem");
    if (a->k % 8 != 0 || a->n % 8 != 0)
        return fail(TDIST_EINVAL, "K and N must be multiples of 8 (16-byte rows for TMA)");
    if (a->mode < TDIST_GEMM_PLAIN || a->mode > TDIST_GEMM_RS) return fail(TDIST_EINVAL, "bad mode");
    if (a->expert_ids != nullptr && (a->mode != TDIST_GEMM_PLAIN || a->world != 1))
        return fail(TDIST_EINVAL, "grouped GEMM (expert_ids) is a single-rank plain-mode feature");
    if ((a->gather_dst != nullptr) != (a->block_ready != nullptr) || (a->gather_dst != nullptr) != (a->gather_counter != nullptr) ||
        (a->gather_dst != nullptr && a->a_gather == nullptr))
        return fail(TDIST_EINVAL, "the staged row gather needs a_gather, gather_dst, block_ready and gather_counter together");
    if ((a->c_scatter != nullptr || a->block_rot != nullptr) && (a->mode != TDIST_GEMM_PLAIN || a->world != 1 || a->cta_pair > 0))
        return fail(TDIST_EINVAL, "c_scatter / block_rot are plain-mode, one-CTA-per-tile features");
    if (a->a_gather != nullptr) {
        if (a->mode != TDIST_GEMM_PLAIN || a->world != 1) return fail(TDIST_EINVAL, "row-gathering A is a plain-mode feature (world = 1 in the GEMM's own terms)");
        if (a->a_gather_rows < 1) return fail(TDIST_EINVAL, "row-gathering A needs the number of source rows");
        if (a->block_src != nullptr && (a->src_flags == nullptr || a->src_world < 1 || a->src_world > TDIST_MAX_RANKS || a->src_rank < 0 || a->src_rank >= a->src_world))
            return fail(TDIST_EINVAL, "block_src needs src_flags and a valid (src_rank, src_world)");
    }

    const GridPlan plan = plan_grid(a);
    const int ctas = plan.ctas_per_tile;
    GemmParams p;
    memset(&p, 0, sizeof(p));
    const CUtensorMapDataType dt = a->dtype == TDIST_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    const uint64_t K = a->k, N = a->n, MPR = a->m_per_rank, W = a->world;
    int rc;
    {
        // A (or the gather workspace): {K, m_per_rank, world}
        const void* base = a->mode == TDIST_GEMM_AG ? a->a_ws : a->a;
        if (a->mode == TDIST_GEMM_AG && a->world == 1) base = a->a;
        if (a->gather_dst != nullptr) base = a->gather_dst;   // the CTAs' own warps fill it, TMA reads it
        if (base == nullptr) return fail(TDIST_EINVAL, "A / workspace pointer is null");
        uint64_t dims[3] = {K, MPR, W};
        uint64_t strides[2] = {K * 2, MPR * K * 2};
        uint32_t box[3] = {BK, BM, 1};
        if ((rc = tdist_host::encode_tmap(&p.tm_a, dt, 2, 3, base, dims, strides, box, tdist_host::Swizzle::B128))) return rc;
    }
    if (a->mode == TDIST_GEMM_AG) {
        uint64_t dims[3] = {K, MPR, 1};
        uint64_t strides[2] = {K * 2, MPR * K * 2};
        uint32_t box[3] = {BK, BM, 1};
        if ((rc = tdist_host::encode_tmap(&p.tm_a_own, dt, 2, 3, a->a, dims, strides, box, tdist_host::Swizzle::B128))) return rc;
    }
    {
        const uint64_t E = a->num_experts > 0 ? a->num_experts : 1;
        uint64_t dims[3] = {K, N, E};
        uint64_t strides[2] = {K * 2, N * K * 2};
        uint32_t box[3] = {BK, static_cast<uint32_t>(BN / ctas), 1};
        if ((rc = tdist_host::encode_tmap(&p.tm_b, dt, 2, 3, a->b, dims, strides, box, tdist_host::Swizzle::B128))) return rc;
    }
    {
        uint64_t dims[3] = {N, MPR, W};
        uint64_t strides[2] = {N * 2, MPR * N * 2};
        uint32_t box[3] = {EPI_COLS, BM, 1};
        if (a->mode == TDIST_GEMM_RS) {
            for (int r = 0; r < a->world; ++r) {
                if (a->c_stage_peer[r] == nullptr) return fail(TDIST_EINVAL, "RS staging pointer is null");
                if ((rc = tdist_host::encode_tmap(&p.tm_c[r], dt, 2, 3, a->c_stage_peer[r], dims, strides, box, tdist_host::Swizzle::B128))) return rc;
            }
        } else if (a->c_scatter == nullptr) {
            if (a->c == nullptr) return fail(TDIST_EINVAL, "C pointer is null");
            if ((rc = tdist_host::encode_tmap(&p.tm_c[0], dt, 2, 3, a->c, dims, strides, box, tdist_host::Swizzle::B128))) return rc;
        } else if (a->c == nullptr || a->c_rows < 1) {
            return fail(TDIST_EINVAL, "the scattering epilogue needs C and its row count");
        }
    }
    p.a_own = static_cast<const char*>(a->a);
    for (int r = 0; r < a->world; ++r) {
        p.a_ws_peer[r] = static_cast<char*>(a->a_ws_peer[r]);
        p.flags_peer[r] = a->flags_peer[r];
    }
    p.a_gather = static_cast<const int*>(a->a_gather);
    p.a_raw = static_cast<const char*>(a->a);
    p.a_gather_rows = a->a_gather_rows;
    p.block_src = static_cast<const int*>(a->block_src);
    p.src_flags = static_cast<const uint64_t*>(a->src_flags);
    p.src_epoch = a->src_epoch;
    p.src_rank = a->src_rank;
    p.src_world = a->src_world;
    p.gather_dst = static_cast<char*>(a->gather_dst);
    p.block_ready = static_cast<uint32_t*>(a->block_ready);
    p.gather_counter = static_cast<uint32_t*>(a->gather_counter);
    {
        // the first wave of tiles: one tile per GEMM CTA, rows of tiles GROUP_M blocks deep
        const int gm = a->group_m > 0 ? a->group_m : DEFAULT_GROUP_M;
        const int n_tiles = (a->n + BN - 1) / BN;
        const int first_wave = (plan.grid - plan.num_comm + n_tiles - 1) / n_tiles;
        p.gather_pro_blocks = a->gather_counter != nullptr ? (first_wave + gm - 1) / gm * gm : 0;
    }
    p.block_rot = static_cast<const int*>(a->block_rot);
    p.c_scatter = static_cast<const int*>(a->c_scatter);
    p.c_out = static_cast<char*>(a->c);
    p.c_rows = a->c_rows;
    p.stage_local = static_cast<const char*>(a->c_stage_peer[a->rank]);
    p.a_ws_mc = (a->mode == TDIST_GEMM_AG && a->world > 1) ? static_cast<char*>(a->a_ws_mc) : nullptr;
    p.rs_out = a->rs_out;
    {
        static const bool fused = [] {
            const char* e = getenv("TDIST_RS_FUSED_REDUCE");
            return e == nullptr || atoi(e) != 0;
        }();
        p.rs_fused = (a->mode == TDIST_GEMM_RS && fused) ? 1 : 0;
    }
    p.flags = a->flags;
    p.m_per_rank = a->m_per_rank;
    p.n = a->n;
    p.k = a->k;
    p.world = a->world;
    p.rank = a->rank;
    p.seg_blocks = (a->m_per_rank + BM - 1) / BM;
    p.seg_m_tiles = (a->m_per_rank + BM * ctas - 1) / (BM * ctas);
    p.n_tiles = (a->n + BN - 1) / BN;
    p.n_pairs = (p.n_tiles + 1) / 2;
    p.k_blocks = (a->k + BK - 1) / BK;
    p.is_f16 = a->dtype == TDIST_F16;
    p.epoch = a->epoch;
    p.debug_delay_ns = a->debug_delay_ns;
    p.trace = static_cast<unsigned long long*>(a->trace);
    p.expert_ids = static_cast<const int*>(a->expert_ids);
    p.num_m_blocks = static_cast<const int*>(a->num_m_blocks);
    p.wctx.status = static_cast<Status*>(a->status);
    p.wctx.timeout_ns = a->timeout_ns;
    p.wctx.kernel_id = kKernelGemm;
    p.wctx.rank = a->rank;
    p.num_comm = plan.num_comm;
    {
        static const int ahead = [] {
            const char* e = getenv("TDIST_AG_PUSH_AHEAD");
            const int v = e ? atoi(e) : PUSH_AHEAD;
            return v < 1 ? 1 : (v > PUSH_AHEAD ? PUSH_AHEAD : v);
        }();
        p.push_ahead = ahead;
    }
    p.push_count = static_cast<uint32_t*>(a->push_count);
    p.push_parts = 1;
    if (a->mode == TDIST_GEMM_AG && a->world > 1 && a->push_count != nullptr && a->a_ws_mc == nullptr) {
        // as many slices as pushers (a power of two, at most eight: 16 rows per slice)
        while (p.push_parts * 2 <= plan.num_comm && p.push_parts < 8) p.push_parts *= 2;
    }
    p.group_m = a->group_m > 0 ? a->group_m : DEFAULT_GROUP_M;
    p.num_tiles = plan.num_tiles;
    p.split_first = 0;
    if (a->mode == TDIST_GEMM_AG && a->world > 1 && plan.wide) {
        // units that would start on a peer's segment, whose rows are still on the wire: cut that many own items in two
        static const bool enabled = [] {
            const char* e = getenv("TDIST_AG_SPLIT_FIRST");
            return e == nullptr || atoi(e) != 0;
        }();
        const int units = (plan.grid - plan.num_comm) / ctas;
        const int own = plan.num_tiles / a->world;
        if (enabled && own < units && units - own <= own) p.split_first = units - own;
    }

    if (a->mode == TDIST_GEMM_AG && a->world > 1) {
        if (a->flags == nullptr) return fail(TDIST_EINVAL, "AG needs flags");
        for (int r = 0; r < a->world; ++r)
            if (a->a_ws_peer[r] == nullptr || a->flags_peer[r] == nullptr)
                return fail(TDIST_EINVAL, "AG needs the workspace and flags of every rank");
    }
    if (a->mode == TDIST_GEMM_RS) {
        if (a->flags == nullptr || a->rs_out == nullptr) return fail(TDIST_EINVAL, "RS needs flags and rs_out");
        for (int r = 0; r < a->world; ++r)
            if (a->flags_peer[r] == nullptr) return fail(TDIST_EINVAL, "RS needs the flags of every rank");
    }

    cudaStream_t stream = static_cast<cudaStream_t>(a->stream);
    const void* fn = kernel_of(ctas, plan.wide, a->mode);  // smem opt-in done by resident_ctas()
    int block_threads = THREADS;
    if (a->a_gather != nullptr && a->gather_dst == nullptr) {
        fn = reinterpret_cast<const void*>(&gemm_sm100_kernel<TDIST_GEMM_PLAIN, 1, true>);
        block_threads = GATHER_THREADS;
        static bool attr_set[64] = {};
        int dev = 0;
        TDIST_CUDA_OK(cudaGetDevice(&dev));
        if (dev >= 0 && dev < 64 && !attr_set[dev]) {
            TDIST_CUDA_OK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
            attr_set[dev] = true;
        }
    }
    void* kargs[] = {&p};
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(plan.grid);
    cfg.blockDim = dim3(block_threads);
    cfg.dynamicSmemBytes = SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ctas;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    TDIST_CUDA_OK(cudaLaunchKernelExC(&cfg, fn, kargs));
    return 0;
}
