/* C ABI of libtdist.so. Every entry point takes raw device pointers plus a CUDA stream and
 * returns 0 on success or a negative TDIST_E* / positive cudaError_t value; none of them
 * synchronises the stream. The Python package binds these with ctypes. */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TDIST_MAX_RANKS 8

#define TDIST_EINVAL (-1)   /* bad shape / alignment / argument            */
#define TDIST_EDRIVER (-2)  /* a CUDA driver entry point is not available  */
#define TDIST_ELIMIT (-3)   /* size beyond a compiled-in maximum           */

const char* tdist_last_error(void);

/* ------------------------------------------------------------------ status block */
/* Device-memory record that bounded device waits write when they give up. */
typedef struct TdistStatus {
    int abort_flag, code, kernel_id, rank, peer, index;
    long long expected, seen;
    int block, where;
    int reserved[4];
} TdistStatus;
int tdist_status_create(void** device_ptr);
int tdist_status_read(const void* device_ptr, TdistStatus* out); /* blocking device-to-host copy */
int tdist_status_reset(void* device_ptr);
int tdist_status_destroy(void* device_ptr);

/* ------------------------------------------------------------------ tcgen05 GEMM family */
enum { TDIST_GEMM_PLAIN = 0, TDIST_GEMM_AG = 1, TDIST_GEMM_RS = 2 };
enum { TDIST_BF16 = 0, TDIST_F16 = 1, TDIST_F32 = 2, TDIST_I32 = 3 };

typedef struct TdistGemmArgs {
    /* A operand. PLAIN/RS: the whole local A, [world*m_per_rank, K] row-major (K contiguous).
     * AG: this rank's shard [m_per_rank, K]. */
    const void* a;
    /* AG only: local gather workspace [world, m_per_rank, K]; peers push their shards into it.
     * a_ws_peer[r] is rank r's workspace as mapped into this process. */
    void* a_ws;
    void* a_ws_peer[TDIST_MAX_RANKS];
    /* B operand [N, K] row-major (K contiguous): C = A * B^T. */
    const void* b;
    /* PLAIN/AG: output [world*m_per_rank, N]. */
    void* c;
    /* RS only: partial-sum staging [world(src), m_per_rank, N] on every rank; c_stage_peer[r]
     * is rank r's staging as mapped here (c_stage_peer[rank] is the local one). */
    void* c_stage_peer[TDIST_MAX_RANKS];
    /* RS only: reduced output [m_per_rank, N]. */
    void* rs_out;
    /* AG: flags[world][m_tiles_per_seg]; RS: flags[tiles_per_seg][world]; 32-bit epochs.
     * flags_peer[r] is rank r's array as mapped here. */
    uint32_t* flags;
    uint32_t* flags_peer[TDIST_MAX_RANKS];
    int m_per_rank, n, k;
    int world, rank;
    int mode;          /* TDIST_GEMM_*           */
    int dtype;         /* TDIST_BF16 / TDIST_F16 */
    uint32_t epoch;    /* value the flags of this call carry; strictly increasing per context */
    int num_sms;       /* CTAs to use in total (0 = all SMs of the device) */
    int num_comm_sms;  /* AG: CTAs that only push this rank's shard to the peers */
    int debug_delay_ns;/* AG: the pusher sleeps this long before every block (race hunting) */
    int group_m;       /* row-tiles per raster group (0 = default 8) */
    int cta_pair;      /* -1 auto, 0 = one CTA per 128x256 tile, 1 = CTA pair per 256x256 tile, 2 = CTA pair per 256x512 tile */
    void* status;      /* device pointer of a TdistStatus, may be NULL */
    uint64_t timeout_ns;
    void* stream;
    /* Optional timeline, 2048 uint64 %globaltimer stamps (NULL = off). Pusher CTA b < 16 writes at
     * [40b]: begin, end, then (start, end) of its first 18 items, at [40b + 38] / [40b + 39] the ns it spent waiting for
     * store completion / publishing flags. GEMM CTA c < 64 writes at
     * [1024 + 4c]: producer begin, producer end, ns spent waiting on flags, waits longer than 2 us. The MMA-issuing
     * thread of tile unit u < 64 writes at [1536 + 4u]: SM cycles in all, cycles waiting for operands (full
     * barriers), cycles waiting for a TMEM slot (epilogue not done), tiles computed. */
    void* trace;
    /* Grouped GEMM (PLAIN mode, world 1): B is [num_experts, N, K]; 128-row block i of A and C uses
     * B[expert_ids[i]]; blocks at or past *num_m_blocks (device int32, may be NULL) are skipped. */
    const void* expert_ids;
    const void* num_m_blocks;
    int num_experts;
    /* AG, optional: multicast alias of `a_ws` (a heap bound to an NVSwitch multicast object). When set, the
     * pushers store every block once with multimem.st instead of once per peer. */
    void* a_ws_mc;
    /* AG, optional: device uint32[(world - 1) * blocks per segment], zero before the first call (the kernel leaves it
     * zero). With it the unicast pushers send every 128-row block as up to eight row slices in parallel and meet on
     * these counters; the pusher that completes a block raises its flag. Without it a block is one pusher's work. */
    void* push_count;
    /* PLAIN, optional row-gathering A: row r of the logical A [m_per_rank, K] is row a_gather[r] (device int32) of
     * the matrix at `a` ([a_gather_rows, K]); indices outside [0, a_gather_rows) read as zeros. One CTA per tile;
     * the producer warp copies the rows with cp.async. With block_src (device int32 per 128-row block) the rows of
     * a block belong to rank block_src[b]'s segment of an all-gather in flight: before loading them the kernel waits
     * (bounded) until src_flags[block_src[b]] >= src_epoch (64-bit words, the all-gather's arrival flags); blocks
     * of src_rank itself are not waited for. */
    const void* a_gather;
    int a_gather_rows;
    const void* block_src;
    const void* src_flags;
    uint64_t src_epoch;
    int src_rank, src_world;
    /* Row-gathering A through a staging matrix (preferred form of the above): with gather_dst set ([m_per_rank, K]
     * workspace) the kernel itself copies the rows block by block into gather_dst, in the order the GEMM consumes
     * them, and raises block_ready[b] = epoch (device uint32 per 128-row block, zero before the first call, epochs
     * strictly increasing); the TMA producers feed on gather_dst and wait per block. All threads of the grid stage
     * the blocks of the first wave of tiles before the roles split; the epilogue warps stage the rest, 16 rows per
     * claim, while they wait for accumulators. The copy of one block overlaps the MMAs of the blocks before it, and
     * with block_src the all-gather in flight. */
    void* gather_dst;
    void* block_ready;
    /* device uint32[4 + blocks], zero before the first call (the kernel leaves it zero): grid-wide arrival counters
     * and the claim cursor of the staging */
    void* gather_counter;
    /* device int32, may be NULL: 128-row block the schedule starts at (blocks are visited cyclically from there),
     * e.g. the first block of this rank's own tokens */
    const void* block_rot;
    /* Scattering epilogue (PLAIN, one CTA per tile), optional: row r of the product goes to row c_scatter[r] (device
     * int32) of the matrix at `c` ([c_rows, N]); rows whose index is outside [0, c_rows) are dropped (padding). */
    const void* c_scatter;
    int c_rows;
} TdistGemmArgs;

int tdist_gemm_run(const TdistGemmArgs* args);
/* Number of CTAs a call with these arguments launches (for occupancy planning and tests). */
int tdist_gemm_grid(const TdistGemmArgs* args);
/* The launch plan of a call with these arguments: out4 = {CTAs per tile (1 or 2), wide tiling (0 / 1), pusher CTAs,
 * grid size}. Launches nothing. */
int tdist_gemm_plan(const TdistGemmArgs* args, int* out4);
/* Host-side replay of the kernel's static tile schedule (no GPU needed): `num_units` CTAs or CTA pairs over a problem
 * of `world` segments of seg_m_tiles x n_tiles 256-column tiles, wide (items of two neighbouring tiles) or narrow,
 * with `split_first` own items cut in two in round 0. Returns 0 when every tile is given out exactly once;
 * *makespan_halves = the longest unit in half items (a wide item counts 2), *first_remote_half = how many half items
 * the earliest unit has done before it first needs another rank's rows. */
int tdist_gemm_schedule_check(int wide, int num_units, int world, int rank, int seg_m_tiles, int n_tiles, int group_m,
                              int split_first, int* makespan_halves, int* first_remote_half);

/* Block-scaled fp8 (e4m3) GEMM, plain or fused AllGather-GEMM (csrc/kernels/gemm_fp8_sm100.cu).
 * C[m, n] = sum_kb sa[m, kb] * sb[n / 128, kb] * dot(A[m, 128kb : 128kb+128], B[n, same]); C is bf16. */
typedef struct TdistGemmFp8Args {
    const void* a;       /* PLAIN: [world*m_per_rank, K] e4m3; AG: this rank's shard [m_per_rank, K] */
    const void* sa;      /* fp32 scales of `a`, [rows, K/128] */
    const void* b;       /* [N, K] e4m3 */
    const void* sb;      /* fp32 [ceil(N/128), K/128] */
    void* c;             /* bf16 [world*m_per_rank, N] */
    /* AG: gather workspaces for rows [world, m_per_rank, K] and scales [world, m_per_rank, K/128];
     * *_peer[r] is rank r's as mapped here. flags[world][ceil(m_per_rank/128)], 32-bit epochs. */
    void* a_ws;
    void* sa_ws;
    void* a_ws_peer[TDIST_MAX_RANKS];
    void* sa_ws_peer[TDIST_MAX_RANKS];
    uint32_t* flags;
    uint32_t* flags_peer[TDIST_MAX_RANKS];
    int m_per_rank, n, k;
    int world, rank;
    int mode;            /* TDIST_GEMM_PLAIN or TDIST_GEMM_AG */
    uint32_t epoch;
    int num_sms;         /* 0 = all */
    int num_comm_sms;    /* AG pusher CTAs, 0 = default 8 */
    void* status;
    uint64_t timeout_ns;
    void* stream;
} TdistGemmFp8Args;

int tdist_gemm_fp8_run(const TdistGemmFp8Args* args);

/* ------------------------------------------------------------------ standalone collectives */
/* PUSH_ORDERED: like PUSH, but all copy CTAs serve one destination after the other, rank - 1 first (the order in which the
 * consumers of a rotated schedule need this rank's segment), so that segments arrive one by one instead of all at the end */
enum { TDIST_AG_PULL = 0, TDIST_AG_PUSH = 1, TDIST_AG_LL = 2, TDIST_AG_PUSH_ORDERED = 3 };

typedef struct TdistCollArgs {
    /* all-gather: the in-place symmetric buffer [world * seg_bytes] of every rank as mapped here.
     * reduce-scatter: the symmetric staging [world][seg_bytes] of every rank (the caller alternates
     * between two such buffers from call to call). */
    void* buf_peer[TDIST_MAX_RANKS];
    void* sig_peer[TDIST_MAX_RANKS];  /* uint64 flags [world] of every rank */
    void* ll_peer[TDIST_MAX_RANKS];   /* LL all-gather only: staging [world][2 * seg_bytes], alternated like above */
    void* counters;                   /* local uint32 [world], zero on first use */
    const void* input;                /* reduce-scatter: local [world * seg_bytes] */
    void* output;                     /* reduce-scatter: local [seg_bytes] */
    size_t seg_bytes;
    int world, rank;
    int mode;           /* TDIST_AG_* (all-gather only) */
    int phase;          /* 0 or 3 = whole op; 1 = send half only, 2 = receive half only (emulated ranks) */
    int ctas_per_peer;  /* 0 = default 4 */
    int dtype;          /* reduce-scatter element type */
    uint64_t epoch;     /* strictly increasing per context, starts at 1 */
    void* status;
    uint64_t timeout_ns;
    void* stream;
    /* reduce-scatter, optional fused top-k reduce (MoE): with topk > 0, `input` is the expert-sorted bf16 output
     * [rows, row_bytes] of a grouped GEMM and logical row t of the [world * seg_bytes] input is
     * sum_k topk_w[t*topk+k] * input_row[pos_of[t*topk+k]] (topk_w may be NULL = 1). */
    const void* pos_of;
    const void* topk_w;
    int topk;
    int row_bytes;
} TdistCollArgs;

int tdist_allgather(const TdistCollArgs* args);
int tdist_reduce_scatter(const TdistCollArgs* args);
/* out [block_bytes] = sum of the `splits` consecutive blocks of `in`, fp32 accumulation for bf16 / fp16, blocks
 * visited in ring order from `begin`. */
int tdist_ring_reduce(const void* in, void* out, size_t block_bytes, int splits, int begin, int dtype, void* stream);
/* Device-side barrier of all ranks on `stream`: flags_peer[r] = rank r's uint64[8] flag array as
 * mapped here, epoch_local = a local uint64 counter owned by the barrier. */
int tdist_barrier_all(void* const* flags_peer, void* epoch_local, int world, int rank, void* status,
                      uint64_t timeout_ns, void* stream);

/* Collectives through the NVSwitch multicast engine (csrc/kernels/nvls.cu). `mc` is the multicast alias
 * of a symmetric buffer [world * seg_bytes] that every rank bound to one multicast object, `local` this
 * rank's own alias. sig_peer[r] = rank r's uint64[2 * TDIST_MAX_RANKS] flags as mapped here. */
enum { TDIST_NVLS_ALLGATHER = 0, TDIST_NVLS_REDUCE_SCATTER = 1, TDIST_NVLS_ALLREDUCE = 2 };

typedef struct TdistNvlsArgs {
    void* mc;
    void* local;
    void* sig_peer[TDIST_MAX_RANKS];
    void* counters;      /* local uint32[2], zero on first use */
    void* output;        /* reduce-scatter: local [seg_bytes]; otherwise unused (in place) */
    size_t seg_bytes;    /* multiple of 16 */
    int world, rank;
    int op;              /* TDIST_NVLS_* */
    int dtype;           /* reductions: TDIST_BF16 / TDIST_F16 / TDIST_F32 */
    int ctas;            /* 0 = sized from seg_bytes, at most 64 */
    uint64_t epoch;      /* strictly increasing per buffer, starts at 1 */
    void* status;
    uint64_t timeout_ns;
    void* stream;
} TdistNvlsArgs;

int tdist_nvls(const TdistNvlsArgs* args);

/* Peer-to-peer copy in one of five data paths (see csrc/kernels/p2p_copy.cu). */
int tdist_p2p_copy(const void* src, void* dst, size_t bytes, int mode, int ctas, int threads, int chunk,
                   void* status, uint64_t timeout_ns, void* stream);

/* Stream-ordered signal operations on an address of this process (a peer's flag as mapped here, or a
 * local one). sig_op: 9 = set, 10 = add. cmp: 0 EQ, 1 NE, 2 GT, 3 LE, 4 LT, 5 GE. The wait is bounded and
 * reports through `status` like every device wait. */
int tdist_signal_op_on_stream(void* sig, uint64_t value, int sig_op, void* stream);
int tdist_signal_wait_on_stream(const void* sig, int cmp, uint64_t value, void* status, uint64_t timeout_ns, void* stream);

/* ------------------------------------------------------------------ MoE all-to-all */
enum { TDIST_A2A_DISPATCH = 0, TDIST_A2A_COMBINE = 1 };

typedef struct TdistA2AArgs {
    const void* send;        /* DISPATCH: [rows, row_bytes_in]; COMBINE: receive-layout [world*max_m, row_bytes_in] */
    const void* src_index;   /* DISPATCH, optional int32 [rows]: source row of each expert-sorted row */
    const void* counts;      /* DISPATCH: int32 cumsum [G+1]; COMBINE: int32 received splits [world*epr] */
    const void* send_scale;  /* optional fp32 [rows, scale_cols], travels with the rows (no quantisation) */
    void* recv_peer[TDIST_MAX_RANKS];   /* this call's parity of every rank: [world(src)][max_m][row_bytes_out] */
    void* scale_peer[TDIST_MAX_RANKS];  /* fp32 [world(src)][max_m][scale_cols], may be NULL */
    void* splits_peer[TDIST_MAX_RANKS]; /* int32 [world(src)][epr] (DISPATCH) */
    void* sig_peer[TDIST_MAX_RANKS];    /* uint64 [world] */
    void* counters;                     /* local uint32 [world], zero on first use */
    /* fused top-k weighted reduction after COMBINE (reduce = 1) */
    const void* slot_of;     /* int32 [ntok*topk] from tdist_moe_route */
    const void* cumsum;      /* int32 [G+1] of this rank's dispatch */
    const void* topk_ids;    /* int32 [ntok*topk] */
    const void* topk_w;      /* fp32 [ntok*topk] */
    void* out;               /* bf16 [ntok, hidden] */
    int ntok, topk;
    int row_bytes_in, row_bytes_out, scale_cols, hidden;
    int max_m, epr, world, rank;
    int mode;                /* TDIST_A2A_* */
    int quant;               /* DISPATCH: 1 = bf16 -> fp8 e4m3 with one fp32 scale per 128 values */
    int reduce;
    int phase;               /* 0/3 whole op, 1 send half, 2 receive half */
    int ctas_per_peer;       /* 0 = default 8 */
    uint64_t epoch;
    void* status;
    uint64_t timeout_ns;
    void* stream;
} TdistA2AArgs;

int tdist_a2a(const TdistA2AArgs* args);
int tdist_dequant_fp8(const void* x, const void* scale, void* out_bf16, int rows, int hidden, void* stream);

/* ------------------------------------------------------------------ expert-parallel dispatch / combine (moe_ep.cu) */
#define TDIST_MOE_ROUTE_IN_PLACE_MAX 8192   /* most (token, k) pairs the dispatch kernel routes by itself */

typedef struct TdistMoeDispatchArgs {
    const void* x;            /* [ntok, hidden] bf16 */
    const void* topk_ids;     /* int32 [ntok * topk]; an id outside [0, num_experts) drops the pair and is reported */
    const void* slot_of;      /* optional routing done beforehand (tdist_moe_route), for more pairs than the kernel */
    const void* cumsum;       /*   routes in place: sorted position of each pair, prefix sum of the counts [E + 1] */
    void* recv_peer[TDIST_MAX_RANKS];    /* receive rows of every rank as mapped here (this call's parity) */
    void* scale_peer[TDIST_MAX_RANKS];   /* quant: fp32 [rows, hidden / 128] beside them */
    void* counts_peer[TDIST_MAX_RANKS];  /* int32 [world(src)][num_experts], this call's parity */
    void* sig_peer[TDIST_MAX_RANKS];     /* uint64 [2 * world]: data flags [0, world), count flags [world, 2 world) */
    void* counters;           /* uint32 [2], local, zero before the first call */
    void* pair_row;           /* out int32 [ntok * topk]: row of each pair in its destination's buffer, -1 = dropped */
    void* send_splits;        /* out int32 [num_experts]: pairs of this rank per expert */
    void* recv_splits;        /* out int32 [world, experts_per_rank]: rows each source sent to my experts */
    void* recv_offset;        /* out int32 [experts_per_rank, world] (compact): first row of each (expert, source) group */
    void* num_recv;           /* out int32 [1]: rows received in all */
    void* block_expert;       /* out int32 [max_m / align], optional (compact): local expert of each block of `align` rows */
    void* num_blocks;         /* out int32 [1], optional (compact): blocks in use */
    int ntok, topk, hidden, num_experts, world, rank;
    int max_m;     /* slots: rows per source slot; compact: capacity of the receive buffer in rows */
    int quant;     /* 1 = rows travel as fp8 e4m3 with one fp32 scale per 128 values, 0 = as bf16 */
    int compact;   /* 0 = per-source slots [world][max_m], 1 = rows grouped by (local expert, source) back to back */
    int align;     /* compact: every expert's group starts on a multiple of this many rows (0/1 = dense, 128 = grouped GEMM) */
    int phase;     /* bit 0 publish counts (compact), bit 1 route + send + flag, bit 2 wait for every source; 0 = all */
    int num_ctas;  /* 0 = sized from the work */
    uint64_t epoch;           /* call number, > 0, the same on every rank */
    void* status;
    uint64_t timeout_ns;
    void* stream;
} TdistMoeDispatchArgs;

typedef struct TdistMoeCombineArgs {
    void* buf_peer[TDIST_MAX_RANKS];   /* expert outputs [rows, hidden] bf16 of every rank as mapped here */
    void* sig_peer[TDIST_MAX_RANKS];   /* uint64 [world]: "my outputs are in place" flags */
    const void* topk_ids;     /* int32 [ntok * topk] */
    const void* topk_w;       /* fp32 [ntok * topk] or NULL (plain sum) */
    const void* pair_row;     /* from the matching dispatch */
    void* out;                /* [ntok, hidden] bf16 */
    int ntok, topk, hidden, epr, world, rank;
    int phase;                /* bit 0 announce, bit 1 wait + gather; 0 = both */
    int num_ctas;
    uint64_t epoch;
    void* status;
    uint64_t timeout_ns;
    void* stream;
} TdistMoeCombineArgs;

int tdist_moe_dispatch(const TdistMoeDispatchArgs* args);
int tdist_moe_combine(const TdistMoeCombineArgs* args);

/* ------------------------------------------------------------------ MoE routing */
/* An expert id outside [0, num_experts) (e.g. -1 for a dropped pair) is left out of the counts and of the sort
   (slot_of = -1 / no sorted entry) and reported once through `status` (may be NULL) as a bad argument. */
int tdist_moe_route(const void* ids, int n, int topk, int num_experts, void* splits, void* cumsum,
                    void* sorted_token, void* slot_of, void* status, void* stream);
int tdist_moe_align_block_size(const void* ids, int numel_per_rank, int num_experts, int num_ranks, int block_size,
                               void* sorted_ids, int sorted_cap, void* expert_ids, void* block_barrier_ids,
                               void* rank_block_num, void* num_tokens_post_pad, void* status, void* stream);
/* dst[p] = src[index[p] / div] (zeros where index[p] is outside [0, limit)); pos_of (optional) gets the inverse map */
int tdist_gather_rows(const void* src, const void* index, int rows_out, int div, int limit, int row_bytes,
                      void* dst, void* pos_of, void* stream);
/* out[t] = sum_k weights[t,k] * y[pos_of[t*topk+k]] (bf16 rows, fp32 accumulation; weights may be NULL = 1) */
int tdist_topk_reduce(const void* y, const void* pos_of, const void* weights, int ntok, int topk, int row_bytes,
                      void* out, void* stream);
int tdist_moe_topk_softmax(const void* logits_f32, int ntok, int num_experts, int topk, int renormalize,
                           void* ids, void* weights, void* stream);

/* ------------------------------------------------------------------ GQA flash decode */
typedef struct TdistDecodeArgs {
    const void* q;            /* [B, Hq, D] bf16/fp16 */
    const void* k_cache;      /* [blocks, page, Hkv, D] (any strides that are multiples of 8 elements) */
    const void* v_cache;
    const void* block_table;  /* int32 [B, max_blocks] */
    const void* kv_lens;      /* int32 [B]: keys held by THIS rank per sequence */
    void* partial;            /* fp32 workspace [B, Hq, splits, D + 2] */
    void* counters;           /* uint32 [B * Hkv], zero on first use */
    void* out;                /* mode 0/2: [B, Hq, D] in q's dtype; mode 1: fp32 [B, Hq, D + 1] (O || LSE) */
    void* ll_peer[TDIST_MAX_RANKS]; /* mode 2: gather buffer of every rank, this call's parity:
                                       [world][B * Hq * (D + 2) / 2] 16-byte packets */
    int B, Hq, Hkv, head_dim, page_size, max_blocks, splits;
    long long stride_block, stride_token, stride_head; /* cache strides in elements */
    float scale, soft_cap;
    int mode;                 /* 0 = final output, 1 = O || LSE for a later cross-rank merge, 2 = sequence-parallel */
    int dtype;
    int world, rank;
    uint32_t epoch;           /* mode 2: non-zero, increasing per call */
    int push_only;            /* mode 2: 1 = compute and send, do not gather (emulated ranks) */
    void* status;
    uint64_t timeout_ns;
    void* stream;
    /* mode 2, optional: the call number lives on the device, so that a captured launch stays valid when it is
     * replayed. epoch_ptr: uint32, the number of the last completed call (starts at 0); the kernel uses
     * *epoch_ptr + 1 and stores it back when its last CTA finishes (not with push_only). epoch_done: uint32
     * scratch, zero on first use. ll_peer then holds the gather buffers of EVEN call numbers and ll_peer_alt
     * those of ODD ones; `epoch` is ignored. */
    void* epoch_ptr;
    void* epoch_done;
    void* ll_peer_alt[TDIST_MAX_RANKS];
    /* mode 2, optional: multicast alias (heap bound to an NVSwitch multicast object) of this call's parity of the
     * gather buffer; the exchange then takes one multimem.st per packet instead of one store per rank.
     * ll_mc_alt = the odd-call parity, needed with epoch_ptr. */
    void* ll_mc;
    void* ll_mc_alt;
} TdistDecodeArgs;

int tdist_flash_decode(const TdistDecodeArgs* args);
/* parts fp32 [ranks, heads, D + 1] -> out [heads, D] */
int tdist_lse_combine(const void* parts, int ranks, int heads, int head_dim, void* out, int dtype, void* stream);

/* ------------------------------------------------------------------ device primitives, one test op each */
enum {
    TDIST_PRIM_RING_PUT = 0, TDIST_PRIM_NOTIFY_WAIT = 1, TDIST_PRIM_NOTIFY_ADD = 2, TDIST_PRIM_PUT_SIGNAL = 3,
    TDIST_PRIM_PUT_QUIET_SIGNAL = 4, TDIST_PRIM_GET = 5, TDIST_PRIM_BROADCAST = 6, TDIST_PRIM_FCOLLECT = 7,
    TDIST_PRIM_GRID_BARRIER = 8, TDIST_PRIM_SCOPED_OPS = 9, TDIST_PRIM_BARRIER = 10,
    TDIST_PRIM_BOUNDS_PROBE = 11   /* only in the bounds-checked build: accesses that must be recorded and skipped */
};

typedef struct TdistPrimArgs {
    void* data_peer[TDIST_MAX_RANKS]; /* symmetric byte buffer of (world + 2) * nbytes: slots 0..world-1 receive, slot `world` is the source */
    void* sig_peer[TDIST_MAX_RANKS];  /* symmetric uint64[16]: words 0..7 signals, 8..15 barrier flags */
    void* result;                     /* local int32[8] */
    void* grid_counter;               /* local uint32, monotonic */
    void* barrier_epoch;              /* local uint64 */
    int world, rank, op, phase, nbytes;
    int scope;                        /* PUT_SIGNAL: 0 thread, 1 warp, 2 block */
    int grid;                         /* GRID_BARRIER: number of CTAs (must all be resident) */
    uint64_t value;
    void* status;
    uint64_t timeout_ns;
    void* stream;
} TdistPrimArgs;

/* 1 when this library was compiled with -DTDIST_BOUNDS_CHECK (checked symmetric-address translation), else 0 */
int tdist_bounds_checked(void);
int tdist_primitive(const TdistPrimArgs* args);

#ifdef __cplusplus
}
#endif
