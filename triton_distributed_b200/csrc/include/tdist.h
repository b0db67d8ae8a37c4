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
enum { TDIST_BF16 = 0, TDIST_F16 = 1 };

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
    int cta_pair;      /* -1 auto, 0 = one CTA per 128x256 tile, 1 = CTA pair per 256x256 tile */
    void* status;      /* device pointer of a TdistStatus, may be NULL */
    uint64_t timeout_ns;
    void* stream;
    /* Optional timeline, 2048 uint64 %globaltimer stamps (NULL = off). Pusher CTA b < 16 writes at
     * [40b]: begin, end, then (start, end) of its first 19 blocks. GEMM CTA c < 64 writes at
     * [1024 + 4c]: producer begin, producer end, ns spent waiting on flags, waits longer than 2 us. */
    void* trace;
} TdistGemmArgs;

int tdist_gemm_run(const TdistGemmArgs* args);
/* Number of CTAs a call with these arguments launches (for occupancy planning and tests). */
int tdist_gemm_grid(const TdistGemmArgs* args);

#ifdef __cplusplus
}
#endif
