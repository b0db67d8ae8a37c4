// Tutorials 07 and 08: the skeletons of the two overlapped tensor-parallel GEMMs, small enough to read in one sitting.
// The production kernels (csrc/kernels/gemm_sm100.cu) have exactly this structure; what they add is the tcgen05 / TMEM /
// TMA machinery that makes the math fast, plus one proxy fence (see the notes marked PRODUCTION below). Here the
// math is a plain per-thread dot product so that nothing distracts from the communication.
//
//   AG-GEMM  (07)  C[M, N] = allgather(A_shard)[M, K] * B[N, K]^T.   Some CTAs of the grid are PUSHERS: they copy this
//                  rank's rows into every peer's gather workspace, 16 rows at a time, and raise one flag per 16-row
//                  block there. The other CTAs are CONSUMERS: each takes 16 x 16 output tiles, own rows first, then
//                  the peers' in ring order, and before it reads a block of a peer's rows it waits for THAT block's
//                  flag only. Transfer and math overlap block by block inside one launch.
//   GEMM-RS  (08)  out[M/ws, N] = reduce_scatter_rows(A[M, K/ws] * B[N, K/ws]^T). Every CTA computes 16 x 16 tiles of the
//                  partial product, remote owners first, and stores each tile straight into the OWNER's staging slot
//                  for this source, then raises that tile's flag there. Once its tiles are done a CTA turns to the
//                  tiles this rank owns: it waits for the `world` flags of a tile and sums the partials in fp32.
//
// (reference tutorials/07-overlapping-allgather-gemm.py and 08-overlapping-gemm-reduce-scatter.py, which walk through
//  kernels/nvidia/allgather_gemm.py:131-252 and gemm_reduce_scatter.py:104-232; there the gather and the scatter are
//  copy-engine streams beside the GEMM kernel, here they are CTAs and epilogue stores of the GEMM kernel itself.)
#include <cuda_runtime.h>

#include "device/shmem.cuh"

using namespace tdist;

constexpr int TB = 16;   // rows per flag block and tile edge

struct OverlapParams {
    float* ws_peer[kMaxRanks];        // AG: gather workspace [world][mpr][K] of every rank; RS: staging [world(src)][mpr][N]
    uint32_t* flags_peer[kMaxRanks];  // AG: [world][blocks]; RS: [tiles][world]; values are call numbers
    const float* a;                   // AG: this rank's shard [mpr, K]; RS: [world * mpr, K]
    const float* b;                   // [N, K]
    float* out;                       // AG: [world * mpr, N]; RS: [mpr, N]
    int mpr, n, k, world, rank, pushers;
    uint32_t epoch;
    WaitCtx wctx;
};

__device__ __forceinline__ float dot(const float* x, const float* y, int k) {
    float acc = 0.f;
    for (int i = 0; i < k; ++i) acc += x[i] * y[i];
    return acc;
}

__global__ void ag_gemm_kernel(const OverlapParams p) {
    const int blocks = (p.mpr + TB - 1) / TB;                 // 16-row blocks per rank
    if (static_cast<int>(blockIdx.x) < p.pushers) {
        // ---------------- pusher: (peer, block) items, nearest consumer first
        for (int item = blockIdx.x; item < (p.world - 1) * blocks; item += p.pushers) {
            const int hop = item / blocks + 1, blk = item % blocks;
            const int dst = (p.rank - hop + p.world) % p.world;       // rank-1 reaches my rows first
            const int rows = min(TB, p.mpr - blk * TB);
            const float* src = p.a + static_cast<size_t>(blk) * TB * p.k;
            float* to = p.ws_peer[dst] + (static_cast<size_t>(p.rank) * p.mpr + blk * TB) * p.k;
            for (int i = threadIdx.x; i < rows * p.k; i += blockDim.x) to[i] = src[i];
            __syncthreads();                                          // all stores of the block issued ...
            if (threadIdx.x == 0) {
                fence_acq_rel_sys();                                  // ... and ordered before the flag, system-wide
                st_release_sys_u32(p.flags_peer[dst] + p.rank * blocks + blk, p.epoch);
            }
        }
        return;
    }
    // ---------------- consumer: tiles in (segment, row block, column tile) order, own segment first
    const int consumers = static_cast<int>(gridDim.x) - p.pushers;
    const int n_tiles = (p.n + TB - 1) / TB;
    const int tr = threadIdx.x / TB, tc = threadIdx.x % TB;           // 256 threads: one output element each
    for (int t = static_cast<int>(blockIdx.x) - p.pushers; t < p.world * blocks * n_tiles; t += consumers) {
        const int seg = (p.rank + t / (blocks * n_tiles)) % p.world;
        const int blk = (t / n_tiles) % blocks, nt = t % n_tiles;
        const float* rows;
        if (seg == p.rank) {
            rows = p.a + static_cast<size_t>(blk) * TB * p.k;         // own rows: never through the workspace
        } else {
            // the per-block wait: only THIS block of THIS source has to be here
            if (threadIdx.x == 0) wait_flag_ge_sys(p.flags_peer[p.rank] + seg * blocks + blk, p.epoch, p.wctx, seg, blk, 1);
            __syncthreads();
            // PRODUCTION: the rows are read by TMA (async proxy) next, so the kernel adds fence.proxy.async here
            rows = p.ws_peer[p.rank] + (static_cast<size_t>(seg) * p.mpr + blk * TB) * p.k;
        }
        const int r = blk * TB + tr, c = nt * TB + tc;
        if (r < p.mpr && c < p.n)
            p.out[(static_cast<size_t>(seg) * p.mpr + r) * p.n + c] = dot(rows + static_cast<size_t>(tr) * p.k, p.b + static_cast<size_t>(c) * p.k, p.k);
    }
}

__global__ void gemm_rs_kernel(const OverlapParams p) {
    const int blocks = (p.mpr + TB - 1) / TB, n_tiles = (p.n + TB - 1) / TB;
    const int tr = threadIdx.x / TB, tc = threadIdx.x % TB;
    // ---------------- produce: partial tiles, the segment after mine first, my own last
    for (int t = blockIdx.x; t < p.world * blocks * n_tiles; t += gridDim.x) {
        const int seg = (p.rank + 1 + t / (blocks * n_tiles)) % p.world;       // owner of these rows
        const int blk = (t / n_tiles) % blocks, nt = t % n_tiles;
        const int r = blk * TB + tr, c = nt * TB + tc;
        if (r < p.mpr && c < p.n) {
            const float v = dot(p.a + (static_cast<size_t>(seg) * p.mpr + r) * p.k, p.b + static_cast<size_t>(c) * p.k, p.k);
            // epilogue store straight into the owner's staging slot for this source, over NVLink
            p.ws_peer[seg][(static_cast<size_t>(p.rank) * p.mpr + r) * p.n + c] = v;
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            fence_acq_rel_sys();
            // PRODUCTION: the tile is written by TMA stores, so the kernel first waits for them (cp.async.bulk.wait_group)
            st_release_sys_u32(p.flags_peer[seg] + (blk * n_tiles + nt) * p.world + p.rank, p.epoch);
        }
    }
    // ---------------- reduce the tiles I own as their partials land
    const float* stage = p.ws_peer[p.rank];
    for (int t = blockIdx.x; t < blocks * n_tiles; t += gridDim.x) {
        if (static_cast<int>(threadIdx.x) < p.world)
            wait_flag_ge_sys(p.flags_peer[p.rank] + t * p.world + threadIdx.x, p.epoch, p.wctx, threadIdx.x, t, 2);
        __syncthreads();
        const int r = (t / n_tiles) * TB + tr, c = (t % n_tiles) * TB + tc;
        if (r < p.mpr && c < p.n) {
            float acc = 0.f;
            for (int s = 0; s < p.world; ++s) acc += *reinterpret_cast<const volatile float*>(stage + (static_cast<size_t>(s) * p.mpr + r) * p.n + c);
            p.out[static_cast<size_t>(r) * p.n + c] = acc;
        }
    }
}

// mode 0 = AG-GEMM, 1 = GEMM-RS. The grid never exceeds the SM count: CTAs of one launch wait for each other (RS) and
// for CTAs of the other ranks' launches, so all of them have to be resident.
extern "C" int tutorial_overlap_launch(int mode, void* const* ws_peer, void* const* flags_peer, const void* a, const void* b,
                                       void* out, int mpr, int n, int k, int rank, int world, int pushers, unsigned epoch,
                                       void* status, unsigned long long timeout_ns, void* stream) {
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || mpr < 1 || n < 1 || k < 1) return -1;
    OverlapParams p = {};
    for (int r = 0; r < world; ++r) {
        p.ws_peer[r] = static_cast<float*>(ws_peer[r]);
        p.flags_peer[r] = static_cast<uint32_t*>(flags_peer[r]);
    }
    p.a = static_cast<const float*>(a);
    p.b = static_cast<const float*>(b);
    p.out = static_cast<float*>(out);
    p.mpr = mpr;
    p.n = n;
    p.k = k;
    p.world = world;
    p.rank = rank;
    p.pushers = (mode == 0 && world > 1) ? (pushers > 0 ? pushers : 4) : 0;
    p.epoch = epoch;
    p.wctx.status = static_cast<Status*>(status);
    p.wctx.timeout_ns = timeout_ns;
    p.wctx.kernel_id = 102;
    p.wctx.rank = rank;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = sms > 8 ? sms - 4 : 4;
    if (mode == 0) ag_gemm_kernel<<<grid, TB * TB, 0, static_cast<cudaStream_t>(stream)>>>(p);
    else gemm_rs_kernel<<<grid, TB * TB, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
