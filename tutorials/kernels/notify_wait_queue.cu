// Tutorial 01: a producer / consumer queue between neighbouring ranks, written with the dialect-level primitives
// of device/signal.cuh: wait, consume_token, notify, symm_at.
//
// Rank r's PRODUCER CTAs stream the tiles of `input` into a small ring of slots that lives in rank r+1's symmetric
// memory; rank r+1's CONSUMER CTAs take them out. Both kinds of CTA run in ONE launch per rank (they must be
// co-resident: they wait for each other), and the ring is shorter than the stream, so the two sides really run in
// lockstep:
//
//      producer (rank r)                                 consumer (rank r+1)
//      wait  empty[slot] == round            <----------  notify(empty[slot] on r, round + 1)   "slot drained"
//      store tile -> symm_at(queue, r+1)
//      notify(full[slot] on r+1, round + 1)  ---------->  wait  full[slot] == round + 1
//                                                         consume_token(queue + slot, token); use the tile
//
// Every flag is a 64-bit word that only grows (base + round + 1): nothing is ever reset, so a second launch can start
// while a slow neighbour is still finishing the first. Every wait is bounded: if a neighbour never shows up, the
// waiter records what it was waiting for in the status block and the kernel drains.
// (reference tutorials/01-distributed-notify-wait.py:64-133: the same queue as a Triton kernel)
#include <cuda_runtime.h>

#include "device/signal.cuh"

using namespace tdist;

struct QueueParams {
    SymmWindow data_win;   // window of `queue`
    SymmWindow flag_win;   // window of `flags`
    float* queue;          // local symmetric [slots][tile]
    uint64_t* full;        // local symmetric [slots]: written by the producer of rank-1
    uint64_t* empty;       // local symmetric [slots]: written by the consumer of rank+1
    const float* input;    // [n_tiles][tile] what this rank sends
    float* output;         // [n_tiles][tile] what this rank receives, doubled
    int n_tiles, tile, slots, producers, consumers;
    uint64_t base;         // flag value the previous launch ended at
    WaitCtx wctx;
};

__global__ void queue_kernel(const QueueParams p) {
    const int next = (p.data_win.rank + 1) % p.data_win.world;
    const int prev = (p.data_win.rank + p.data_win.world - 1) % p.data_win.world;
    const bool warp0 = threadIdx.x < 32;
    if (static_cast<int>(blockIdx.x) < p.producers) {
        // ---------------- producer: tiles blockIdx.x, blockIdx.x + producers, ...
        for (int t = blockIdx.x; t < p.n_tiles; t += p.producers) {
            const int slot = t % p.slots;
            const uint64_t round = static_cast<uint64_t>(t / p.slots);
            if (round > 0) {
                // the consumer on `next` has drained what this slot held one round ago
                if (warp0) wait(p.empty + slot, 1, p.base + round, p.wctx, 1);
                __syncthreads();
            }
            float* remote = symm_at(p.data_win, p.queue + static_cast<size_t>(slot) * p.tile, next);
            for (int i = threadIdx.x; i < p.tile; i += blockDim.x) remote[i] = p.input[static_cast<size_t>(t) * p.tile + i];
            __syncthreads();   // the whole tile is stored before one thread publishes it
            if (threadIdx.x == 0) notify(p.flag_win, p.full + slot, next, p.base + round + 1, kSignalSet);
        }
    } else {
        // ---------------- consumer: tiles c, c + consumers, ...
        const int c = static_cast<int>(blockIdx.x) - p.producers;
        for (int t = c; t < p.n_tiles; t += p.consumers) {
            const int slot = t % p.slots;
            const uint64_t round = static_cast<uint64_t>(t / p.slots);
            __shared__ int token_s;
            if (warp0) {
                const bool token = wait(p.full + slot, 1, p.base + round + 1, p.wctx, 2);
                if (threadIdx.x == 0) token_s = token ? 1 : 0;
            }
            __syncthreads();
            // consume_token ties the data to the wait that guards it (and fences the async proxy for TMA readers)
            const float* tile = consume_token(p.queue + static_cast<size_t>(slot) * p.tile, token_s != 0);
            for (int i = threadIdx.x; i < p.tile; i += blockDim.x)
                p.output[static_cast<size_t>(t) * p.tile + i] = token_s ? 2.f * *reinterpret_cast<const volatile float*>(tile + i) : -1.f;
            __syncthreads();   // every thread has read the slot before it is handed back
            if (threadIdx.x == 0) notify(p.flag_win, p.empty + slot, prev, p.base + round + 1, kSignalSet);
        }
    }
}

// queue_peer[r] / flags_peer[r]: rank r's copy of the symmetric queue ([slots * tile] fp32) and flags (2 * slots
// uint64: full, then empty) as mapped into this process. Returns the flag value this launch ends at (pass it as `base`
// of the next launch), or 0 on a bad argument.
extern "C" unsigned long long tutorial_queue_launch(void* const* queue_peer, void* const* flags_peer, int rank, int world,
                                                    const void* input, void* output, int n_tiles, int tile, int slots,
                                                    int producers, int consumers, unsigned long long base, void* status,
                                                    unsigned long long timeout_ns, void* stream) {
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world || slots < 1 || producers < 1 || consumers < 1 ||
        producers > slots)
        return 0;   // more producers than slots would let two of them fill one slot in the same round
    QueueParams p = {};
    for (int r = 0; r < world; ++r) {
        p.data_win.base[r] = static_cast<char*>(queue_peer[r]);
        p.flag_win.base[r] = static_cast<char*>(flags_peer[r]);
    }
    p.data_win.rank = p.flag_win.rank = rank;
    p.data_win.world = p.flag_win.world = world;
    p.data_win.bytes = static_cast<size_t>(slots) * tile * sizeof(float);
    p.flag_win.bytes = static_cast<size_t>(2 * slots) * sizeof(uint64_t);
    p.data_win.dbg = p.flag_win.dbg = static_cast<Status*>(status);
    p.queue = static_cast<float*>(queue_peer[rank]);
    p.full = static_cast<uint64_t*>(flags_peer[rank]);
    p.empty = p.full + slots;
    p.input = static_cast<const float*>(input);
    p.output = static_cast<float*>(output);
    p.n_tiles = n_tiles;
    p.tile = tile;
    p.slots = slots;
    p.producers = producers;
    p.consumers = consumers;
    p.base = base;
    p.wctx.status = static_cast<Status*>(status);
    p.wctx.timeout_ns = timeout_ns;
    p.wctx.kernel_id = 100;   // user kernels: any id the status table does not know prints as a number
    p.wctx.rank = rank;
    queue_kernel<<<producers + consumers, 128, 0, static_cast<cudaStream_t>(stream)>>>(p);
    if (cudaGetLastError() != cudaSuccess) return 0;
    return base + static_cast<unsigned long long>((n_tiles + slots - 1) / slots);
}
