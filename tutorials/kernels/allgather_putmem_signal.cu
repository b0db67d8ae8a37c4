// Tutorial 02: a push all-gather written with the OpenSHMEM-style device API of device/shmem.cuh.
//
// One CTA per destination: CTA g of rank r copies r's segment into slot r of rank (r + g)'s copy of the symmetric buffer
// with putmem_signal_block, which raises that rank's signal word `r` to the call number once the data is ordered before
// it. Then every rank waits (signal_wait_until, bounded) until all of its own signal words carry the call number.
// (reference tutorials/02-intra-node-allgather.py and kernels/nvidia/low_latency_allgather.py:345-397, the same
// protocol with libshmem_device.putmem_signal_block / signal_wait_until in a Triton kernel)
#include <cuda_runtime.h>

#include "device/shmem.cuh"

using namespace tdist;

struct GatherParams {
    SymmWindow buf_win, sig_win;
    char* buf;         // local symmetric [world][seg_bytes]
    uint64_t* sig;     // local symmetric [world]
    size_t seg_bytes;
    uint64_t epoch;
    WaitCtx wctx;
};

__global__ void allgather_kernel(const GatherParams p) {
    const int rank = my_pe(p.buf_win), world = n_pes(p.buf_win);
    const int peer = (rank + static_cast<int>(blockIdx.x)) % world;
    char* mine = p.buf + static_cast<size_t>(rank) * p.seg_bytes;
    // dst and sig are LOCAL symmetric addresses; the helper translates them into `peer`'s copy
    if (peer != rank) putmem_signal_block(p.buf_win, mine, mine, p.seg_bytes, p.sig_win, p.sig + rank, p.epoch, kSignalSet, peer);
    if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < world && static_cast<int>(threadIdx.x) != rank)
        signal_wait_until(p.sig + threadIdx.x, kCmpGe, p.epoch, p.wctx, threadIdx.x, 1);
}

extern "C" int tutorial_allgather_launch(void* const* buf_peer, void* const* sig_peer, int rank, int world,
                                         unsigned long long seg_bytes, unsigned long long epoch, void* status,
                                         unsigned long long timeout_ns, void* stream) {
    if (world < 1 || world > kMaxRanks || rank < 0 || rank >= world) return -1;
    GatherParams p = {};
    for (int r = 0; r < world; ++r) {
        p.buf_win.base[r] = static_cast<char*>(buf_peer[r]);
        p.sig_win.base[r] = static_cast<char*>(sig_peer[r]);
    }
    p.buf_win.rank = p.sig_win.rank = rank;
    p.buf_win.world = p.sig_win.world = world;
    p.buf_win.bytes = static_cast<size_t>(world) * seg_bytes;
    p.sig_win.bytes = static_cast<size_t>(world) * sizeof(uint64_t);
    p.buf_win.dbg = p.sig_win.dbg = static_cast<Status*>(status);
    p.buf = static_cast<char*>(buf_peer[rank]);
    p.sig = static_cast<uint64_t*>(sig_peer[rank]);
    p.seg_bytes = seg_bytes;
    p.epoch = epoch;
    p.wctx.status = static_cast<Status*>(status);
    p.wctx.timeout_ns = timeout_ns;
    p.wctx.kernel_id = 101;
    p.wctx.rank = rank;
    allgather_kernel<<<world, 512, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
