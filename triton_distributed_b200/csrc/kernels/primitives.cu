// One small kernel per device primitive, so that every function of signal.cuh / shmem.cuh can be
// driven and checked from the host (and serves as a usage example). Mirrors what the reference
// tests exercise through Triton kernels: test_notify.py (ring set, add-to-rank-0), test_ring_put.py
// (int_p), test_nvshmem_api.py (put / get / putmem_signal at thread, warp and block scope,
// signal_op + signal_wait_until, fence / quiet, barrier, broadcast, fcollect), test_common_ops.py
// (grid barrier).
//
// Ops that wait take a `phase`: 1 = the sending half, 2 = the waiting / checking half, 3 = both.
// With one process per GPU a test passes 3; with all ranks emulated on one GPU it runs phase 1 on
// every rank first, so that no launch ever waits for a launch that has not run.
#include <cuda_runtime.h>

#include "../device/language_extra.cuh"
#include "../device/shmem.cuh"
#include "../include/tdist.h"
#include "../runtime/host_common.h"

namespace tdist {

constexpr int kKernelPrim = 5;

struct PrimParams {
    SymmWindow win;     // window of `data`
    SymmWindow sigwin;  // window of `sig`
    char* data;         // local symmetric buffer, >= (world + 2) * nbytes
    uint64_t* sig;      // local symmetric uint64[16]
    int* result;        // local (non-symmetric) int[8]: op-specific check results
    uint32_t* grid_counter;
    BarrierState barrier;
    int op, phase, nbytes, scope;
    uint64_t value;
    WaitCtx wctx;
};

// data layout: slot s occupies [s * nbytes, (s + 1) * nbytes). Slot `world` is the local source.
__device__ __forceinline__ char* slot(const PrimParams& p, int s) { return p.data + static_cast<size_t>(s) * p.nbytes; }

__global__ void prim_kernel(const PrimParams p) {
    const int rank = p.win.rank, world = p.win.world;
    const int next = (rank + 1) % world, prev = (rank + world - 1) % world;
    const bool t0 = threadIdx.x == 0 && blockIdx.x == 0;
    switch (p.op) {
        case TDIST_PRIM_RING_PUT:  // int_p: write my rank into the next rank's slot 0
            if ((p.phase & 1) && t0) int_p(p.win, reinterpret_cast<int*>(slot(p, 0)), rank + 100, next);
            break;
        case TDIST_PRIM_NOTIFY_WAIT:  // ring: notify(next, value) ; wait for prev's notify
            if ((p.phase & 1) && t0) {
                *reinterpret_cast<volatile int*>(symm_at(p.win, reinterpret_cast<int*>(slot(p, 0)), next)) = rank + 7;
                notify(p.sigwin, p.sig, next, p.value, kSignalSet);
            }
            if ((p.phase & 2) && blockIdx.x == 0 && threadIdx.x < 32) {
                const bool token = wait(p.sig, 1, p.value, p.wctx, 1);
                int* guarded = consume_token(reinterpret_cast<int*>(slot(p, 0)), token);
                if (threadIdx.x == 0) {
                    p.result[0] = token ? 1 : 0;
                    p.result[1] = *reinterpret_cast<volatile int*>(guarded);  // must be prev + 7
                }
            }
            break;
        case TDIST_PRIM_NOTIFY_ADD:  // every rank adds 1 on rank 0's signal; rank 0 waits for world
            if ((p.phase & 1) && t0) notify(p.sigwin, p.sig + 1, 0, 1, kSignalAdd);
            if ((p.phase & 2) && t0 && rank == 0)
                p.result[0] = signal_wait_until(p.sig + 1, kCmpGe, p.value, p.wctx, -1, 2) ? 1 : 0;
            break;
        case TDIST_PRIM_PUT_SIGNAL: {  // putmem_signal at the requested scope into next's slot `rank`
            if (p.phase & 1) {
                if (p.scope == 0) {
                    if (t0) putmem_signal(p.win, slot(p, rank), slot(p, world), p.nbytes, p.sigwin, p.sig + 2, p.value, kSignalSet, next);
                } else if (p.scope == 1) {
                    if (blockIdx.x == 0 && threadIdx.x < 32)
                        putmem_signal_warp(p.win, slot(p, rank), slot(p, world), p.nbytes, p.sigwin, p.sig + 2, p.value, kSignalSet, next);
                } else if (blockIdx.x == 0) {
                    putmem_signal_block(p.win, slot(p, rank), slot(p, world), p.nbytes, p.sigwin, p.sig + 2, p.value, kSignalSet, next);
                }
            }
            if ((p.phase & 2) && t0) p.result[0] = signal_wait_until(p.sig + 2, kCmpEq, p.value, p.wctx, prev, 3) ? 1 : 0;
            break;
        }
        case TDIST_PRIM_PUT_QUIET_SIGNAL:  // putmem_nbi_block ; quiet ; signal_op(ADD) — the explicit form
            if ((p.phase & 1) && blockIdx.x == 0) {
                putmem_nbi_block(p.win, slot(p, rank), slot(p, world), p.nbytes, next);
                quiet();
                __syncthreads();
                if (threadIdx.x == 0) {
                    fence();
                    signal_op(p.sigwin, p.sig + 3, p.value, kSignalAdd, next);
                }
            }
            if ((p.phase & 2) && t0) p.result[0] = signal_wait_until(p.sig + 3, kCmpGe, p.value, p.wctx, prev, 4) ? 1 : 0;
            break;
        case TDIST_PRIM_GET:  // getmem at the requested scope: pull prev's source slot into my slot `prev`
            if ((p.phase & 2) && blockIdx.x == 0) {
                if (p.scope == 0) {
                    if (threadIdx.x == 0) getmem_nbi(p.win, slot(p, prev), slot(p, world), p.nbytes, prev);
                } else if (p.scope == 1) {
                    if (threadIdx.x < 32) getmem_nbi_warp(p.win, slot(p, prev), slot(p, world), p.nbytes, prev);
                } else {
                    getmem_block(p.win, slot(p, prev), slot(p, world), p.nbytes, prev);
                }
            }
            break;
        case TDIST_PRIM_BROADCAST:  // root 0's source slot lands in everybody's slot 0, then a barrier of the same scope
            if ((p.phase & 1) && blockIdx.x == 0) {
                if (p.scope == 0) {
                    if (threadIdx.x == 0) broadcast(p.win, slot(p, 0), slot(p, world), p.nbytes, 0);
                } else if (p.scope == 1) {
                    if (threadIdx.x < 32) broadcast_warp(p.win, slot(p, 0), slot(p, world), p.nbytes, 0);
                } else {
                    broadcast_block(p.win, slot(p, 0), slot(p, world), p.nbytes, 0);
                }
            }
            if (p.phase == 3 && blockIdx.x == 0) {
                if (p.scope == 0) {
                    if (threadIdx.x == 0) p.result[0] = barrier_all(p.sigwin, p.barrier, p.wctx) ? 1 : 0;
                } else if (p.scope == 1) {
                    if (threadIdx.x < 32) {
                        const bool ok = sync_all_warp(p.sigwin, p.barrier, p.wctx);
                        if (threadIdx.x == 0) p.result[0] = ok ? 1 : 0;
                    }
                } else {
                    p.result[0] = barrier_all_block(p.sigwin, p.barrier, p.wctx) ? 1 : 0;
                }
            }
            break;
        case TDIST_PRIM_FCOLLECT:  // everybody's source slot lands in slot `rank` of everybody
            if ((p.phase & 1) && blockIdx.x == 0) {
                if (p.scope == 0) {
                    if (threadIdx.x == 0) fcollect(p.win, slot(p, 0), slot(p, world), p.nbytes);
                } else if (p.scope == 1) {
                    if (threadIdx.x < 32) fcollect_warp(p.win, slot(p, 0), slot(p, world), p.nbytes);
                } else {
                    fcollect_block(p.win, slot(p, 0), slot(p, world), p.nbytes);
                }
            }
            if (p.phase == 3 && blockIdx.x == 0) {
                if (p.scope == 0) {
                    if (threadIdx.x == 0) p.result[0] = sync_all(p.sigwin, p.barrier, p.wctx) ? 1 : 0;
                } else if (p.scope == 1) {
                    if (threadIdx.x < 32) {
                        const bool ok = barrier_all_warp(p.sigwin, p.barrier, p.wctx);
                        if (threadIdx.x == 0) p.result[0] = ok ? 1 : 0;
                    }
                } else {
                    p.result[0] = barrier_all_block(p.sigwin, p.barrier, p.wctx) ? 1 : 0;
                }
            }
            break;
        case TDIST_PRIM_BARRIER:  // barrier_all at the requested scope, `value` rounds back to back
            if (p.phase == 3 && blockIdx.x == 0) {
                int fails = 0;
                for (uint64_t it = 0; it < p.value; ++it) {
                    bool ok = true;
                    if (p.scope == 0) {
                        if (threadIdx.x == 0) ok = barrier_all(p.sigwin, p.barrier, p.wctx);
                    } else if (p.scope == 1) {
                        if (threadIdx.x < 32) ok = barrier_all_warp(p.sigwin, p.barrier, p.wctx);
                    } else {
                        ok = barrier_all_block(p.sigwin, p.barrier, p.wctx);
                    }
                    fails += ok ? 0 : 1;
                }
                if (threadIdx.x == 0) p.result[0] = fails;
            }
            break;
#ifdef TDIST_BOUNDS_CHECK
        case TDIST_PRIM_BOUNDS_PROBE:
            // Three accesses that leave the symmetric object or name a rank that does not exist. The checked
            // translation records the first and skips all of them; result[1] counts what was skipped.
            if (t0) {
                int skipped = 0;
                // (a) a put whose span runs 16 bytes past the end of the object
                char* last = slot(p, world + 1);
                if (symm_span(p.win, last, static_cast<size_t>(p.nbytes) + 16, next, 1) == nullptr) ++skipped;
                putmem(p.win, last, slot(p, world), static_cast<size_t>(p.nbytes) + 16, next);
                // (b) a single-element put to rank `world`
                if (symm_at(p.win, reinterpret_cast<int*>(slot(p, 0)), world) == nullptr) ++skipped;
                int_p(p.win, reinterpret_cast<int*>(slot(p, 0)), 12345, world);
                // (c) a signal on a word past the signal array
                if (symm_at(p.sigwin, p.sig + 16, next) == nullptr) ++skipped;
                signal_op(p.sigwin, p.sig + 16, 1, kSignalSet, next);
                p.result[1] = skipped;
            }
            break;
#endif
        case TDIST_PRIM_GRID_BARRIER: {  // every CTA publishes, all meet, every CTA reads its neighbour
            int* buf = reinterpret_cast<int*>(slot(p, 0));
            if (threadIdx.x == 0) buf[blockIdx.x] = static_cast<int>(blockIdx.x) + static_cast<int>(p.value);
            const bool ok = grid_barrier(p.grid_counter, p.wctx);
            if (threadIdx.x == 0) {
                const int nb = (blockIdx.x + 1) % gridDim.x;
                const int seen = *reinterpret_cast<volatile int*>(buf + nb);
                if (!ok || seen != nb + static_cast<int>(p.value)) atomicAdd(p.result, 1);  // counts failures
            }
            break;
        }
        case TDIST_PRIM_SCOPED_OPS: {
            // The scoped load / store / atomic helpers and warp intrinsics, in the spirit of the reference's
            // test_language_extra.py: all counters live in slot 0 (uint32 words), zeroed by the host.
            //   word 0: every thread adds 1 (red.release.gpu)           -> grid * block
            //   word 1: lane 0 of every warp adds 32 (atom.acq_rel.gpu) -> grid * block
            //   word 2: CAS lock (0 free / 1 taken); word 3: plain counter incremented under the lock by thread 0
            //           of every CTA                                      -> grid
            //   word 4: st.release.gpu / ld.acquire.gpu hand-over inside the CTA; word 5: warps whose ballot / shuffle
            //           results were right                                -> grid * block / 32
            uint32_t* w = reinterpret_cast<uint32_t*>(slot(p, 0));
            red_release_gpu_add_u32(w + 0, 1u);
            language_extra::atomic_add_per_warp(w + 1, 32u, language_extra::kScopeGpu);  // lane 0 adds for its warp
            if (threadIdx.x == 0) {
                bool got = false;
                for (int spin = 0; spin < (1 << 22) && !got; ++spin) got = atom_cas_acq_rel_sys_u32(w + 2, 0u, 1u) == 0u;
                if (got) {
                    *reinterpret_cast<volatile uint32_t*>(w + 3) = *reinterpret_cast<volatile uint32_t*>(w + 3) + 1u;
                    st_release_gpu_u32(w + 2, 0u);
                } else {
                    atomicAdd(p.result, 1);  // lock never obtained
                }
            }
            const int ln = static_cast<int>(threadIdx.x & 31);
            const unsigned ballot = language_extra::ballot_sync(0xffffffffu, (threadIdx.x & 1) != 0);
            int sum = ln;
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            const int up = language_extra::shfl_up_sync_i32(0xffffffffu, ln, 1);
            const int down = language_extra::shfl_down_sync_i32(0xffffffffu, ln, 2);
            const int from7 = language_extra::shfl_sync_i32(0xffffffffu, ln * 3, 7);
            const bool warp_ok = ballot == 0xaaaaaaaau && sum == 496 && (ln == 0 || up == ln - 1) && (ln >= 30 || down == ln + 2) && from7 == 21;
            if (__all_sync(0xffffffffu, warp_ok) && (threadIdx.x & 31) == 0) red_release_gpu_add_u32(w + 5, 1u);
            break;
        }
        default: break;
    }
}

// Never launched: instantiates every helper of language_extra.cuh so that ptxas checks their PTX at build time.
__global__ void language_extra_compile_check(uint32_t* a, uint64_t* b, void* mc, WaitCtx w) {
    namespace le = language_extra;
    uint32_t acc = le::tid(0) + le::ntid(0) + le::laneid();
    le::fence_sc(le::kScopeGpu);
    le::fence_sc(le::kScopeSys);
    acc += le::ld(a, le::kScopeSys, le::kAcquire) + le::ld_acquire(a, le::kScopeGpu) + static_cast<uint32_t>(le::ld(b, le::kScopeGpu, le::kRelaxed));
    le::st(a, acc, le::kScopeSys, le::kRelease);
    le::st(b, acc, le::kScopeGpu, le::kRelaxed);
    acc += le::atomic_add(a, 1u, le::kScopeSys) + le::atomic_cas(a, 0u, 1u) + le::atomic_add_per_warp(a, 1u, le::kScopeGpu);
    le::red_release(a, 1u, le::kScopeSys);
    le::arrive_inc(a, 0, 1u, le::kScopeGpu);
    acc += le::wait_eq(b, 1, w) ? 1u : 0u;
    const uint4 v4 = le::load_v4_u32(a);
    const ulonglong2 v2 = le::load_v2_b64(b);
    le::store_v2_u32(a, v4.x + static_cast<uint32_t>(v2.x), acc);
    le::multimem_st_b32(mc, acc);
    le::multimem_st_b64(mc, v2.y);
    le::multimem_st_v2_b32(mc, v4.y, v4.z);
}
// Likewise for the warp- and thread-scope forms of shmem.cuh that no test op launches.
__global__ void shmem_scopes_compile_check(SymmWindow win, BarrierState st, char* mc_base, char* buf, size_t bytes, WaitCtx w) {
    getmem_nbi(win, buf, buf + bytes, bytes, 0);
    broadcast_warp(win, buf, buf + bytes, bytes, 0);
    broadcast(win, buf, buf + bytes, bytes, 0);
    broadcastmem_block(win, buf, buf + bytes, bytes, 0);
    fcollect_warp(win, buf, buf + bytes, bytes);
    fcollect(win, buf, buf + bytes, bytes);
    bool ok = barrier_all_warp(win, st, w) && barrier_all(win, st, w) && sync_all_warp(win, st, w) && sync_all(win, st, w);
    if (ok) language_extra::multimem_st_b32(remote_mc_ptr(win, mc_base, reinterpret_cast<int*>(buf)), 0u);
}

}  // namespace tdist

using namespace tdist;

extern "C" int tdist_bounds_checked(void) {
#ifdef TDIST_BOUNDS_CHECK
    return 1;
#else
    return 0;
#endif
}

extern "C" int tdist_primitive(const TdistPrimArgs* a) {
    if (a->world < 1 || a->world > TDIST_MAX_RANKS || a->rank < 0 || a->rank >= a->world)
        return tdist_host::fail(TDIST_EINVAL, "primitive: world/rank out of range");
    if (a->op < 0 || a->op > TDIST_PRIM_BOUNDS_PROBE) return tdist_host::fail(TDIST_EINVAL, "primitive: unknown op");
#ifndef TDIST_BOUNDS_CHECK
    if (a->op == TDIST_PRIM_BOUNDS_PROBE)
        return tdist_host::fail(TDIST_EINVAL, "primitive: the bounds probe only exists in the bounds-checked build (TDIST_BOUNDS_CHECK=1)");
#endif
    PrimParams p;
    memset(&p, 0, sizeof(p));
    for (int r = 0; r < a->world; ++r) {
        p.win.base[r] = static_cast<char*>(a->data_peer[r]);
        p.sigwin.base[r] = static_cast<char*>(a->sig_peer[r]);
        if (!p.win.base[r] || !p.sigwin.base[r]) return tdist_host::fail(TDIST_EINVAL, "primitive: null peer pointer");
    }
    p.win.rank = p.sigwin.rank = a->rank;
    p.win.world = p.sigwin.world = a->world;
    p.win.bytes = static_cast<size_t>(a->world + 2) * static_cast<size_t>(a->nbytes > 0 ? a->nbytes : 0);
    p.sigwin.bytes = 16 * sizeof(uint64_t);
    p.win.dbg = p.sigwin.dbg = static_cast<Status*>(a->status);
    p.data = p.win.base[a->rank];
    p.sig = reinterpret_cast<uint64_t*>(p.sigwin.base[a->rank]);
    p.result = static_cast<int*>(a->result);
    p.grid_counter = static_cast<uint32_t*>(a->grid_counter);
    p.barrier.flags = p.sig + 8;  // words 8..15 of the signal array are the barrier's flags
    p.barrier.epoch = static_cast<uint64_t*>(a->barrier_epoch);
    p.op = a->op;
    p.phase = a->phase ? a->phase : 3;
    p.nbytes = a->nbytes;
    p.scope = a->scope;
    p.value = a->value;
    p.wctx.status = static_cast<Status*>(a->status);
    p.wctx.timeout_ns = a->timeout_ns;
    p.wctx.kernel_id = kKernelPrim;
    p.wctx.rank = a->rank;
    const int grid = (a->op == TDIST_PRIM_GRID_BARRIER || a->op == TDIST_PRIM_SCOPED_OPS) ? (a->grid > 0 ? a->grid : 64) : 1;
    prim_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(a->stream)>>>(p);
    TDIST_CUDA_OK(cudaGetLastError());
    return 0;
}
