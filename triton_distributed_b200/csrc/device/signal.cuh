// Cross-GPU signalling primitives: the CUDA restatement of the reference's `distributed`
// dialect ops (wait / consume_token / notify / symm_at / rank / num_ranks; reference
// python/triton_dist/language.py:57-112 and their NVPTX lowering in
// patches/triton/third_party/nvidia/lib/TritonNVIDIAGPUToLLVM/DistributedOpToLLVM.cpp:144-421)
// and of its raw-PTX helper set (ld / st / atomic_add / atomic_cas / red_release / wait_eq;
// patches/triton/third_party/nvidia/language/cuda/language_extra.py:244-558).
//
// Unlike the reference, no wait here is unbounded: every spin has a wall-clock limit
// (`%globaltimer`), after which the waiter records what it was waiting for in a status
// block, raises a sticky abort word that makes every later wait in the kernel return at
// once, and returns `false`. Callers carry on with whatever data is there (all memory they
// touch stays valid), so the kernel drains and the host raises from the status block.
#pragma once
#include <stdint.h>

#include "ptx.cuh"

namespace tdist {

constexpr int kMaxRanks = 8;

// One per process, in device memory (spin loops poll `abort`, so it must not sit behind PCIe);
// the host copies it back after the stream has been synchronised.
struct Status {
    int abort;       // sticky: non-zero once any wait gave up
    int code;        // kStatus*
    int kernel_id;   // which kernel family reported
    int rank;        // reporting rank
    int peer;        // peer / source the wait was on (or -1)
    int index;       // flag index / tile index
    long long expected;
    long long seen;
    int block;       // blockIdx.x of the reporter
    int where;       // call-site tag inside the kernel
    int reserved[4];
};

enum : int {
    kStatusOk = 0,
    kStatusFlagTimeout = 1,      // a cross-GPU or cross-CTA flag never reached its value
    kStatusMbarTimeout = 2,      // an mbarrier phase never completed
    kStatusBadArgument = 3,
};

struct WaitCtx {
    Status* status;        // may be nullptr (then nothing is recorded)
    uint64_t timeout_ns;   // 0 = use the default below
    int kernel_id;
    int rank;
};

constexpr uint64_t kDefaultTimeoutNs = 4000000000ull;

__device__ __forceinline__ bool aborted(const WaitCtx& w) {
    return w.status != nullptr && *reinterpret_cast<volatile int*>(&w.status->abort) != 0;
}

static __device__ __noinline__ void report_timeout(const WaitCtx& w, int code, int peer, int index,
                                            long long expected, long long seen, int where) {
    if (w.status == nullptr) return;
    if (atomicCAS(&w.status->abort, 0, 1) == 0) {
        w.status->code = code;
        w.status->kernel_id = w.kernel_id;
        w.status->rank = w.rank;
        w.status->peer = peer;
        w.status->index = index;
        w.status->expected = expected;
        w.status->seen = seen;
        w.status->block = static_cast<int>(blockIdx.x);
        w.status->where = where;
        __threadfence();
    }
}

// ---------------------------------------------------------------- scoped loads / stores
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t ld_acquire_sys_u64(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t ld_acquire_gpu_u64(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ uint64_t ld_relaxed_sys_u64(const uint64_t* p) {
    uint64_t v;
    asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u32(uint32_t* p, uint32_t v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys_u64(uint64_t* p, uint64_t v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_release_gpu_u64(uint64_t* p, uint64_t v) {
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u64(uint64_t* p, uint64_t v) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add_u32(uint32_t* p, uint32_t v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_gpu_add_u32(uint32_t* p, uint32_t v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add_u64(uint64_t* p, uint64_t v) {
    asm volatile("red.release.sys.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint32_t atom_add_acq_rel_gpu_u32(uint32_t* p, uint32_t v) {
    uint32_t old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ uint32_t atom_add_acq_rel_sys_u32(uint32_t* p, uint32_t v) {
    uint32_t old;
    asm volatile("atom.acq_rel.sys.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ uint32_t atom_cas_acq_rel_sys_u32(uint32_t* p, uint32_t cmp, uint32_t val) {
    uint32_t old;
    asm volatile("atom.acq_rel.sys.global.cas.b32 %0, [%1], %2, %3;"
                 : "=r"(old)
                 : "l"(p), "r"(cmp), "r"(val)
                 : "memory");
    return old;
}

// ---------------------------------------------------------------- bounded waits
// Comparison codes follow the reference's NVSHMEM_CMP_* numbering
// (patches/triton/python/triton/language/extra/libshmem_device.py:28-60).
enum : int { kCmpEq = 0, kCmpNe = 1, kCmpGt = 2, kCmpLe = 3, kCmpLt = 4, kCmpGe = 5 };

__device__ __forceinline__ bool cmp_holds(int cmp, long long seen, long long want) {
    switch (cmp) {
        case kCmpEq: return seen == want;
        case kCmpNe: return seen != want;
        case kCmpGt: return seen > want;
        case kCmpLe: return seen <= want;
        case kCmpLt: return seen < want;
        default: return seen >= want;
    }
}

// Spin until the 32-bit flag at `p` is at or past `epoch` (wrap-safe). System scope: the
// writer may be another GPU. Returns false if the wait was abandoned.
__device__ __forceinline__ bool wait_flag_ge_sys(const uint32_t* p, uint32_t epoch, const WaitCtx& w,
                                                 int peer, int index, int where) {
    uint32_t v = ld_acquire_sys_u32(p);
    if (static_cast<int32_t>(v - epoch) >= 0) return true;
    const uint64_t limit = w.timeout_ns ? w.timeout_ns : kDefaultTimeoutNs;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        v = ld_acquire_sys_u32(p);
        if (static_cast<int32_t>(v - epoch) >= 0) return true;
        __nanosleep(spins < 64 ? 20 : 200);
        if ((++spins & 63u) == 0) {
            if (aborted(w)) return false;
            if (globaltimer_ns() - t0 > limit) {
                report_timeout(w, kStatusFlagTimeout, peer, index, epoch, v, where);
                return false;
            }
        }
    }
}
// Same, GPU scope (writer is another CTA of this GPU).
__device__ __forceinline__ bool wait_flag_ge_gpu(const uint32_t* p, uint32_t epoch, const WaitCtx& w,
                                                 int peer, int index, int where) {
    uint32_t v = ld_acquire_gpu_u32(p);
    if (static_cast<int32_t>(v - epoch) >= 0) return true;
    const uint64_t limit = w.timeout_ns ? w.timeout_ns : kDefaultTimeoutNs;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        v = ld_acquire_gpu_u32(p);
        if (static_cast<int32_t>(v - epoch) >= 0) return true;
        __nanosleep(spins < 64 ? 20 : 200);
        if ((++spins & 63u) == 0) {
            if (aborted(w)) return false;
            if (globaltimer_ns() - t0 > limit) {
                report_timeout(w, kStatusFlagTimeout, peer, index, epoch, v, where);
                return false;
            }
        }
    }
}

// signal_wait_until on a 64-bit signal word (reference libshmem_device.signal_wait_until).
__device__ __forceinline__ bool signal_wait_until(const uint64_t* sig, int cmp, uint64_t value,
                                                  const WaitCtx& w, int peer = -1, int where = 0) {
    uint64_t v = ld_acquire_sys_u64(sig);
    if (cmp_holds(cmp, static_cast<long long>(v), static_cast<long long>(value))) return true;
    const uint64_t limit = w.timeout_ns ? w.timeout_ns : kDefaultTimeoutNs;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while (true) {
        v = ld_acquire_sys_u64(sig);
        if (cmp_holds(cmp, static_cast<long long>(v), static_cast<long long>(value))) return true;
        __nanosleep(spins < 64 ? 20 : 200);
        if ((++spins & 63u) == 0) {
            if (aborted(w)) return false;
            if (globaltimer_ns() - t0 > limit) {
                report_timeout(w, kStatusFlagTimeout, peer, 0, static_cast<long long>(value),
                               static_cast<long long>(v), where);
                return false;
            }
        }
    }
}

// Bounded mbarrier wait. A phase that never completes is a bug or the echo of an abandoned
// flag wait upstream; either way the waiter gives up after the same limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const WaitCtx& w, int where) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t limit = w.timeout_ns ? w.timeout_ns : kDefaultTimeoutNs;
    uint64_t t0 = 0;
    uint32_t spins = 0;
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((++spins & 255u) == 0) {
            if (aborted(w)) return false;
            const uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > limit) {
                report_timeout(w, kStatusMbarTimeout, -1, static_cast<int>(bar), parity, -1, where);
                return false;
            }
        }
    }
}

// Barrier of all CTAs of a grid that is fully resident (grid <= co-resident capacity). Thread 0 of
// each CTA adds to one 32-bit word: CTA 0 adds 0x80000000 - (n - 1), the others add 1, so a complete
// round adds exactly 0x80000000 — the top bit flips and the low bits return to where they were.
// Each CTA spins until the top bit differs from what its own add saw. Needs no reset and works
// when consecutive launches use different grid sizes.
// (reference kernels/nvidia/common_ops.py:62-85 `barrier_on_this_grid`)
__device__ __forceinline__ bool grid_barrier(uint32_t* counter, const WaitCtx& w) {
    __shared__ int ok_s;
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint32_t n = gridDim.x * gridDim.y * gridDim.z;
        const uint32_t me = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        const uint32_t old = atom_add_acq_rel_gpu_u32(counter, me == 0 ? 0x80000000u - (n - 1) : 1u);
        const uint64_t limit = w.timeout_ns ? w.timeout_ns : kDefaultTimeoutNs;
        const uint64_t t0 = globaltimer_ns();
        uint32_t spins = 0;
        int ok = 1;
        while (((old ^ ld_acquire_gpu_u32(counter)) & 0x80000000u) == 0) {
            __nanosleep(40);
            if ((++spins & 63u) == 0) {
                if (aborted(w)) { ok = 0; break; }
                if (globaltimer_ns() - t0 > limit) {
                    report_timeout(w, kStatusFlagTimeout, -1, static_cast<int>(me), old ^ 0x80000000u, old, 300);
                    ok = 0;
                    break;
                }
            }
        }
        ok_s = ok;
    }
    __syncthreads();
    return ok_s != 0;
}

// ---------------------------------------------------------------- dialect-level ops
// Table of the same symmetric allocation as seen from this process: base[r] is the address at
// which rank r's copy is mapped here (base[rank] is the local copy).
struct SymmWindow {
    char* base[kMaxRanks];
    int rank;
    int world;
    size_t bytes;   // size of the symmetric object (0 = not known: spans are then not checked)
    Status* dbg;    // where the bounds-checked build records a violation (may be nullptr)
};

// Bounds-checked build (-DTDIST_BOUNDS_CHECK, `TDIST_BOUNDS_CHECK=1` selects that library at load time): every
// translation of a symmetric address checks that the peer exists and that the span [offset, offset + len) lies inside
// the symmetric object. The first violation is recorded in the status block (kStatusBadArgument: peer, index = byte
// offset, expected = object size, seen = end of the span) and the access is SKIPPED: the translation returns nullptr
// and every helper of shmem.cuh returns without touching memory. Nothing traps, the context stays usable. This is the
// stand-in for running the kernels under a memory checker, which is not available where these kernels are developed.
constexpr int kKernelBounds = 8;
#ifdef TDIST_BOUNDS_CHECK
#define TDIST_SKIP_IF_NULL(ptr) \
    do {                        \
        if ((ptr) == nullptr) return; \
    } while (0)
#define TDIST_SKIP_IF_NULL_RET(ptr, value) \
    do {                                   \
        if ((ptr) == nullptr) return (value); \
    } while (0)
static __device__ __noinline__ void report_bounds(const SymmWindow& win, int peer, long long off, long long end, int where) {
    WaitCtx w;
    w.status = win.dbg;
    w.timeout_ns = 0;
    w.kernel_id = kKernelBounds;
    w.rank = win.rank;
    report_timeout(w, kStatusBadArgument, peer, static_cast<int>(off), static_cast<long long>(win.bytes), end, where);
}
template <typename T>
__device__ __forceinline__ T* symm_span(const SymmWindow& win, T* local_ptr, size_t len, int peer, int where = 0) {
    const ptrdiff_t off = reinterpret_cast<char*>(local_ptr) - win.base[win.rank];
    const bool bad_peer = peer < 0 || peer >= win.world;
    const bool bad_span = win.bytes != 0 && (off < 0 || static_cast<size_t>(off) + len > win.bytes);
    if (bad_peer || bad_span) {
        report_bounds(win, peer, off, off + static_cast<long long>(len), where);
        return nullptr;
    }
    return reinterpret_cast<T*>(win.base[peer] + off);
}
#else
#define TDIST_SKIP_IF_NULL(ptr) \
    do {                        \
    } while (0)
#define TDIST_SKIP_IF_NULL_RET(ptr, value) \
    do {                                   \
    } while (0)
template <typename T>
__device__ __forceinline__ T* symm_span(const SymmWindow& win, T* local_ptr, size_t len, int peer, int where = 0) {
    (void)len;
    (void)where;
    const ptrdiff_t off = reinterpret_cast<char*>(local_ptr) - win.base[win.rank];
    return reinterpret_cast<T*>(win.base[peer] + off);
}
#endif

// symm_at: translate a local symmetric address to the same offset in `peer`'s copy
// (reference language.py:96-100; lowering DistributedOpToLLVM.cpp:342-421).
template <typename T>
__device__ __forceinline__ T* symm_at(const SymmWindow& win, T* local_ptr, int peer) {
    return symm_span(win, local_ptr, sizeof(T), peer, 200);
}
__device__ __forceinline__ int rank(const SymmWindow& win) { return win.rank; }
__device__ __forceinline__ int num_ranks(const SymmWindow& win) { return win.world; }

enum : int { kSignalSet = 9, kSignalAdd = 10 };  // reference NVSHMEM_SIGNAL_SET / _ADD

// notify: one thread publishes `value` on `peer`'s signal word after making this thread's
// earlier writes visible system-wide (reference language.py:103-112; lowering :231-340 is
// `membar.sys; st.relaxed.sys` / `atom.add`). Call from a single thread after a CTA barrier
// when the data was written by the whole CTA.
__device__ __forceinline__ void notify(const SymmWindow& win, uint64_t* local_sig, int peer,
                                       uint64_t value, int sig_op) {
    uint64_t* remote = symm_at(win, local_sig, peer);
    TDIST_SKIP_IF_NULL(remote);
    fence_acq_rel_sys();
    if (sig_op == kSignalAdd) red_release_sys_add_u64(remote, value);
    else st_release_sys_u64(remote, value);
}

// wait: lanes [0, n) of the calling warp each poll one of n consecutive 64-bit words until it
// equals `value`; the warp re-converges before returning (reference language.py:57-71;
// lowering DistributedOpToLLVM.cpp:144-217). The return value plays the role of the token:
// feed it to consume_token() before touching the guarded data.
__device__ __forceinline__ bool wait(const uint64_t* sigs, int n, uint64_t value, const WaitCtx& w,
                                     int where = 0) {
    bool ok = true;
    const int lane = static_cast<int>(lane_id());
    for (int i = lane; i < n; i += 32) ok &= signal_wait_until(sigs + i, kCmpEq, value, w, i, where);
    ok = __all_sync(0xffffffffu, ok);
    return ok;
}
// consume_token: orders later accesses to `x` after the wait that produced `token`. The
// acquire loads inside wait() already order them for the generic proxy; when `x` is next
// read by TMA the async proxy needs its own fence, which is issued here.
template <typename T>
__device__ __forceinline__ T consume_token(T x, bool token) {
    (void)token;
    fence_proxy_async();
    return x;
}

}  // namespace tdist
