// OpenSHMEM-style device primitives over peer-mapped symmetric memory: the CUDA restatement
// of the reference's `libshmem_device` surface (my_pe / n_pes / int_p / remote_ptr /
// putmem[_nbi][_block|_warp] / getmem* / putmem_signal* / signal_op / signal_wait_until /
// fence / quiet / barrier_all* / sync_all* / broadcast* / fcollect*; reference
// patches/triton/third_party/nvidia/language/cuda/libnvshmem_device.py:85-1001 and the NVSHMEM
// trampolines in shmem/nvshmem_bind/runtime/nvshmem_wrapper.cu:26-695).
//
// There is no NVSHMEM underneath: a "PE" is a rank of the node, a remote address is the same
// offset inside that rank's mapping of the symmetric object (SymmWindow), and every transfer
// is plain ld/st (or TMA bulk copies in the GEMM kernels) over NVLink. All puts are
// non-blocking in the NVSHMEM sense (stores are posted); `quiet()` / `fence()` order them
// before later signals. Waits are bounded (signal.cuh).
#pragma once
#include "signal.cuh"

namespace tdist {

__device__ __forceinline__ int my_pe(const SymmWindow& w) { return w.rank; }
__device__ __forceinline__ int n_pes(const SymmWindow& w) { return w.world; }

template <typename T>
__device__ __forceinline__ T* remote_ptr(const SymmWindow& w, T* local, int pe) {
    return symm_at(w, local, pe);
}

// Orders this thread's earlier puts before its later puts / signals, system-wide.
__device__ __forceinline__ void fence() { fence_acq_rel_sys(); }
// Completes this thread's earlier puts (same mechanism on NVLink: a system-scope fence).
__device__ __forceinline__ void quiet() { fence_acq_rel_sys(); }

__device__ __forceinline__ uint4 ld_nc_v4(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_v4(void* p, const uint4& v) {
    asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// Cooperative copy by `nthreads` threads (`tid` in [0, nthreads)): 16-byte vectors when both
// pointers allow, bytes otherwise. Either side may be peer memory.
__device__ __forceinline__ void copy_coop(void* dst, const void* src, size_t bytes, int tid, int nthreads) {
    char* d = static_cast<char*>(dst);
    const char* s = static_cast<const char*>(src);
    if (((reinterpret_cast<uintptr_t>(d) | reinterpret_cast<uintptr_t>(s)) & 15u) == 0) {
        const size_t nvec = bytes >> 4;
        size_t i = tid;
        for (; i + 3 * static_cast<size_t>(nthreads) < nvec; i += 4 * static_cast<size_t>(nthreads)) {
            const uint4 a = ld_nc_v4(s + (i << 4));
            const uint4 b = ld_nc_v4(s + ((i + nthreads) << 4));
            const uint4 c = ld_nc_v4(s + ((i + 2 * static_cast<size_t>(nthreads)) << 4));
            const uint4 e = ld_nc_v4(s + ((i + 3 * static_cast<size_t>(nthreads)) << 4));
            st_v4(d + (i << 4), a);
            st_v4(d + ((i + nthreads) << 4), b);
            st_v4(d + ((i + 2 * static_cast<size_t>(nthreads)) << 4), c);
            st_v4(d + ((i + 3 * static_cast<size_t>(nthreads)) << 4), e);
        }
        for (; i < nvec; i += nthreads) st_v4(d + (i << 4), ld_nc_v4(s + (i << 4)));
        for (size_t b = (nvec << 4) + tid; b < bytes; b += nthreads) d[b] = s[b];
    } else {
        for (size_t b = tid; b < bytes; b += nthreads) d[b] = s[b];
    }
}

// ---- put / get: `dst` and `src` are LOCAL symmetric addresses; the remote side is `pe`'s copy.
__device__ __forceinline__ void putmem_block(const SymmWindow& w, void* dst, const void* src, size_t bytes, int pe) {
    char* remote = symm_span(w, static_cast<char*>(dst), bytes, pe, 201);
    TDIST_SKIP_IF_NULL(remote);
    copy_coop(remote, src, bytes, threadIdx.x, blockDim.x);
}
__device__ __forceinline__ void putmem_warp(const SymmWindow& w, void* dst, const void* src, size_t bytes, int pe) {
    char* remote = symm_span(w, static_cast<char*>(dst), bytes, pe, 202);
    TDIST_SKIP_IF_NULL(remote);
    copy_coop(remote, src, bytes, lane_id(), 32);
}
__device__ __forceinline__ void putmem(const SymmWindow& w, void* dst, const void* src, size_t bytes, int pe) {
    char* remote = symm_span(w, static_cast<char*>(dst), bytes, pe, 203);
    TDIST_SKIP_IF_NULL(remote);
    copy_coop(remote, src, bytes, 0, 1);
}
// The *_nbi forms are the same code: stores to peer memory never block the issuing thread.
__device__ __forceinline__ void putmem_nbi_block(const SymmWindow& w, void* dst, const void* src, size_t bytes, int pe) {
    putmem_block(w, dst, src, bytes, pe);
}
__device__ __forceinline__ void putmem_nbi_warp(const SymmWindow& w, void* dst, const void* src, size_t bytes, int pe) {
    putmem_warp(w, dst, src, bytes, pe);
}
__device__ __forceinline__ void putmem_nbi(const SymmWindow& w, void* dst, const void* src, size_t bytes, int pe) {
    putmem(w, dst, src, bytes, pe);
}
__device__ __forceinline__ void getmem_block(const SymmWindow& w, void* dst, const void* src, size_t bytes, int pe) {
    const char* remote = symm_span(w, const_cast<char*>(static_cast<const char*>(src)), bytes, pe, 204);
    TDIST_SKIP_IF_NULL(remote);
    copy_coop(dst, remote, bytes, threadIdx.x, blockDim.x);
}
__device__ __forceinline__ void getmem_warp(const SymmWindow& w, void* dst, const void* src, size_t bytes, int pe) {
    const char* remote = symm_span(w, const_cast<char*>(static_cast<const char*>(src)), bytes, pe, 205);
    TDIST_SKIP_IF_NULL(remote);
    copy_coop(dst, remote, bytes, lane_id(), 32);
}
__device__ __forceinline__ void getmem(const SymmWindow& w, void* dst, const void* src, size_t bytes, int pe) {
    const char* remote = symm_span(w, const_cast<char*>(static_cast<const char*>(src)), bytes, pe, 206);
    TDIST_SKIP_IF_NULL(remote);
    copy_coop(dst, remote, bytes, 0, 1);
}
__device__ __forceinline__ void getmem_nbi_block(const SymmWindow& w, void* dst, const void* src, size_t bytes, int pe) {
    getmem_block(w, dst, src, bytes, pe);
}
__device__ __forceinline__ void getmem_nbi_warp(const SymmWindow& w, void* dst, const void* src, size_t bytes, int pe) {
    getmem_warp(w, dst, src, bytes, pe);
}
__device__ __forceinline__ void int_p(const SymmWindow& w, int* dst, int value, int pe) {
    int* remote = symm_at(w, dst, pe);
    TDIST_SKIP_IF_NULL(remote);
    *reinterpret_cast<volatile int*>(remote) = value;
}

// ---- signals
__device__ __forceinline__ void signal_op(const SymmWindow& w, uint64_t* sig, uint64_t value, int sig_op, int pe) {
    uint64_t* remote = symm_at(w, sig, pe);
    TDIST_SKIP_IF_NULL(remote);
    if (sig_op == kSignalAdd) red_release_sys_add_u64(remote, value);
    else st_release_sys_u64(remote, value);
}
// put, then signal `pe` once the data is ordered before the signal. `w` is the window of `dst`,
// `sw` the window of `sig` (the same window when both live in one symmetric object).
__device__ __forceinline__ void putmem_signal_block(const SymmWindow& w, void* dst, const void* src, size_t bytes,
                                                    const SymmWindow& sw, uint64_t* sig, uint64_t value, int sig_op, int pe) {
    putmem_block(w, dst, src, bytes, pe);
    __syncthreads();  // one fencing thread: the barrier orders the block's stores before its release
    if (threadIdx.x == 0) {
        fence();
        signal_op(sw, sig, value, sig_op, pe);
    }
}
__device__ __forceinline__ void putmem_signal_warp(const SymmWindow& w, void* dst, const void* src, size_t bytes,
                                                   const SymmWindow& sw, uint64_t* sig, uint64_t value, int sig_op, int pe) {
    putmem_warp(w, dst, src, bytes, pe);
    __syncwarp();
    if (lane_id() == 0) {
        fence();
        signal_op(sw, sig, value, sig_op, pe);
    }
}
__device__ __forceinline__ void putmem_signal(const SymmWindow& w, void* dst, const void* src, size_t bytes,
                                              const SymmWindow& sw, uint64_t* sig, uint64_t value, int sig_op, int pe) {
    putmem(w, dst, src, bytes, pe);
    fence();
    signal_op(sw, sig, value, sig_op, pe);
}
__device__ __forceinline__ void putmem_signal_nbi_block(const SymmWindow& w, void* dst, const void* src, size_t bytes,
                                                        const SymmWindow& sw, uint64_t* sig, uint64_t value, int sig_op, int pe) {
    putmem_signal_block(w, dst, src, bytes, sw, sig, value, sig_op, pe);
}
__device__ __forceinline__ void putmem_signal_nbi_warp(const SymmWindow& w, void* dst, const void* src, size_t bytes,
                                                       const SymmWindow& sw, uint64_t* sig, uint64_t value, int sig_op, int pe) {
    putmem_signal_warp(w, dst, src, bytes, sw, sig, value, sig_op, pe);
}
__device__ __forceinline__ void putmem_signal_nbi(const SymmWindow& w, void* dst, const void* src, size_t bytes,
                                                  const SymmWindow& sw, uint64_t* sig, uint64_t value, int sig_op, int pe) {
    putmem_signal(w, dst, src, bytes, sw, sig, value, sig_op, pe);
}

// ---- barriers. `flags` is a symmetric array of kMaxRanks 64-bit words per rank, `epoch` a
// LOCAL 64-bit counter (same value on every rank between barriers). Rank r writes epoch+1 into
// slot r of every peer, then waits for all slots of its own array. Monotonic values: no reset.
// (reference kernels/nvidia/common_ops.py:104-159 `barrier_all_intra_node_non_atomic`.)
struct BarrierState {
    uint64_t* flags;   // local symmetric address
    uint64_t* epoch;   // local (non-symmetric is fine)
};

// Call with the whole block; at least n_pes threads. Returns false if a peer never arrived.
__device__ __forceinline__ bool barrier_all_block(const SymmWindow& w, const BarrierState& b, const WaitCtx& wc) {
    __shared__ int ok_s;
    __syncthreads();
    const uint64_t target = *reinterpret_cast<volatile uint64_t*>(b.epoch) + 1;
    if (threadIdx.x == 0) ok_s = 1;
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < w.world) {
        fence_acq_rel_sys();
        uint64_t* peer_flags = symm_span(w, b.flags, static_cast<size_t>(w.world) * 8, threadIdx.x, 207);
        if (peer_flags != nullptr) st_release_sys_u64(peer_flags + w.rank, target);
        if (!signal_wait_until(b.flags + threadIdx.x, kCmpGe, target, wc, threadIdx.x, 100)) ok_s = 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) *reinterpret_cast<volatile uint64_t*>(b.epoch) = target;
    __syncthreads();
    return ok_s != 0;
}
// sync_all = barrier without the implied quiet; identical here.
__device__ __forceinline__ bool sync_all_block(const SymmWindow& w, const BarrierState& b, const WaitCtx& wc) {
    return barrier_all_block(w, b, wc);
}

// ---- collectives on symmetric buffers (block scope)
// Every PE's `dst` receives root's `src` (reference libshmem_device.broadcast*).
__device__ __forceinline__ void broadcast_block(const SymmWindow& w, void* dst, const void* src, size_t bytes, int root) {
    if (w.rank != root) return;
    for (int pe = 0; pe < w.world; ++pe) putmem_block(w, dst, src, bytes, pe);
}
// Every PE's `dst[pe_i * bytes ...]` receives PE i's `src` (reference libshmem_device.fcollect*).
__device__ __forceinline__ void fcollect_block(const SymmWindow& w, void* dst, const void* src, size_t bytes) {
    for (int i = 0; i < w.world; ++i) {
        int pe = w.rank + i;
        if (pe >= w.world) pe -= w.world;
        putmem_block(w, static_cast<char*>(dst) + static_cast<size_t>(w.rank) * bytes, src, bytes, pe);
    }
}

// ---- the same collectives at warp and thread scope, and the remaining names of the reference's device library
__device__ __forceinline__ void getmem_nbi(const SymmWindow& w, void* dst, const void* src, size_t bytes, int pe) {
    getmem(w, dst, src, bytes, pe);
}
__device__ __forceinline__ void broadcast_warp(const SymmWindow& w, void* dst, const void* src, size_t bytes, int root) {
    if (w.rank != root) return;
    for (int pe = 0; pe < w.world; ++pe) putmem_warp(w, dst, src, bytes, pe);
}
__device__ __forceinline__ void broadcast(const SymmWindow& w, void* dst, const void* src, size_t bytes, int root) {
    if (w.rank != root) return;
    for (int pe = 0; pe < w.world; ++pe) putmem(w, dst, src, bytes, pe);
}
__device__ __forceinline__ void broadcastmem_block(const SymmWindow& w, void* dst, const void* src, size_t bytes, int root) {
    broadcast_block(w, dst, src, bytes, root);
}
__device__ __forceinline__ void fcollect_warp(const SymmWindow& w, void* dst, const void* src, size_t bytes) {
    for (int i = 0; i < w.world; ++i) {
        int pe = w.rank + i;
        if (pe >= w.world) pe -= w.world;
        putmem_warp(w, static_cast<char*>(dst) + static_cast<size_t>(w.rank) * bytes, src, bytes, pe);
    }
}
__device__ __forceinline__ void fcollect(const SymmWindow& w, void* dst, const void* src, size_t bytes) {
    for (int i = 0; i < w.world; ++i) {
        int pe = w.rank + i;
        if (pe >= w.world) pe -= w.world;
        putmem(w, static_cast<char*>(dst) + static_cast<size_t>(w.rank) * bytes, src, bytes, pe);
    }
}
// Barrier called by ONE warp (at least n_pes lanes take part) or ONE thread: same flags and epoch as the block form.
__device__ __forceinline__ bool barrier_all_warp(const SymmWindow& w, const BarrierState& b, const WaitCtx& wc) {
    __syncwarp();
    const uint64_t target = *reinterpret_cast<volatile uint64_t*>(b.epoch) + 1;
    bool ok = true;
    const int lane = static_cast<int>(lane_id());
    if (lane < w.world) {
        fence_acq_rel_sys();
        uint64_t* peer_flags = symm_span(w, b.flags, static_cast<size_t>(w.world) * 8, lane, 208);
        if (peer_flags != nullptr) st_release_sys_u64(peer_flags + w.rank, target);
        ok = signal_wait_until(b.flags + lane, kCmpGe, target, wc, lane, 101);
    }
    ok = __all_sync(0xffffffffu, ok);
    if (lane == 0) *reinterpret_cast<volatile uint64_t*>(b.epoch) = target;
    __syncwarp();
    return ok;
}
__device__ __forceinline__ bool barrier_all(const SymmWindow& w, const BarrierState& b, const WaitCtx& wc) {
    const uint64_t target = *reinterpret_cast<volatile uint64_t*>(b.epoch) + 1;
    bool ok = true;
    fence_acq_rel_sys();
    for (int pe = 0; pe < w.world; ++pe) {
        uint64_t* peer_flags = symm_span(w, b.flags, static_cast<size_t>(w.world) * 8, pe, 209);
        if (peer_flags != nullptr) st_release_sys_u64(peer_flags + w.rank, target);
    }
    for (int pe = 0; pe < w.world; ++pe) ok = signal_wait_until(b.flags + pe, kCmpGe, target, wc, pe, 102) && ok;
    *reinterpret_cast<volatile uint64_t*>(b.epoch) = target;
    return ok;
}
__device__ __forceinline__ bool sync_all_warp(const SymmWindow& w, const BarrierState& b, const WaitCtx& wc) { return barrier_all_warp(w, b, wc); }
__device__ __forceinline__ bool sync_all(const SymmWindow& w, const BarrierState& b, const WaitCtx& wc) { return barrier_all(w, b, wc); }
// Address of `local` inside the multicast alias of its buffer (`mc_base` = SymmTensor.mc of the same object): what
// multimem.st / multimem.ld_reduce take (reference libshmem_device.remote_mc_ptr).
template <typename T>
__device__ __forceinline__ T* remote_mc_ptr(const SymmWindow& w, char* mc_base, T* local) {
    return reinterpret_cast<T*>(mc_base + (reinterpret_cast<char*>(local) - w.base[w.rank]));
}

}  // namespace tdist
