// The reference's raw-PTX helper names (patches/triton/third_party/nvidia/language/cuda/language_extra.py:33-558) as
// CUDA device functions, for kernels ported from Triton code that spells them out. Thin inline wrappers over
// signal.cuh / ptx.cuh plus the few that have no counterpart there (multimem stores, vector loads).
#pragma once
#include "signal.cuh"

namespace tdist {
namespace language_extra {

enum Scope { kScopeGpu = 0, kScopeSys = 1 };
enum Semantic { kRelaxed = 0, kAcquire = 1, kRelease = 2, kAcqRel = 3 };

__device__ __forceinline__ int tid(int axis) { return axis == 0 ? threadIdx.x : (axis == 1 ? threadIdx.y : threadIdx.z); }
__device__ __forceinline__ int ntid(int axis) { return axis == 0 ? blockDim.x : (axis == 1 ? blockDim.y : blockDim.z); }
__device__ __forceinline__ int laneid() { return static_cast<int>(lane_id()); }
__device__ __forceinline__ void fence_sc(Scope scope) {  // reference `__fence(scope)` -> fence.sc
    if (scope == kScopeSys) asm volatile("fence.sc.sys;" ::: "memory");
    else asm volatile("fence.sc.gpu;" ::: "memory");
}

// ld / st with scope and semantic (reference `ld`, `st`, `ld_acquire`, `ld_b32`, `st_b32`)
__device__ __forceinline__ uint32_t ld(const uint32_t* p, Scope scope, Semantic sem) {
    if (sem == kAcquire) return scope == kScopeSys ? ld_acquire_sys_u32(p) : ld_acquire_gpu_u32(p);
    return ld_relaxed_sys_u32(p);
}
__device__ __forceinline__ uint64_t ld(const uint64_t* p, Scope scope, Semantic sem) {
    if (sem == kAcquire) return scope == kScopeSys ? ld_acquire_sys_u64(p) : ld_acquire_gpu_u64(p);
    return ld_relaxed_sys_u64(p);
}
__device__ __forceinline__ void st(uint32_t* p, uint32_t v, Scope scope, Semantic sem) {
    if (sem == kRelease) {
        if (scope == kScopeSys) st_release_sys_u32(p, v);
        else st_release_gpu_u32(p, v);
    } else {
        st_relaxed_sys_u32(p, v);
    }
}
__device__ __forceinline__ void st(uint64_t* p, uint64_t v, Scope scope, Semantic sem) {
    if (sem == kRelease) {
        if (scope == kScopeSys) st_release_sys_u64(p, v);
        else st_release_gpu_u64(p, v);
    } else {
        st_relaxed_sys_u64(p, v);
    }
}
__device__ __forceinline__ uint32_t ld_acquire(const uint32_t* p, Scope scope) { return ld(p, scope, kAcquire); }

// atomics
__device__ __forceinline__ uint32_t atomic_add(uint32_t* p, uint32_t v, Scope scope) {
    return scope == kScopeSys ? atom_add_acq_rel_sys_u32(p, v) : atom_add_acq_rel_gpu_u32(p, v);
}
__device__ __forceinline__ uint32_t atomic_cas(uint32_t* p, uint32_t cmp, uint32_t val) { return atom_cas_acq_rel_sys_u32(p, cmp, val); }
// lane 0 adds for the warp, everybody gets the old value (reference `atomic_add_per_warp`)
__device__ __forceinline__ uint32_t atomic_add_per_warp(uint32_t* p, uint32_t v, Scope scope) {
    uint32_t old = 0;
    if (laneid() == 0) old = atomic_add(p, v, scope);
    return __shfl_sync(0xffffffffu, old, 0);
}
__device__ __forceinline__ void red_release(uint32_t* p, uint32_t v, Scope scope) {
    if (scope == kScopeSys) red_release_sys_add_u32(p, v);
    else red_release_gpu_add_u32(p, v);
}
// after a CTA barrier, one thread publishes the CTA's arrival (reference `arrive_inc`)
__device__ __forceinline__ void arrive_inc(uint32_t* p, int thread, uint32_t v, Scope scope) {
    __syncthreads();
    if (static_cast<int>(threadIdx.x) == thread) red_release(p, v, scope);
}
// bounded spin until *p == value (reference `wait_eq` on the device)
__device__ __forceinline__ bool wait_eq(const uint64_t* p, uint64_t value, const WaitCtx& w) {
    return signal_wait_until(p, kCmpEq, value, w, -1, 50);
}

// warp intrinsics over 32-bit values (reference `__shfl_sync_i32`, `__shfl_up_sync_i32`, `__shfl_down_sync_i32`,
// `__ballot_sync`; spelled without the leading underscores, which C++ reserves)
__device__ __forceinline__ int shfl_sync_i32(unsigned mask, int value, int src_lane) { return __shfl_sync(mask, value, src_lane); }
__device__ __forceinline__ int shfl_up_sync_i32(unsigned mask, int value, unsigned delta) { return __shfl_up_sync(mask, value, delta); }
__device__ __forceinline__ int shfl_down_sync_i32(unsigned mask, int value, unsigned delta) { return __shfl_down_sync(mask, value, delta); }
__device__ __forceinline__ unsigned ballot_sync(unsigned mask, bool predicate) { return __ballot_sync(mask, predicate); }

// vector loads / stores used by the LL protocol
__device__ __forceinline__ uint4 load_v4_u32(const void* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ ulonglong2 load_v2_b64(const void* p) {
    ulonglong2 v;
    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(v.x), "=l"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void store_v2_u32(void* p, uint32_t a, uint32_t b) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

// stores through the NVSwitch multicast engine: `mc` is an address inside the multicast alias of a symmetric
// buffer (SymmTensor.mc), the value lands in every rank's copy
__device__ __forceinline__ void multimem_st_b32(void* mc, uint32_t v) {
    asm volatile("multimem.st.weak.global.b32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_st_b64(void* mc, uint64_t v) {
    asm volatile("multimem.st.weak.global.b64 [%0], %1;" ::"l"(mc), "l"(v) : "memory");
}
__device__ __forceinline__ void multimem_st_v2_b32(void* mc, uint32_t a, uint32_t b) {
    asm volatile("multimem.st.weak.global.v2.f32 [%0], {%1, %2};" ::"l"(mc), "r"(a), "r"(b) : "memory");
}

}  // namespace language_extra
}  // namespace tdist
