#include "host_common.h"

#include <cstring>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "../include/tdist.h"

namespace tdist_host {

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }
int fail(int code, const std::string& msg) {
    g_last_error = msg;
    return code;
}

void* driver_fn(const char* name) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr) {
        cudaGetLastError();
        set_error(std::string("CUDA driver entry point not available: ") + name);
        return nullptr;
    }
    return fn;
}

namespace {
struct TmapKey {
    uint64_t words[16];
    bool operator==(const TmapKey& o) const { return std::memcmp(words, o.words, sizeof(words)) == 0; }
};
struct TmapKeyHash {
    size_t operator()(const TmapKey& k) const {
        uint64_t h = 1469598103934665603ull;
        for (uint64_t w : k.words) {
            h ^= w;
            h *= 1099511628211ull;
        }
        return static_cast<size_t>(h);
    }
};
std::mutex g_tmap_mu;
std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> g_tmap_cache;
}  // namespace

int encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int elem_bytes, int rank_, const void* base,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box, Swizzle sw) {
    if (rank_ < 2 || rank_ > 3) return fail(TDIST_EINVAL, "encode_tmap: rank must be 2 or 3");
    if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
        return fail(TDIST_EINVAL, "tensor map base address is not 16-byte aligned");
    for (int i = 0; i + 1 < rank_; ++i)
        if (strides_bytes[i] % 16 != 0)
            return fail(TDIST_EINVAL, "tensor map stride is not a multiple of 16 bytes");
    if ((static_cast<uint64_t>(box[0]) * elem_bytes) % 16 != 0)
        return fail(TDIST_EINVAL, "tensor map box inner extent is not a multiple of 16 bytes");

    TmapKey key;
    std::memset(&key, 0, sizeof(key));
    key.words[0] = reinterpret_cast<uint64_t>(base);
    key.words[1] = (static_cast<uint64_t>(dtype) << 32) | (static_cast<uint64_t>(rank_) << 8) |
                   static_cast<uint64_t>(sw == Swizzle::B128);
    for (int i = 0; i < rank_; ++i) {
        key.words[2 + i] = dims[i];
        key.words[8 + i] = box[i];
    }
    for (int i = 0; i + 1 < rank_; ++i) key.words[5 + i] = strides_bytes[i];
    {
        std::lock_guard<std::mutex> lk(g_tmap_mu);
        auto it = g_tmap_cache.find(key);
        if (it != g_tmap_cache.end()) {
            *out = it->second;
            return 0;
        }
    }
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
    static EncodeFn encode = reinterpret_cast<EncodeFn>(driver_fn("cuTensorMapEncodeTiled"));
    if (encode == nullptr) return TDIST_EDRIVER;
    cuuint64_t gdims[3];
    cuuint64_t gstrides[2];
    cuuint32_t gbox[3];
    cuuint32_t estr[3] = {1, 1, 1};
    for (int i = 0; i < rank_; ++i) {
        gdims[i] = dims[i];
        gbox[i] = box[i];
    }
    for (int i = 0; i + 1 < rank_; ++i) gstrides[i] = strides_bytes[i];
    CUresult r = encode(out, dtype, static_cast<cuuint32_t>(rank_), const_cast<void*>(base), gdims, gstrides,
                        gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        sw == Swizzle::B128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(TDIST_EINVAL, "cuTensorMapEncodeTiled failed with CUresult " + std::to_string(static_cast<int>(r)));
    {
        std::lock_guard<std::mutex> lk(g_tmap_mu);
        if (g_tmap_cache.size() > 4096) g_tmap_cache.clear();
        g_tmap_cache.emplace(key, *out);
    }
    return 0;
}

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace tdist_host

extern "C" const char* tdist_last_error(void) { return tdist_host::g_last_error.c_str(); }

// The status block lives in device memory: waiting kernels poll its abort word, and a poll that
// crossed PCIe to host memory would slow every spin loop down whenever the bus is busy.
extern "C" int tdist_status_create(void** device_ptr) {
    void* d = nullptr;
    TDIST_CUDA_OK(cudaMalloc(&d, sizeof(TdistStatus)));
    TDIST_CUDA_OK(cudaMemset(d, 0, sizeof(TdistStatus)));
    *device_ptr = d;
    return 0;
}

// Blocking copy of the block to the host (call after the producing stream was synchronised).
extern "C" int tdist_status_read(const void* device_ptr, TdistStatus* out) {
    TDIST_CUDA_OK(cudaMemcpy(out, device_ptr, sizeof(TdistStatus), cudaMemcpyDeviceToHost));
    return 0;
}

extern "C" int tdist_status_reset(void* device_ptr) {
    TDIST_CUDA_OK(cudaMemset(device_ptr, 0, sizeof(TdistStatus)));
    return 0;
}

extern "C" int tdist_status_destroy(void* device_ptr) {
    if (device_ptr != nullptr) TDIST_CUDA_OK(cudaFree(device_ptr));
    return 0;
}
