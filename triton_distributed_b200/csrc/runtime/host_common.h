// Host-side helpers shared by the launchers: error reporting, driver entry points fetched at
// run time (the library does not link libcuda), and a cache of encoded TMA descriptors.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace tdist_host {

void set_error(const std::string& msg);
int fail(int code, const std::string& msg);

#define TDIST_CUDA_OK(expr)                                                              \
    do {                                                                                 \
        cudaError_t _e = (expr);                                                         \
        if (_e != cudaSuccess)                                                           \
            return ::tdist_host::fail(static_cast<int>(_e),                              \
                                      std::string(#expr) + ": " + cudaGetErrorString(_e)); \
    } while (0)

// Returns nullptr (and records an error) if the driver does not export `name`.
void* driver_fn(const char* name);

enum class Swizzle { None, B128 };

// Encodes (or fetches from the cache) a tiled tensor map of rank 2 or 3. dims/box are in
// elements, innermost first; strides_bytes[i] is the byte stride of dimension i+1.
// Returns 0 or a TDIST_E* code.
int encode_tmap(CUtensorMap* out, CUtensorMapDataType dtype, int elem_bytes, int rank_, const void* base,
                const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box, Swizzle sw);

int sm_count();

}  // namespace tdist_host
