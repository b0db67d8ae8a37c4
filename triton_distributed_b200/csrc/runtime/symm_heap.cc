// Symmetric-heap backing store: physical allocations that every rank of a node maps into its
// own address space, plus optional NVLS multicast objects over them.
//
// This is the native half of what the reference gets from NVSHMEM through its `_pynvshmem`
// binding (shmem/nvshmem_bind/pynvshmem/src/pynvshmem.cc:107-215: nvshmem_malloc / nvshmem_ptr /
// nvshmemx_mc_ptr). Here a segment is a cuMemCreate allocation exported as a POSIX file
// descriptor; the Python side passes descriptors between the ranks' processes, and every rank
// maps all `world` segments back to back into one reserved virtual range, so the address of
// rank r's copy of a symmetric object is `local + (r - me) * segment_bytes`. A cudaIpc path
// (cudaMalloc + cudaIpcGetMemHandle) is kept for systems where descriptor export is refused.
//
// All driver entry points are resolved at run time; the library does not link libcuda.
#include <cuda.h>
#include <cuda_runtime.h>
#include <string.h>
#include <unistd.h>

#include <string>

#include "../include/tdist.h"
#include "host_common.h"

using tdist_host::driver_fn;
using tdist_host::fail;

namespace {

struct Driver {
    CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long);
    CUresult (*MemRelease)(CUmemGenericAllocationHandle);
    CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags);
    CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
    CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType);
    CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*MemAddressFree)(CUdeviceptr, size_t);
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*MemUnmap)(CUdeviceptr, size_t);
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t);
    CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*);
    CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice);
    CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long);
    CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags);
    CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t);
    CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice);
    CUresult (*StreamWriteValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
    CUresult (*StreamWaitValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
    CUresult (*StreamWriteValue64)(CUstream, CUdeviceptr, cuuint64_t, unsigned int);
    CUresult (*StreamWaitValue64)(CUstream, CUdeviceptr, cuuint64_t, unsigned int);
    bool ok = false;
};

Driver* drv() {
    static Driver d;
    static bool tried = false;
    if (!tried) {
        tried = true;
        cudaFree(nullptr);  // make sure the primary context exists
#define LOAD(field, name)                                        \
    d.field = reinterpret_cast<decltype(d.field)>(driver_fn(name)); \
    if (d.field == nullptr) return &d;
        LOAD(MemCreate, "cuMemCreate")
        LOAD(MemRelease, "cuMemRelease")
        LOAD(MemGetAllocationGranularity, "cuMemGetAllocationGranularity")
        LOAD(MemExportToShareableHandle, "cuMemExportToShareableHandle")
        LOAD(MemImportFromShareableHandle, "cuMemImportFromShareableHandle")
        LOAD(MemAddressReserve, "cuMemAddressReserve")
        LOAD(MemAddressFree, "cuMemAddressFree")
        LOAD(MemMap, "cuMemMap")
        LOAD(MemUnmap, "cuMemUnmap")
        LOAD(MemSetAccess, "cuMemSetAccess")
        LOAD(MulticastCreate, "cuMulticastCreate")
        LOAD(MulticastAddDevice, "cuMulticastAddDevice")
        LOAD(MulticastBindMem, "cuMulticastBindMem")
        LOAD(MulticastGetGranularity, "cuMulticastGetGranularity")
        LOAD(MulticastUnbind, "cuMulticastUnbind")
        LOAD(DeviceGetAttribute, "cuDeviceGetAttribute")
        LOAD(StreamWriteValue32, "cuStreamWriteValue32")
        LOAD(StreamWaitValue32, "cuStreamWaitValue32")
        LOAD(StreamWriteValue64, "cuStreamWriteValue64")
        LOAD(StreamWaitValue64, "cuStreamWaitValue64")
#undef LOAD
        d.ok = true;
    }
    return &d;
}

int cu_fail(const char* what, CUresult r) {
    return fail(TDIST_EDRIVER, std::string(what) + " failed with CUresult " + std::to_string(static_cast<int>(r)));
}

#define TDIST_CU_OK(what, expr)                      \
    do {                                             \
        CUresult _r = (expr);                        \
        if (_r != CUDA_SUCCESS) return cu_fail(what, _r); \
    } while (0)

CUmemAllocationProp local_prop(int dev) {
    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = dev;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

}  // namespace

extern "C" {

// Capabilities of device `dev`: bit 0 = VMM + POSIX fd export, bit 1 = NVLS multicast.
int tdist_symm_caps(int dev, int* caps) {
    *caps = 0;
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    int v = 0;
    if (d->DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev) == CUDA_SUCCESS && v) {
        int fd_ok = 0;
        if (d->DeviceGetAttribute(&fd_ok, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev) == CUDA_SUCCESS && fd_ok)
            *caps |= 1;
    }
    v = 0;
    if (d->DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS && v) *caps |= 2;
    return 0;
}

// Rounds `bytes` up to what a segment on `dev` (and, if asked, a multicast object over `world`
// devices) can be created with.
int tdist_symm_round_size(int dev, size_t bytes, int world_for_multicast, size_t* rounded) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    CUmemAllocationProp prop = local_prop(dev);
    size_t gran = 0;
    TDIST_CU_OK("cuMemGetAllocationGranularity", d->MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    if (world_for_multicast > 1) {
        CUmulticastObjectProp mp;
        memset(&mp, 0, sizeof(mp));
        mp.numDevices = static_cast<unsigned>(world_for_multicast);
        mp.size = bytes;
        mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t mg = 0;
        if (d->MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
    }
    if (gran == 0) gran = 2u << 20;
    *rounded = (bytes + gran - 1) / gran * gran;
    return 0;
}

// Creates this rank's physical segment and exports it. `bytes` must come from
// tdist_symm_round_size.
int tdist_symm_create(int dev, size_t bytes, uint64_t* handle, int* fd) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    CUmemAllocationProp prop = local_prop(dev);
    CUmemGenericAllocationHandle h;
    TDIST_CU_OK("cuMemCreate", d->MemCreate(&h, bytes, &prop, 0));
    int out_fd = -1;
    CUresult r = d->MemExportToShareableHandle(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) {
        d->MemRelease(h);
        return cu_fail("cuMemExportToShareableHandle", r);
    }
    *handle = static_cast<uint64_t>(h);
    *fd = out_fd;
    return 0;
}

int tdist_symm_import(int fd, uint64_t* handle) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    CUmemGenericAllocationHandle h;
    TDIST_CU_OK("cuMemImportFromShareableHandle",
                d->MemImportFromShareableHandle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
    *handle = static_cast<uint64_t>(h);
    return 0;
}

int tdist_symm_release(uint64_t handle) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    TDIST_CU_OK("cuMemRelease", d->MemRelease(static_cast<CUmemGenericAllocationHandle>(handle)));
    return 0;
}

int tdist_symm_reserve(size_t bytes, uint64_t* va) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    CUdeviceptr p = 0;
    TDIST_CU_OK("cuMemAddressReserve", d->MemAddressReserve(&p, bytes, 0, 0, 0));
    *va = static_cast<uint64_t>(p);
    return 0;
}

// Maps `handle` (bytes long) at `va` and grants device `dev` read/write access.
int tdist_symm_map(uint64_t va, size_t bytes, uint64_t handle, int dev) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    TDIST_CU_OK("cuMemMap", d->MemMap(static_cast<CUdeviceptr>(va), bytes, 0, static_cast<CUmemGenericAllocationHandle>(handle), 0));
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = dev;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    CUresult r = d->MemSetAccess(static_cast<CUdeviceptr>(va), bytes, &acc, 1);
    if (r != CUDA_SUCCESS) {
        d->MemUnmap(static_cast<CUdeviceptr>(va), bytes);
        return cu_fail("cuMemSetAccess", r);
    }
    return 0;
}

int tdist_symm_unmap(uint64_t va, size_t bytes) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    TDIST_CU_OK("cuMemUnmap", d->MemUnmap(static_cast<CUdeviceptr>(va), bytes));
    return 0;
}

int tdist_symm_address_free(uint64_t va, size_t bytes) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    TDIST_CU_OK("cuMemAddressFree", d->MemAddressFree(static_cast<CUdeviceptr>(va), bytes));
    return 0;
}

// ---- NVLS multicast objects (off unless the Python side asks for them) ----
int tdist_mc_create(int world, size_t bytes, uint64_t* handle, int* fd) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = static_cast<unsigned>(world);
    mp.size = bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUmemGenericAllocationHandle h;
    TDIST_CU_OK("cuMulticastCreate", d->MulticastCreate(&h, &mp));
    int out_fd = -1;
    CUresult r = d->MemExportToShareableHandle(&out_fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) {
        d->MemRelease(h);
        return cu_fail("cuMemExportToShareableHandle(multicast)", r);
    }
    *handle = static_cast<uint64_t>(h);
    *fd = out_fd;
    return 0;
}
int tdist_mc_add_device(uint64_t mc_handle, int dev) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    TDIST_CU_OK("cuMulticastAddDevice", d->MulticastAddDevice(static_cast<CUmemGenericAllocationHandle>(mc_handle), dev));
    return 0;
}
int tdist_mc_bind(uint64_t mc_handle, uint64_t mem_handle, size_t bytes) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    TDIST_CU_OK("cuMulticastBindMem",
                d->MulticastBindMem(static_cast<CUmemGenericAllocationHandle>(mc_handle), 0,
                                    static_cast<CUmemGenericAllocationHandle>(mem_handle), 0, bytes, 0));
    return 0;
}
int tdist_mc_unbind(uint64_t mc_handle, int dev, size_t bytes) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    TDIST_CU_OK("cuMulticastUnbind", d->MulticastUnbind(static_cast<CUmemGenericAllocationHandle>(mc_handle), dev, 0, bytes));
    return 0;
}

// ---- cudaIpc fallback ----
int tdist_ipc_alloc(size_t bytes, void** ptr, char handle_out[64]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "ipc handle size");
    TDIST_CUDA_OK(cudaMalloc(ptr, bytes));
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, *ptr);
    if (e != cudaSuccess) {
        cudaFree(*ptr);
        return fail(static_cast<int>(e), std::string("cudaIpcGetMemHandle: ") + cudaGetErrorString(e));
    }
    memcpy(handle_out, &h, 64);
    return 0;
}
int tdist_ipc_open(const char handle[64], void** ptr) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    TDIST_CUDA_OK(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return 0;
}
int tdist_ipc_close(void* ptr) {
    TDIST_CUDA_OK(cudaIpcCloseMemHandle(ptr));
    return 0;
}
int tdist_ipc_free(void* ptr) {
    TDIST_CUDA_OK(cudaFree(ptr));
    return 0;
}

// ---- stream-ordered flag operations (reference kernels/nvidia/common_ops.py:178-211) ----
int tdist_stream_write_value(void* stream, uint64_t addr, uint64_t value, int is_64) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    if (is_64) TDIST_CU_OK("cuStreamWriteValue64", d->StreamWriteValue64(static_cast<CUstream>(stream), addr, value, 0));
    else TDIST_CU_OK("cuStreamWriteValue32", d->StreamWriteValue32(static_cast<CUstream>(stream), addr, static_cast<cuuint32_t>(value), 0));
    return 0;
}
int tdist_stream_wait_value(void* stream, uint64_t addr, uint64_t value, int is_64, int geq) {
    Driver* d = drv();
    if (!d->ok) return TDIST_EDRIVER;
    const unsigned flag = geq ? CU_STREAM_WAIT_VALUE_GEQ : CU_STREAM_WAIT_VALUE_EQ;
    if (is_64) TDIST_CU_OK("cuStreamWaitValue64", d->StreamWaitValue64(static_cast<CUstream>(stream), addr, value, flag));
    else TDIST_CU_OK("cuStreamWaitValue32", d->StreamWaitValue32(static_cast<CUstream>(stream), addr, static_cast<cuuint32_t>(value), flag));
    return 0;
}

}  // extern "C"
