/* Allocation-free flash decode.
 *
 * This entry point has no counterpart in the reference library; it exists for callers of this
 * library that are not in a position to allocate device memory around a decode step:
 *   - a serving loop whose latency budget cannot absorb cudaMalloc / cudaFree (both may
 *     synchronise the whole device, stalling every other stream of the process);
 *   - a host application that gave all device memory to its own pool at start-up, so that a
 *     later allocation by a library simply fails;
 *   - a foreign-function caller (plain C, ctypes, another runtime's plugin ABI) that holds raw
 *     device pointers for q / caches / output but has no allocator to size and own a workspace.
 *
 * tdist_flash_decode (tdist.h) needs two scratch buffers from its caller: the split-merge workspace
 * `partial` and the per-(sequence, kv head) arrival `counters`. Here both live in one array that is
 * part of the library image: a file-scope `static __device__` array of TDIST_DECODE_STATIC_SCRATCH_BYTES
 * (8 MiB), which every GPU that loads libtdist.so holds from load until the process exits.
 *
 * Contract
 *   - `args->partial` and `args->counters` are ignored; everything else means what it means for
 *     tdist_flash_decode, modes 0 and 1 only (the sequence-parallel mode needs symmetric memory
 *     that only the caller can provide).
 *   - The problem must fit:  B*Hkv*4  rounded up to 256, plus  B*Hq*splits*(head_dim+2)*4  bytes,
 *     at most TDIST_DECODE_STATIC_SCRATCH_BYTES. Anything larger is rejected with TDIST_ELIMIT and a
 *     message in tdist_last_error(); nothing is launched.
 *   - No cudaMalloc, cudaFree or other allocating call is made, on any call.
 *   - The first call on each device resolves the array's device address (cudaGetSymbolAddress, with
 *     that device current) and raises the kernel's shared-memory limit; make that first call
 *     outside any stream capture. Later calls only enqueue a small memset and the kernel.
 *   - The array is shared by every call on the device and keeps the last call's contents. The
 *     counters region is cleared on the stream before each launch; the partial region is fully
 *     rewritten by each launch before it is read. Two calls that overlap on the GPU (different
 *     streams, no ordering between them) race on the array: order them.
 */
#pragma once
#include "tdist.h"

#ifdef __cplusplus
extern "C" {
#endif

#define TDIST_DECODE_STATIC_SCRATCH_BYTES (8u << 20)

int tdist_flash_decode_static(const TdistDecodeArgs* args);

#ifdef __cplusplus
}
#endif
