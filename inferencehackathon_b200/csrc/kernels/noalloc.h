// Entry point for callers that must not allocate device memory. It has no counterpart in the reference code.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need attention: code running between
// cudaStreamBeginCapture and cudaStreamEndCapture of someone else's graph, a plug-in living inside a process
// whose memory pool owns every byte of the device, a real-time loop that may not take the allocator's lock.
// For them the split-KV flash-decode kernel is offered once more with its scratch (the per-split partial
// results and the arrival counters) in a fixed array that is part of the library image itself.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest problem the built-in scratch holds: nq * nsplit <= IHB_FD_STATIC_MAX_PARTIALS (and nq <= 64).
// The array is about 1 MiB; every GPU that loads the library keeps it until the process exits.
// The kernel's own limits apply as well: at most IHB_FD_STATIC_MAX_SPLITS splits, nkv divides nq, and the number
// of query heads per KV head is 1, 2, 4 or a multiple of 8.
#define IHB_FD_STATIC_MAX_PARTIALS 2048
#define IHB_FD_STATIC_MAX_HEADS 64
#define IHB_FD_STATIC_MAX_SPLITS 256

// Same computation and argument meaning as ihb_flash_decode (api.h), minus the scratch, counters and quantised
// output arguments: q [nq, 128] fp32, k_cache / v_cache [nkv, max_seq, 128] bf16, positions 0..*pos, out [nq, 128]
// fp32. Calls no cudaMalloc / cudaFree and no allocating library routine.
//
// * The first call on a device looks up the device address of the built-in array (the device must be current);
//   make that first call outside any stream capture.
// * Every call uses the same array. It still holds the previous call's partials; the arrival counters are
//   cleared on the stream at the start of each call. Two calls that overlap on the GPU (different streams, or
//   two host threads) race on it: serialise them.
// * Returns a cudaError_t value; cudaErrorInvalidValue when the problem exceeds any of the limits above (nothing has
//   been enqueued then). After every failure ihb_flash_decode_static_error() says why.
int ihb_flash_decode_static(const float* q, const void* k_cache, const void* v_cache, int nq, int nkv, int max_seq,
                            const int* pos, int nsplit, float* out, cudaStream_t stream);

// Text of the last error reported by ihb_flash_decode_static on this host thread ("" if none).
const char* ihb_flash_decode_static_error(void);

// Bytes of the built-in scratch array.
size_t ihb_flash_decode_static_bytes(void);

#ifdef __cplusplus
}
#endif
