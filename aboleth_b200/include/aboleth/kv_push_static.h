// KV page push that allocates nothing.
//
// This entry point has no counterpart in the reference project; it exists for callers
// of this library that are not able to allocate device memory at the moment they push:
//
//   * a serving engine that has already handed every free byte of the device to its
//     KV-cache pool, so that one more allocation - even of a few KB - can fail;
//   * a step loop in which an allocation or a free may stall the whole device behind
//     work that is still running on other streams;
//   * a plain C or C++ client that links this library without a tensor library and
//     therefore has no caching allocator to borrow scratch memory from.
//
// `ab_kv_push` needs one zeroed 32-bit arrival counter per batch from its caller.
// `ab_kv_push_static` keeps those counters in a fixed array inside the library image
// instead (AB_KV_PUSH_STATIC_MAX_BATCHES counters, 16 KB per device) and is otherwise
// the same operation: every worker CTA of a batch copies its slice, and the worker
// that arrives last publishes `epoch` in the batch's readiness cell on the consumer.
//
// What the call does, in stream order on `stream`:
//   1. on the first call for the current device only: looks up the device address of
//      the counter array (cudaGetSymbolAddress) and remembers it.  That lookup may
//      load the library's device code, so make one call on each device before any
//      stream capture begins;
//   2. clears the first `count` counters with an asynchronous memset (the counters
//      must be zero when the kernel starts, whatever an earlier call left behind);
//   3. launches the push kernel on a (count, workers) grid of `threads` threads.
// It never calls cudaMalloc, cudaFree or any routine that allocates on its behalf.
//
// Limits and rules:
//   * count must be in 1 .. AB_KV_PUSH_STATIC_MAX_BATCHES; a larger count is refused
//     with AB_KV_PUSH_STATIC_TOO_MANY and nothing is enqueued.  Split the transfer
//     into several calls on ONE stream instead.
//   * The counters are shared by every call on the same device.  Two calls whose
//     execution may overlap (different streams, or different host threads without
//     stream ordering between them) race on them and can publish readiness early or
//     never.  Order such calls on one stream or with events.
//   * `batches` and `status` are the caller's device memory, as for `ab_kv_push`:
//     `count` records of {src, dst, bytes, ready} (four 64-bit words each; src and dst
//     16-byte aligned) and two 64-bit status words.  A run whose src or dst is not
//     16-byte aligned is reported as malformed in the status words AND still copied
//     (through the 8-byte or the byte path), so the data is right either way.
//   * Every batch of one call must name a readiness cell OF ITS OWN.  There is one
//     counter per batch: a cell that two batches share is published as soon as the
//     first of them has finished, while the other may still be copying.  A caller that
//     wants one cell for several runs (a readiness group of several layers) either
//     makes them one contiguous batch, gives each its own cell and waits for all of
//     them, or uses `ab_kv_push` with its group arguments.
//   * The remembered address of the counter array belongs to the device context it
//     was looked up in.  After cudaDeviceReset in the same process it is stale; a
//     process that resets a device must not call this entry point for that device again.
//
// Returns 0 when the work was enqueued, a negative AB_KV_PUSH_STATIC_* code for a
// rejected argument, or the positive cudaError_t of a failed runtime call.
#pragma once

#include <stdint.h>

#include <cuda_runtime_api.h>

#define AB_KV_PUSH_STATIC_MAX_BATCHES 4096
#define AB_KV_PUSH_STATIC_BAD_ARGUMENT (-1)
#define AB_KV_PUSH_STATIC_TOO_MANY (-2)

#ifdef __cplusplus
extern "C" {
#endif

int ab_kv_push_static(const void *batches, int count, uint64_t epoch, int workers, int threads,
                      unsigned long long *status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
