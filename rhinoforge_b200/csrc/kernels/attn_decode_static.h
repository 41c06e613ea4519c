// Paged decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference: it exists for hosts that
// hand this library nothing but input and output pointers and forbid device
// allocation once they are running -- a robot control loop that cannot afford
// the device-wide synchronisation hidden in cudaMalloc, or an embedding runtime
// that has already given every byte of device memory to its own pool and has no
// spare block to lend for split-KV partial results.
#pragma once
#include "../rf_api.h"

#ifdef __cplusplus
extern "C" {
#endif

// Largest split-KV scratch the built-in buffer can serve, in bytes.  The buffer
// is part of the library image: every GPU whose context loads the library holds
// this much memory until the process exits, whether or not the entry point is used.
#define RF_ATTN_DECODE_STATIC_SCRATCH_BYTES (8u << 20)

// Same contract and same kernels as rf_attn_decode(), except that the split-KV
// scratch is the library's own fixed buffer: the `ws` / `ws_bytes` fields of `a`
// are ignored, and nothing is allocated or freed on the device or through any
// allocating library routine.
//
//  * A request whose split-KV partials would exceed
//    RF_ATTN_DECODE_STATIC_SCRATCH_BYTES is refused with RF_ERR_NO_MEMORY and a
//    message naming both sizes; use rf_attn_decode() with caller memory instead.
//  * The first call on each device looks up the buffer's device address (once
//    per device, with that device current).  Make that first call outside any
//    stream capture.
//  * Every call on a device shares the one buffer, and the buffer keeps whatever
//    the previous call left in it.  Nothing has to be cleared between calls:
//    each slot the merge pass reads is rewritten by the same call first, with a
//    partial result or -- when a bounded wait inside the kernel ran out -- with an
//    "empty" marker, so a timed-out call never blends an earlier call's partials
//    into `out`.  After a reported timeout (non-zero status word) `out` is still
//    not a valid result: check the status before using it.
//  * Two calls that overlap on the GPU (different streams, or the same stream
//    from concurrent graph launches) race on the buffer.  Serialise them.
//  * The entry point may be used on several devices of one process: the buffer's
//    address, the kernels' shared-memory limits and the SM count that sizes the
//    split are all kept per device.
int rf_attn_decode_static(const RfAttn* a, rf_stream_t stream);

#ifdef __cplusplus
}
#endif
