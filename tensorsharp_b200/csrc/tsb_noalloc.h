// Allocation-free entry point of the decode-attention kernel.
//
// This entry point has no counterpart in the reference: it exists for hosts that may not
// allocate device memory at call time.
//
// Who needs it.  tsb_attn_decode() takes two caller-provided scratch buffers for the
// split-KV partial results.  Some embedders cannot supply them: a serving process that has
// already handed the whole device to its own arena and forbids any further cudaMalloc, a
// latency-critical decode loop that must never hit the allocator's implicit
// synchronisation, or a foreign-language binding that can pass only the tensors it already
// owns.  For those callers the scratch lives inside this library, in a file-scope
// `static __device__` array, and the call allocates nothing: no cudaMalloc, no cudaFree and
// no allocating library routine.
//
// Limits and rules
//   * The scratch holds TSB_ATTN_NOALLOC_MAX_FLOATS floats (16 MiB).  A call needs
//     B * Hq * splits * (Dh + 2) floats; a larger request is rejected with TSB_ERR_ARG and a
//     message from tsb_last_error() - lower `splits` or the batch.
//   * The array is part of the loaded library image: every GPU whose context loads the
//     library holds those 16 MiB until the process exits.
//   * The first call on each device looks up the array's device address
//     (cudaGetSymbolAddress, with that device current) and caches it; make that first call
//     before starting any stream capture.  The lookup is guarded per device (std::call_once),
//     so host threads may race to that first call.
//   * All calls on a device share the one array and it keeps the previous call's contents.
//     Nothing in it has to start at zero: every slot the combine pass reads is written by
//     the partial pass of the same call first.  Two calls that overlap on the GPU (different
//     streams, no ordering between them) race on the array; order them.  This entry point
//     always runs the two-kernel form (partials, then combine), whatever TSB_ATTN_FUSED_COMBINE
//     says, so the scratch array is the only state that calls share.
//   * args->part_o and args->part_ml are ignored; everything else in AttnArgs (inputs,
//     output, sizes) is passed by the caller exactly as for tsb_attn_decode().
#pragma once

#define TSB_ATTN_NOALLOC_MAX_FLOATS (4 * 1024 * 1024)

struct AttnArgs;

#ifdef __cplusplus
extern "C" {
#endif
// Same contract and result as tsb_attn_decode(args, stream), without caller scratch.
int tsb_attn_decode_noalloc(const struct AttnArgs* args, void* stream);
// Capacity of the built-in scratch, in floats (for callers that want to size `splits`).
long tsb_attn_decode_noalloc_capacity(void);
#ifdef __cplusplus
}
#endif
