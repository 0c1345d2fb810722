// Attention backward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference system; it exists for users of this library.
//
// Who needs it: a host program that has already handed every byte of device memory to its own pool (a
// serving engine that sizes its KV cache to "all that is left", a trainer running under a hard memory
// partition), or a plugin that runs inside such a program and is not allowed to call cudaMalloc / cudaFree,
// because an allocation there either fails outright or fragments the owner's pool and stalls every stream on
// the implicit synchronisation of cudaFree. The regular gv_attn_bwd asks its caller for two scratch buffers
// (an fp32 dQ accumulator and the per-row delta = rowsum(dO * O)); this variant brings its own, in a fixed
// file-scope device array, so the caller passes only the inputs and the outputs.
//
// Limits (checked, never exceeded silently):
//   b * sq * hq * dh <= GV_NOALLOC_ATTN_MAX_DQ_ELEMS   (fp32 dQ accumulator, 16 MiB)
//   b * hq * sq      <= GV_NOALLOC_ATTN_MAX_ROWS       (fp32 delta, 256 KiB)
// Every GPU that loads the library carries these 16.25 MiB until the process exits.
//
// Behaviour to know about:
//   * The first call on each device looks up the device address of the scratch array (a one-time host-side
//     set-up step for that device, done with that device current). Make that first call outside any stream
//     capture.
//   * All calls share the one array and it keeps whatever the previous call left in it; the part that must
//     start at zero (the dQ accumulator) is cleared on the stream at the start of every call.
//   * Because the scratch is shared, two calls whose GPU work overlaps (different streams, or different host
//     threads) race on it. Serialise calls on one stream, or order the streams with events.
//   * No cudaMalloc, cudaFree or allocating library routine is called on any path, including the error paths.
#pragma once
#include "gv_kernels.h"

#ifdef __cplusplus
extern "C" {
#endif

#define GV_NOALLOC_ATTN_MAX_DQ_ELEMS (4ll * 1024 * 1024)
#define GV_NOALLOC_ATTN_MAX_ROWS (64ll * 1024)

// Error codes specific to this entry point (0 = launched; other positive values come from gv_attn_bwd).
#define GV_NOALLOC_ERR_TOO_LARGE (-2401)   // problem exceeds the fixed scratch size
#define GV_NOALLOC_ERR_SYMBOL (-2402)      // the scratch array's device address could not be obtained
#define GV_NOALLOC_ERR_DEVICE (-2403)      // current device could not be queried / index out of range
#define GV_NOALLOC_ERR_ARGS (-2404)        // NULL argument block or non-positive / inconsistent head counts

// Same contract as gv_attn_bwd, except that args->dq_accum and args->delta are ignored (may be NULL).
int gv_attn_bwd_noalloc(const gv_attn_args* args, gv_stream_t stream);

// Human-readable text for a return code of gv_attn_bwd_noalloc (static storage, never NULL).
const char* gv_attn_bwd_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
