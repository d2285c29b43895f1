// Allocation-free greedy argmax (one exported function).
//
// This entry point has no counterpart in the reference engine. It exists for callers that must not, or cannot,
// allocate device memory at the moment they need a greedy token: a host program that handed every byte of the
// GPU to its own pools at start-up and treats a late cudaMalloc as a failure; a plain C or C++ integrator that
// links this library without PyTorch and therefore has no caching allocator to lean on; a serving loop that wants
// its steady state to make no allocator calls at all so that memory use is provable ahead of time. The regular
// path (hb_argmax2) takes two scratch arrays from its caller; here the same two-stage reduction keeps its
// partials in a fixed array that is part of the library image itself.
//
// What the caller must know:
//   * The scratch is one file-scope device array of HB_NOALLOC_SCRATCH_BYTES bytes. Every GPU that loads the
//     library holds that much memory until the process exits. With HB_NOALLOC_CHUNKS partial results per row it
//     serves at most HB_NOALLOC_MAX_ROWS rows per call; a larger request is refused with
//     HB_NOALLOC_TOO_MANY_ROWS and nothing is launched.
//   * The first call on a device looks the array's device address up (cudaGetSymbolAddress, once per device, with
//     that device current) and remembers it. Make that first call before any stream capture begins.
//   * The function calls no cudaMalloc / cudaFree and no allocating library routine.
//   * All calls on a device share the one array and it keeps whatever the previous call left behind. The kernels
//     overwrite every partial they later read, so nothing has to be cleared between calls; but two calls whose
//     kernels overlap in time on the same device (different streams, or different host threads) race on it.
//     Serialise them.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define HB_NOALLOC_CHUNKS 32
#define HB_NOALLOC_MAX_ROWS 1024
#define HB_NOALLOC_SCRATCH_BYTES (HB_NOALLOC_MAX_ROWS * HB_NOALLOC_CHUNKS * 8)

enum {
  HB_NOALLOC_OK = 0,
  HB_NOALLOC_BAD_ARGUMENT = 1,     // null pointer, non-positive vocabulary, negative row count
  HB_NOALLOC_TOO_MANY_ROWS = 2,    // rows > HB_NOALLOC_MAX_ROWS
  HB_NOALLOC_SETUP_FAILED = 3,     // the device address of the scratch array could not be obtained
  HB_NOALLOC_LAUNCH_FAILED = 4,
};

// Greedy token of every row: out[r] = index of the largest of logits[r, 0..vocab) (lowest index on ties).
// logits: device pointer, row pitch `ld` elements, fp32 when is_f32 != 0 else bf16. out: device int64 [rows].
// stream: a cudaStream_t. errbuf (may be null) receives a one-line description when the call is refused.
int hb_argmax_noalloc(const void* logits, long long ld, int rows, int vocab, int is_f32, void* out, void* stream,
                      char* errbuf, int errbuf_len);

#ifdef __cplusplus
}
#endif
