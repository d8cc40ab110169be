// An attention entry point that allocates nothing.  It has no counterpart in the reference.
//
// Who needs it: code that may not (or cannot) ask the CUDA allocator for memory at the
// moment it wants attention computed -- a host thread inside a real-time loop where a
// cudaMalloc could stall behind another context's work, a plug-in loaded into a process
// whose memory budget is fixed at start-up, or a caller that has no tensor library at
// hand to lend it a workspace.  The regular split-key attention needs scratch for the
// partial results of the key splits and expects the caller to bring it; this variant keeps
// that scratch inside the library, in a fixed array in device memory that exists from the
// moment the library is loaded on a GPU until the process exits.
//
// The price is a limit.  The array holds PMM_NOALLOC_SCRATCH_FLOATS floats (4 MiB) on every
// GPU that loads the library, and a call needs
//     tokens * query_heads * n_splits * (head_dim + 2)
// of them; a larger call is refused with PMM_ERR_NOALLOC_TOO_LARGE and nothing is launched.
// The same holds for every other refusal (a head shape the kernel does not take, more than
// PMM_NOALLOC_MAX_SPLITS key splits, a scale that is not positive, a null pointer): all checks
// run before the first launch.  pmm_attention_noalloc_last_error() returns a sentence describing
// the last refusal or failed launch on the calling thread.
//
// All calls share the one array, and it keeps whatever the last call left in it.  Nothing in
// it has to start at zero: every (row, split) cell that the merge reads is written by the same
// call first, empty splits included.  Two calls whose kernels overlap on the GPU (different
// streams, no dependency between them) would overwrite each other's partial results; order
// them on one stream or with events.
//
// The first call on each device looks up the array's device address (a one-time set-up that
// is not a stream operation).  Make that first call outside of any stream capture.  Host threads
// may call concurrently; the look-up is done under a lock.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PMM_NOALLOC_SCRATCH_FLOATS (1 << 20)
#define PMM_NOALLOC_MAX_SPLITS 12288  /* the merge kernel keeps one weight per split in 48 KB of shared memory */
#define PMM_ERR_NOALLOC_TOO_LARGE 1002
#define PMM_ERR_NOALLOC_SETUP 1003

// Split-key paged attention, bfloat16, same arguments and result as
// pmm_flash_paged_attention followed by pmm_flash_combine, minus the scratch pointers.
// Returns 0 when the kernels were launched on `stream`.
int pmm_attention_noalloc(const void* q, const void* pool, const int* block_table, int max_blocks,
                          const int* positions, const int* cu, void* out, float scale, int window,
                          int split_len, int n_splits, int page_size, int n_seq, int n_tokens,
                          int n_tiles, int rows16, int Hq, int Hkv, int Dh, cudaStream_t stream);

const char* pmm_attention_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
