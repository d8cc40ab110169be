// Allocation-free variant of the split-key attention: see attention_noalloc.h for who it is
// for, its limit and its rules.  No counterpart in the reference.
#include "attention_noalloc.h"
#include "common.cuh"
#include <stdio.h>
#include <mutex>

// The regular launchers (attention_mma.cu); this file only supplies their scratch.
extern "C" int pmm_flash_supported(int Hq, int Hkv, int Dh);
extern "C" int pmm_flash_paged_attention(const void* q, const void* pool, const int* block_table,
                                         int max_blocks, const int* positions, const int* cu, void* out,
                                         float* part_o, float* part_ml, float scale, int window,
                                         int split_len, int n_splits, int page_size, int n_seq, int n_tiles,
                                         int tile_rows, int Hq, int Hkv, int Dh, int* split_counter,
                                         cudaStream_t stream);
extern "C" int pmm_flash_combine(const float* part_o, const float* part_ml, void* out, int n_rows,
                                 int n_splits, int Dh, int dtype, cudaStream_t stream);

namespace {

// Partial results of the key splits: [rows, n_splits, Dh] outputs, then [rows, n_splits, 2]
// (max, sum).  Lives in every GPU's memory from library load to process exit.
static __device__ __align__(256) float g_noalloc_scratch[PMM_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
// In host code g_noalloc_scratch is only a handle for the runtime, not an address a kernel
// can use; the device address is asked for once per device and kept here.
// Host threads may make their first calls at the same time: the table is filled under a lock.
float* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_addr_lock;
thread_local char g_last_error[256] = "";

int fail(int code, const char* fmt, long long a = 0, long long b = 0) {
  snprintf(g_last_error, sizeof(g_last_error), fmt, a, b);
  return code;
}

// Device address of the scratch array on the current device (looked up at the first call there).
int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices)
    return fail(PMM_ERR_NOALLOC_SETUP, "cannot tell the current device (cuda error %lld, device %lld)",
                static_cast<long long>(e), dev);
  std::lock_guard<std::mutex> guard(g_scratch_addr_lock);
  if (!g_scratch_addr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || !p)
      return fail(PMM_ERR_NOALLOC_SETUP, "cudaGetSymbolAddress failed on device %lld (cuda error %lld)", dev,
                  static_cast<long long>(e));
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace

PMM_EXPORT int pmm_attention_noalloc(const void* q, const void* pool, const int* block_table, int max_blocks,
                                     const int* positions, const int* cu, void* out, float scale, int window,
                                     int split_len, int n_splits, int page_size, int n_seq, int n_tokens,
                                     int n_tiles, int rows16, int Hq, int Hkv, int Dh, cudaStream_t stream) {
  g_last_error[0] = 0;
  if (n_seq <= 0 || n_tokens <= 0 || n_tiles <= 0) return 0;
  // Everything the two launchers would refuse is refused here, before anything is launched, so
  // that a refused call never leaves half its work behind and always leaves a sentence.
  const int tile_rows = rows16 ? 16 : 64;
  if (!pmm_flash_supported(Hq, Hkv, Dh))
    return fail(PMM_ERR_BAD_ARGUMENT, "head shape (%lld query heads of size %lld) outside what the kernel supports",
                Hq, Dh);
  if (Hq / Hkv > tile_rows)
    return fail(PMM_ERR_BAD_ARGUMENT, "%lld query heads per key head do not fit a row tile of %lld", Hq / Hkv,
                tile_rows);
  if (n_splits < 1 || n_splits > PMM_NOALLOC_MAX_SPLITS)
    return fail(PMM_ERR_BAD_ARGUMENT, "n_splits is %lld; 1 to %lld are supported", n_splits, PMM_NOALLOC_MAX_SPLITS);
  if (!(scale > 0.f) || page_size <= 0 || Hkv > 65535 || (n_splits > 1 && split_len <= 0))
    return fail(PMM_ERR_BAD_ARGUMENT, "scale, page_size and split_len must be positive (page_size %lld, split_len %lld)",
                page_size, split_len);
  if (!q || !pool || !block_table || !positions || !cu || !out)
    return fail(PMM_ERR_BAD_ARGUMENT, "a null pointer among the inputs and outputs");
  if (n_splits == 1) {  // no partial results, so no scratch: the regular path allocates nothing either
    int rc1 = pmm_flash_paged_attention(q, pool, block_table, max_blocks, positions, cu, out, nullptr, nullptr, scale,
                                        window, split_len, 1, page_size, n_seq, n_tiles, tile_rows, Hq, Hkv, Dh,
                                        nullptr, stream);
    return rc1 == 0 ? 0 : fail(rc1, "attention launch failed (code %lld)", rc1);
  }
  const long long rows = static_cast<long long>(n_tokens) * Hq;
  const long long need = rows * n_splits * (Dh + 2);
  if (need > PMM_NOALLOC_SCRATCH_FLOATS)
    return fail(PMM_ERR_NOALLOC_TOO_LARGE,
                "this call needs %lld floats of scratch for its key splits but the built-in array holds %lld; "
                "use fewer tokens or splits per call, or the entry point that takes caller scratch",
                need, static_cast<long long>(PMM_NOALLOC_SCRATCH_FLOATS));
  float* scratch = nullptr;
  if (int rc = scratch_for_current_device(&scratch)) return rc;
  float* part_o = scratch;
  float* part_ml = scratch + rows * n_splits * Dh;
  int rc = pmm_flash_paged_attention(q, pool, block_table, max_blocks, positions, cu, out, part_o, part_ml, scale,
                                     window, split_len, n_splits, page_size, n_seq, n_tiles, tile_rows, Hq, Hkv, Dh,
                                     nullptr, stream);
  if (rc != 0) return fail(rc, "attention launch failed (code %lld)", rc);
  rc = pmm_flash_combine(part_o, part_ml, out, static_cast<int>(rows), n_splits, Dh, PMM_DTYPE_BF16, stream);
  if (rc != 0) return fail(rc, "merge launch failed (code %lld)", rc);
  return 0;
}

PMM_EXPORT const char* pmm_attention_noalloc_last_error(void) { return g_last_error; }
