// Weights of the next layer pulled into L2 while the current layer runs.
//
// A decode step of few tokens reads every weight once; each kernel alone moves a few megabytes
// and is over before DRAM reaches its steady rate.  One small launch per layer asks the memory
// system for the next layer's weights with cp.async.bulk.prefetch.L2 (a hint: nothing waits for
// it and nothing depends on it), so that the kernels of that layer find them in the 126 MB L2.
// It is issued beside the products that follow the mixers (latency-bound, memory idle), not
// beside the mixers (which read caches and states at the memory's full rate: there it cost more
// than it gained).  The requests pass through each SM's copy engine, whose rate is limited: a
// warp on each of some tens of SMs (two blocks took 35 us a layer; a request stream spread over
// all 148 SMs with scattered chunks per SM slowed the products beside it).  Also measured: asking
// for the next layer's cache pages and states in the same way makes the step slower (1.43 against
// 1.19 ms): 48 MB a layer no longer fit beside the current layer's own traffic.
#include "common.cuh"

namespace pmm {

constexpr int kPrefetchRanges = 8;
// bytes per request: inside a decode step of the 0.5B sizes, 4 and 8 KB are alike, 16 KB costs 3 to 4 %
// of the step at 4 and 8 tokens, 64 and 256 KB triple it (the requests then block the copy engines)
constexpr unsigned kPrefetchChunk = 8 * 1024;
constexpr int kPrefetchBlocks = 50;              // one warp each; 24 to 100 measured alike

struct PrefetchArgs {
  const char* ptr[kPrefetchRanges];
  unsigned long long bytes[kPrefetchRanges];  // multiples of 16
  int n;
};

__global__ void __launch_bounds__(32) l2_prefetch_kernel(PrefetchArgs a) {
  for (int r = 0; r < a.n; ++r) {
    const unsigned long long chunks = (a.bytes[r] + kPrefetchChunk - 1) / kPrefetchChunk;
    for (unsigned long long c = blockIdx.x * blockDim.x + threadIdx.x; c < chunks;
         c += static_cast<unsigned long long>(gridDim.x) * blockDim.x) {
      const unsigned long long off = c * kPrefetchChunk;
      const unsigned long long left = a.bytes[r] - off;
      const unsigned size = left < kPrefetchChunk ? static_cast<unsigned>(left) : kPrefetchChunk;
      asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;\n" ::"l"(a.ptr[r] + off), "r"(size) : "memory");
    }
  }
}

}  // namespace pmm

// Up to 8 ranges (16-byte aligned start; the length is rounded down to a multiple of 16).
PMM_EXPORT int pmm_l2_prefetch(const void* const* ptrs, const long long* bytes, int n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (n > pmm::kPrefetchRanges) return PMM_ERR_BAD_ARGUMENT;
  pmm::PrefetchArgs a{};
  a.n = n;
  for (int i = 0; i < n; ++i) {
    if (!ptrs[i] || bytes[i] < 0 || reinterpret_cast<uintptr_t>(ptrs[i]) % 16) return PMM_ERR_BAD_ARGUMENT;
    a.ptr[i] = static_cast<const char*>(ptrs[i]);
    a.bytes[i] = static_cast<unsigned long long>(bytes[i]) / 16 * 16;
  }
  pmm::l2_prefetch_kernel<<<pmm::kPrefetchBlocks, 32, 0, stream>>>(a);
  return pmm::launch_status();
}
