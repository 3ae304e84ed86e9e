// dsa_indexer_topk_static: indexer logits + top-k for callers that cannot allocate.
//
// Some hosts of this library have no way to hand over a workspace: a serving
// loop whose memory pool is frozen once it starts, a plugin called from a
// runtime that owns all device memory and forbids cudaMalloc in its callbacks,
// an embedding whose allocator is not re-entrant.
// For them the fp32 logits scratch of dsa_indexer_topk lives here, in a
// file-scope device array that every GPU loading the library holds until exit.
#include <mutex>

#include "dsa_host.h"

namespace dsa {

// 64 MiB of fp32 logits: 256 query rows x 65536 keys per chunk.
constexpr size_t kStaticScratchBytes = size_t(64) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// The array's name is only a host-side handle; kernels need the device address,
// looked up once per device with that device current.  Under CUDA's lazy module
// loading this lookup is also the moment the driver creates the array's 64 MiB on
// that device, so it can fail with "out of memory" on a GPU that is already full:
// hosts make one T = 0 call per device at start-up, before they freeze their pool.
static void* static_scratch_ptr() {
  static void* ptrs[64] = {nullptr};
  static std::mutex mu;
  std::lock_guard<std::mutex> lock(mu);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
    set_error(DSA_ERR_CUDA, "indexer_topk_static: cannot query the current device");
    return nullptr;
  }
  if (!ptrs[dev]) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) {
      set_error(DSA_ERR_CUDA, "indexer_topk_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    ptrs[dev] = p;
  }
  return ptrs[dev];
}

}  // namespace dsa

extern "C" size_t dsa_indexer_topk_static_max_bytes(void) { return dsa::kStaticScratchBytes; }

extern "C" int dsa_indexer_topk_static(const void* q_fp8, const void* k_fp8, const float* k_scale, const void* w,
                                       int w_dtype, const int32_t* ks, const int32_t* ke, int T, int S, int H, int D,
                                       int k, int32_t* out_idx, int32_t* status, void* stream) {
  dsa::set_error(DSA_OK, "%s", "");      // a fresh call starts with an empty error string, like the other entry points
  if (T > 0 && S > 0) {
    // one chunk of min(T, 256) rows of the padded row length must fit
    const size_t ld = (size_t(S) + 3) & ~size_t(3);
    const size_t rows = T < 256 ? size_t(T) : 256;
    if (rows * ld * sizeof(float) > dsa::kStaticScratchBytes)
      return dsa::set_error(DSA_ERR_WORKSPACE,
                            "indexer_topk_static: %zu rows x %d keys need %zu B of scratch, the built-in array holds "
                            "%zu B (at most 65536 keys with 256 or more query rows); use dsa_indexer_topk",
                            rows, S, rows * ld * sizeof(float), dsa::kStaticScratchBytes);
  }
  void* scratch = dsa::static_scratch_ptr();
  if (!scratch) return DSA_ERR_CUDA;
  return dsa_indexer_topk(q_fp8, k_fp8, k_scale, w, w_dtype, ks, ke, T, S, H, D, k, out_idx, scratch,
                          dsa::kStaticScratchBytes, status, stream);
}
