// extern "C" surface of libdsa_b200.so (declared in include/dsa_b200.h): argument
// checks, error strings and the calls into the kernel launchers.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "dsa_host.h"

namespace dsa {

struct IndexerArgs;   // defined with the kernel

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return set_error(DSA_ERR_CUDA, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return DSA_OK;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cached[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

// launchers implemented next to their kernels
int indexer_logits_contiguous(const void* q, const void* k, const float* k_scale, const void* w, int w_dtype,
                              const int32_t* ks, const int32_t* ke, float* logits, int64_t ld, int T, int S,
                              int H, int D, int clean, int general, int32_t* status, cudaStream_t stream);
int indexer_logits_paged(const void* q, const void* w, int w_dtype, const void* kcache, const float* kscale,
                         const int32_t* block_table, int64_t table_stride, const int32_t* ctx_len, float* logits,
                         int64_t ld, int B, int H, int D, int num_pages, int max_ctx, int32_t* status,
                         cudaStream_t stream);
int topk_select_launch(const float* logits, int64_t ld, const int32_t* ks, const int32_t* ke, int T, int S, int k,
                       int32_t* out, int sample, cudaStream_t stream);
int bounded_wait_probe_launch(uint32_t poll_limit, int32_t* status, cudaStream_t stream);

int sparse_mla_prefill_launch(const void* q, const void* kv, const int32_t* idx, void* out, int T, int H, int S_kv,
                              int K, float scale, int32_t* status, cudaStream_t stream);
int sparse_mla_decode_launch(const void* q, const void* cache, const int32_t* block_table, int64_t table_stride,
                             const int32_t* idx, void* out, int B, int H, int K, int num_pages, int max_ctx,
                             float scale, void* workspace, size_t workspace_bytes, int32_t* status,
                             cudaStream_t stream);
size_t mla_decode_workspace_bytes(int B, int H, int K);
int block_sparse_mha_launch(const void* q, const void* k, const void* v, const int32_t* lut, const int32_t* num,
                            void* out, int B, int S, int H, int topk, float scale, int32_t* status,
                            cudaStream_t stream);

int fp8_quant_launch(const void* x, int x_is_bf16, int64_t n_blocks, int block, void* q, float* scale,
                     cudaStream_t stream);
int rope_fp8_quant_launch(const void* x, int64_t n_rows, int head_dim, int rope_dim, int interleave, int rows_per_pos,
                          const float* cos_t, const float* sin_t, void* q, float* scale, cudaStream_t stream);

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace dsa

using namespace dsa;

static int indexer_logits_checked(const void* q_fp8, const void* k_fp8, const float* k_scale, const void* w, int w_dtype,
                                  const int32_t* ks, const int32_t* ke, float* logits, int64_t ld_logits, int T, int S,
                                  int H, int D, int clean, int general, int32_t* status, void* stream) {
  g_err[0] = 0;
  if (T < 0 || S < 0) return set_error(DSA_ERR_SHAPE, "indexer_logits: negative size (T=%d, S=%d)", T, S);
  if (T == 0 || S == 0) return DSA_OK;
  if (!q_fp8 || !k_fp8 || !k_scale || !w || !ke || !logits)
    return set_error(DSA_ERR_ARG, "indexer_logits: NULL pointer argument");
  if (w_dtype != DSA_W_F32 && w_dtype != DSA_W_BF16)
    return set_error(DSA_ERR_ARG, "indexer_logits: w_dtype must be DSA_W_F32 or DSA_W_BF16");
  if (ld_logits < S) return set_error(DSA_ERR_SHAPE, "indexer_logits: ld_logits (%lld) < S (%d)", (long long)ld_logits, S);
  if (!aligned16(q_fp8) || !aligned16(k_fp8))
    return set_error(DSA_ERR_ALIGN, "indexer_logits: q_fp8 and k_fp8 must be 16-byte aligned");
  if ((int64_t)T * H > 0x7fffffffLL) return set_error(DSA_ERR_SHAPE, "indexer_logits: T*H exceeds 2^31");
  if (ld_logits * 64 > 0x7fffffffLL)
    return set_error(DSA_ERR_SHAPE, "indexer_logits: ld_logits (%lld) too large (64 * ld must stay below 2^31)",
                     (long long)ld_logits);
  return indexer_logits_contiguous(q_fp8, k_fp8, k_scale, w, w_dtype, ks, ke, logits, ld_logits, T, S, H, D, clean,
                                   general, status, static_cast<cudaStream_t>(stream));
}

static int topk_select_checked(const float* logits, int64_t ld_logits, const int32_t* ks, const int32_t* ke, int T, int S,
                               int k, int32_t* out_idx, int sample, void* stream) {
  g_err[0] = 0;
  if (T < 0 || S < 0 || k < 0) return set_error(DSA_ERR_SHAPE, "topk_select: negative size");
  if (T == 0 || k == 0) return DSA_OK;
  if (!logits || !out_idx) return set_error(DSA_ERR_ARG, "topk_select: NULL pointer argument");
  if (ld_logits < S) return set_error(DSA_ERR_SHAPE, "topk_select: ld_logits < S");
  if (k > 65535) return set_error(DSA_ERR_SHAPE, "topk_select: k (%d) exceeds 65535", k);
  return topk_select_launch(logits, ld_logits, ks, ke, T, S, k, out_idx, sample, static_cast<cudaStream_t>(stream));
}

extern "C" {

int dsa_version(void) { return 100; }

const char* dsa_last_error_string(void) { return g_err; }

int dsa_indexer_logits(const void* q_fp8, const void* k_fp8, const float* k_scale, const void* w, int w_dtype,
                       const int32_t* ks, const int32_t* ke, float* logits, int64_t ld_logits, int T, int S,
                       int H, int D, int clean, int32_t* status, void* stream) {
  return indexer_logits_checked(q_fp8, k_fp8, k_scale, w, w_dtype, ks, ke, logits, ld_logits, T, S, H, D, clean,
                                /*general=*/0, status, stream);
}

/* Test hooks (declared in include/dsa_b200.h under "test hooks"): the same calls pinned to the code path that the
 * normal entry points only take for some shapes or rows, so that tests can compare the two. */
int dsa_test_indexer_logits_general(const void* q_fp8, const void* k_fp8, const float* k_scale, const void* w,
                                    int w_dtype, const int32_t* ks, const int32_t* ke, float* logits,
                                    int64_t ld_logits, int T, int S, int H, int D, int clean, int32_t* status,
                                    void* stream) {
  return indexer_logits_checked(q_fp8, k_fp8, k_scale, w, w_dtype, ks, ke, logits, ld_logits, T, S, H, D, clean,
                                /*general=*/1, status, stream);
}

int dsa_test_topk_select_two_pass(const float* logits, int64_t ld_logits, const int32_t* ks, const int32_t* ke, int T,
                                  int S, int k, int32_t* out_idx, void* stream) {
  return topk_select_checked(logits, ld_logits, ks, ke, T, S, k, out_idx, /*sample=*/0, stream);
}

int dsa_test_bounded_wait(int poll_limit, int32_t* status, void* stream) {
  g_err[0] = 0;
  if (poll_limit < 1 || poll_limit > (1 << 16)) return set_error(DSA_ERR_ARG, "test_bounded_wait: poll_limit must be in [1, 65536]");
  if (!status) return set_error(DSA_ERR_ARG, "test_bounded_wait: NULL status");
  return bounded_wait_probe_launch((uint32_t)poll_limit, status, static_cast<cudaStream_t>(stream));
}

int dsa_indexer_logits_paged(const void* q_fp8, const void* w, int w_dtype, const void* kcache,
                             const float* kscale, const int32_t* block_table, int64_t table_stride,
                             const int32_t* ctx_len, float* logits, int64_t ld_logits, int B, int H, int D,
                             int num_pages, int max_ctx, int32_t* status, void* stream) {
  g_err[0] = 0;
  if (B < 0 || max_ctx < 0 || num_pages < 0)
    return set_error(DSA_ERR_SHAPE, "indexer_logits_paged: negative size");
  if (B == 0 || max_ctx == 0) return DSA_OK;
  if (!q_fp8 || !w || !kcache || !kscale || !block_table || !ctx_len || !logits)
    return set_error(DSA_ERR_ARG, "indexer_logits_paged: NULL pointer argument");
  if (w_dtype != DSA_W_F32 && w_dtype != DSA_W_BF16)
    return set_error(DSA_ERR_ARG, "indexer_logits_paged: bad w_dtype");
  if (ld_logits < max_ctx) return set_error(DSA_ERR_SHAPE, "indexer_logits_paged: ld_logits < max_ctx");
  if (ld_logits * 64 > 0x7fffffffLL) return set_error(DSA_ERR_SHAPE, "indexer_logits_paged: ld_logits too large");
  if (table_stride * 64 < max_ctx)
    return set_error(DSA_ERR_SHAPE, "indexer_logits_paged: block table row (%lld pages) shorter than max_ctx %d",
                     (long long)table_stride, max_ctx);
  if (!aligned16(q_fp8) || !aligned16(kcache) || !aligned16(kscale))
    return set_error(DSA_ERR_ALIGN, "indexer_logits_paged: q_fp8, kcache and kscale must be 16-byte aligned");
  if ((int64_t)num_pages * 64 > 0x7fffffffLL) return set_error(DSA_ERR_SHAPE, "indexer_logits_paged: cache too large");
  return indexer_logits_paged(q_fp8, w, w_dtype, kcache, kscale, block_table, table_stride, ctx_len, logits,
                              ld_logits, B, H, D, num_pages, max_ctx, status, static_cast<cudaStream_t>(stream));
}

int dsa_topk_select(const float* logits, int64_t ld_logits, const int32_t* ks, const int32_t* ke, int T, int S,
                    int k, int32_t* out_idx, void* stream) {
  return topk_select_checked(logits, ld_logits, ks, ke, T, S, k, out_idx, /*sample=*/1, stream);
}

int dsa_sparse_mla_prefill(const void* q_bf16, const void* kv_bf16, const int32_t* idx, void* out_bf16, int T, int H,
                           int S_kv, int K, float scale, int32_t* status, void* stream) {
  g_err[0] = 0;
  if (T < 0 || H < 0 || S_kv < 0 || K < 0) return set_error(DSA_ERR_SHAPE, "sparse_mla_prefill: negative size");
  if (T == 0 || H == 0) return DSA_OK;
  if (!q_bf16 || !out_bf16 || (K > 0 && (!idx || !kv_bf16)))
    return set_error(DSA_ERR_ARG, "sparse_mla_prefill: NULL pointer argument");
  if (!aligned16(q_bf16) || !aligned16(kv_bf16) || !aligned16(out_bf16))
    return set_error(DSA_ERR_ALIGN, "sparse_mla_prefill: q, kv and out must be 16-byte aligned");
  if ((int64_t)T * H > 0x7fffffffLL || T > 0x7fffffff / 2) return set_error(DSA_ERR_SHAPE, "sparse_mla_prefill: T*H too large");
  if (H > 128 * 65535) return set_error(DSA_ERR_SHAPE, "sparse_mla_prefill: too many heads");
  if (K > 2048) return set_error(DSA_ERR_SHAPE, "sparse_mla_prefill: K (%d) exceeds 2048 selected keys per query", K);
  if (!(scale > 0.f)) return set_error(DSA_ERR_ARG, "sparse_mla_prefill: the softmax scale must be positive");
  return sparse_mla_prefill_launch(q_bf16, kv_bf16, idx, out_bf16, T, H, S_kv, K, scale, status,
                                   static_cast<cudaStream_t>(stream));
}

int dsa_block_sparse_mha(const void* q_bf16, const void* k_bf16, const void* v_bf16, const int32_t* lut,
                         const int32_t* num, void* out_bf16, int B, int S, int H, int D, int topk, float scale,
                         int32_t* status, void* stream) {
  g_err[0] = 0;
  if (B < 0 || S < 0 || H < 0 || topk < 0) return set_error(DSA_ERR_SHAPE, "block_sparse_mha: negative size");
  if (D != 128) return set_error(DSA_ERR_SHAPE, "block_sparse_mha: head dim %d, only 128 is built", D);
  if (!(scale > 0.f)) return set_error(DSA_ERR_ARG, "block_sparse_mha: the softmax scale must be positive");
  if (S % 64) return set_error(DSA_ERR_SHAPE, "block_sparse_mha: S (%d) must be a multiple of the 64-token block", S);
  if (B == 0 || S == 0 || H == 0) return DSA_OK;
  if (!q_bf16 || !k_bf16 || !v_bf16 || !out_bf16 || !num || (topk > 0 && !lut))
    return set_error(DSA_ERR_ARG, "block_sparse_mha: NULL pointer argument");
  if (!aligned16(q_bf16) || !aligned16(k_bf16) || !aligned16(v_bf16) || !aligned16(out_bf16))
    return set_error(DSA_ERR_ALIGN, "block_sparse_mha: q, k, v and out must be 16-byte aligned");
  if ((int64_t)B * S > 0x7fffffffLL || H > 65535 || B > 65535)
    return set_error(DSA_ERR_SHAPE, "block_sparse_mha: B*S, H or B too large");
  return block_sparse_mha_launch(q_bf16, k_bf16, v_bf16, lut, num, out_bf16, B, S, H, topk, scale, status,
                                 static_cast<cudaStream_t>(stream));
}

int dsa_sparse_mla_decode_paged(const void* q_bf16, const void* cache, const int32_t* block_table,
                                int64_t table_stride, const int32_t* idx, void* out_bf16, int B, int H, int K,
                                int num_pages, int max_ctx, float scale, void* workspace, size_t workspace_bytes,
                                int32_t* status, void* stream) {
  g_err[0] = 0;
  if (B < 0 || H < 0 || K < 0 || num_pages < 0 || max_ctx < 0)
    return set_error(DSA_ERR_SHAPE, "sparse_mla_decode_paged: negative size");
  if (B == 0 || H == 0) return DSA_OK;
  if (!q_bf16 || !out_bf16 || (K > 0 && (!idx || !cache || !block_table)))
    return set_error(DSA_ERR_ARG, "sparse_mla_decode_paged: NULL pointer argument");
  if (!aligned16(q_bf16) || !aligned16(cache) || !aligned16(out_bf16))
    return set_error(DSA_ERR_ALIGN, "sparse_mla_decode_paged: q, cache and out must be 16-byte aligned");
  if (table_stride * 64 < max_ctx)
    return set_error(DSA_ERR_SHAPE, "sparse_mla_decode_paged: block table row shorter than max_ctx");
  if (K > 2048) return set_error(DSA_ERR_SHAPE, "sparse_mla_decode_paged: K (%d) exceeds 2048 selected keys per query", K);
  if (!(scale > 0.f)) return set_error(DSA_ERR_ARG, "sparse_mla_decode_paged: the softmax scale must be positive");
  if ((int64_t)num_pages * 64 > 0x7fffffffLL || (int64_t)B * H > 0x7fffffffLL)
    return set_error(DSA_ERR_SHAPE, "sparse_mla_decode_paged: problem too large");
  if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 15))
    return set_error(DSA_ERR_WORKSPACE, "sparse_mla_decode_paged: workspace must be 16-byte aligned");
  return sparse_mla_decode_launch(q_bf16, cache, block_table, table_stride, idx, out_bf16, B, H, K, num_pages,
                                  max_ctx, scale, workspace, workspace_bytes, status, static_cast<cudaStream_t>(stream));
}

size_t dsa_sparse_mla_decode_workspace_bytes(int B, int H, int K) {
  if (B <= 0 || H <= 0 || K <= 0) return 0;
  return mla_decode_workspace_bytes(B, H, K);
}

int dsa_fp8_quant_per_block(const void* x, int x_dtype, int64_t n_blocks, int block_size, void* q_fp8, float* scale,
                            void* stream) {
  g_err[0] = 0;
  if (n_blocks < 0) return set_error(DSA_ERR_SHAPE, "fp8_quant_per_block: negative size");
  if (n_blocks == 0) return DSA_OK;
  if (!x || !q_fp8 || !scale) return set_error(DSA_ERR_ARG, "fp8_quant_per_block: NULL pointer argument");
  if (x_dtype != DSA_X_F32 && x_dtype != DSA_X_BF16) return set_error(DSA_ERR_ARG, "fp8_quant_per_block: bad x_dtype");
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(q_fp8) & 3))
    return set_error(DSA_ERR_ALIGN, "fp8_quant_per_block: x must be 16-byte and q_fp8 4-byte aligned");
  return fp8_quant_launch(x, x_dtype == DSA_X_BF16, n_blocks, block_size, q_fp8, scale, static_cast<cudaStream_t>(stream));
}

int dsa_rope_fp8_quant(const void* x_bf16, int64_t n_rows, int head_dim, int rope_dim, int interleave, int rows_per_pos,
                       const float* cos_table, const float* sin_table, int64_t n_pos, void* q_fp8, float* scale,
                       void* stream) {
  g_err[0] = 0;
  if (n_rows < 0 || n_pos < 0) return set_error(DSA_ERR_SHAPE, "rope_fp8_quant: negative size");
  if (n_rows == 0) return DSA_OK;
  if (!x_bf16 || !cos_table || !sin_table || !q_fp8 || !scale) return set_error(DSA_ERR_ARG, "rope_fp8_quant: NULL pointer argument");
  if (head_dim != 64 && head_dim != 128) return set_error(DSA_ERR_SHAPE, "rope_fp8_quant: head dim %d, only 64 and 128 are built", head_dim);
  // the rotated part is made of whole lanes (head_dim / 32 values each) and, in the halves form, of two equal lane groups
  const int per = head_dim / 32;
  if (rope_dim <= 0 || rope_dim > head_dim || rope_dim % (2 * per)) return set_error(DSA_ERR_SHAPE, "rope_fp8_quant: rope_dim %d does not fit head dim %d", rope_dim, head_dim);
  if (!interleave && ((rope_dim / 2 / per) & (rope_dim / 2 / per - 1))) return set_error(DSA_ERR_SHAPE, "rope_fp8_quant: rope_dim / 2 must span a power-of-two number of lanes");
  if (rows_per_pos <= 0 || (n_rows + rows_per_pos - 1) / rows_per_pos > n_pos)
    return set_error(DSA_ERR_SHAPE, "rope_fp8_quant: %lld rows at %d per position need more than the %lld positions of the tables",
                     (long long)n_rows, rows_per_pos, (long long)n_pos);
  if (!aligned16(x_bf16) || (reinterpret_cast<uintptr_t>(q_fp8) & 3)) return set_error(DSA_ERR_ALIGN, "rope_fp8_quant: x must be 16-byte and q_fp8 4-byte aligned");
  return rope_fp8_quant_launch(x_bf16, n_rows, head_dim, rope_dim, interleave, rows_per_pos, cos_table, sin_table, q_fp8, scale,
                               static_cast<cudaStream_t>(stream));
}

static const int kMinChunkRows = 256;

static int64_t logits_ld(int S) { return ((int64_t)S + 3) & ~int64_t(3); }

size_t dsa_indexer_topk_workspace_bytes(int T, int S) {
  if (T <= 0 || S <= 0) return 0;
  return (size_t)T * (size_t)logits_ld(S) * sizeof(float);
}

int dsa_indexer_topk(const void* q_fp8, const void* k_fp8, const float* k_scale, const void* w, int w_dtype,
                     const int32_t* ks, const int32_t* ke, int T, int S, int H, int D, int k, int32_t* out_idx,
                     void* workspace, size_t workspace_bytes, int32_t* status, void* stream) {
  g_err[0] = 0;
  if (T < 0 || S < 0 || k < 0) return set_error(DSA_ERR_SHAPE, "indexer_topk: negative size");
  if (T == 0 || k == 0) return DSA_OK;
  if (S == 0) return set_error(DSA_ERR_SHAPE, "indexer_topk: S = 0 with k > 0");
  if (!out_idx || !ke) return set_error(DSA_ERR_ARG, "indexer_topk: NULL pointer argument");
  const int64_t ld = logits_ld(S);
  const size_t row_bytes = (size_t)ld * sizeof(float);
  if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 15))
    return set_error(DSA_ERR_WORKSPACE, "indexer_topk: workspace missing or not 16-byte aligned");
  int64_t rows = (int64_t)(workspace_bytes / row_bytes);
  const int min_rows = T < kMinChunkRows ? T : kMinChunkRows;
  if (rows < min_rows)
    return set_error(DSA_ERR_WORKSPACE, "indexer_topk: workspace %zu B holds %lld rows, need >= %d (%zu B)",
                     workspace_bytes, (long long)rows, min_rows, (size_t)min_rows * row_bytes);
  if (rows > T) rows = T;
  if (rows < T) rows &= ~int64_t(kMinChunkRows - 1);   // whole query groups per chunk
  float* logits = static_cast<float*>(workspace);
  const size_t w_elt = w_dtype == DSA_W_BF16 ? 2 : 4;
  for (int64_t r0 = 0; r0 < T; r0 += rows) {
    const int n = (int)((T - r0 < rows) ? T - r0 : rows);
    int rc = dsa_indexer_logits(static_cast<const uint8_t*>(q_fp8) + (size_t)r0 * H * D, k_fp8, k_scale,
                                static_cast<const uint8_t*>(w) + (size_t)r0 * H * w_elt, w_dtype,
                                ks ? ks + r0 : nullptr, ke + r0, logits, ld, n, S, H, D, /*clean=*/0, status, stream);
    if (rc) return rc;
    rc = dsa_topk_select(logits, ld, ks ? ks + r0 : nullptr, ke + r0, n, S, k, out_idx + (size_t)r0 * k, stream);
    if (rc) return rc;
  }
  return DSA_OK;
}

}  // extern "C"
