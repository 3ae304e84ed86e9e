/* C ABI of libdsa_b200.so: the sm_100a kernels of the DeepSeek Sparse Attention
 * (DSA) hot path -- lightning-indexer logits, per-row top-k selection and sparse
 * MLA -- behind plain pointers and sizes.
 *
 * The reference project (sparse_attn/DSA.py) has no native ABI: it reaches its
 * GPU kernels through late-bound Python imports.  Each entry point below names
 * the reference call site it stands in for.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its comment says "host".
 *   - The caller owns all buffers (inputs, outputs, workspace, status word); the
 *     library allocates nothing and keeps no pointer after the call returns.
 *   - Calls are asynchronous on `stream` (a cudaStream_t passed as void*; NULL =
 *     the default stream) and never synchronise.
 *   - Return value: 0 on success, a negative DSA_ERR_* code otherwise; nothing is
 *     launched on error and dsa_last_error_string() describes it.
 *   - `status` (may be NULL) is one int32 in device memory, zeroed by the caller.
 *     Kernels write a non-zero code there instead of faulting: 1 = an internal
 *     bounded wait expired, 2 = an index or page id was out of range (the access
 *     was skipped).  Read it after synchronising when you want to check.
 */
#ifndef DSA_B200_H_
#define DSA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DSA_OK 0
#define DSA_ERR_SHAPE (-1)     /* unsupported or inconsistent sizes */
#define DSA_ERR_ALIGN (-2)     /* pointer or stride alignment */
#define DSA_ERR_WORKSPACE (-3) /* workspace missing or too small */
#define DSA_ERR_CUDA (-4)      /* a CUDA runtime / driver call failed */
#define DSA_ERR_ARG (-5)       /* NULL pointer or bad flag */

#define DSA_W_F32 0
#define DSA_W_BF16 1
#define DSA_X_F32 0
#define DSA_X_BF16 1

/* Library version (major*10000 + minor*100 + patch). */
int dsa_version(void);
/* Message of the most recent error on the calling thread ("" if none). */
const char* dsa_last_error_string(void);

/* Per-block FP8 quantiser, one kernel.  Stands in for fp8_quant_per_block
 * (sparse_attn/DSA.py:102-132): for every block of block_size (64 or 128)
 * consecutive values, scale = max(absmax, 1e-6) / 448 (fp32) and
 * q = round_to_e4m3(x / scale).  x is fp32 (DSA_X_F32) or bf16 (DSA_X_BF16),
 * n_blocks * block_size values, 16-byte aligned; q_fp8 gets one byte per value,
 * scale one fp32 per block.  Bytes and scales equal the reference's CPU result. */
int dsa_fp8_quant_per_block(const void* x, int x_dtype, int64_t n_blocks, int block_size, void* q_fp8, float* scale,
                            void* stream);

/* RoPE + per-row FP8 quantiser in one pass: stands in for DsaIndexer.rope followed by fp8_quant_per_block
 * (sparse_attn/DSA.py:513-524, 530-531).  x_bf16 [n_rows, head_dim] (head_dim 64 or 128 = one FP8 block per
 * row); row r is at position r / rows_per_pos (heads per token for q, 1 for k); cos_table / sin_table
 * [n_pos, rope_dim / 2] fp32 as built by the reference's _rope_cossin (DSA.py:430-441).  The first rope_dim values
 * of a row are rotated -- halves form (interleave = 0: fp32 products, not rounded, DSA.py:444-454) or even/odd
 * pairs (interleave = 1: rounded to bf16, DSA.py:457-469) -- with the reference's operation order, then the row is
 * quantised: bytes and scales equal the eager chain's. */
int dsa_rope_fp8_quant(const void* x_bf16, int64_t n_rows, int head_dim, int rope_dim, int interleave, int rows_per_pos,
                       const float* cos_table, const float* sin_table, int64_t n_pos, void* q_fp8, float* scale,
                       void* stream);

/* Lightning-indexer logits, contiguous keys.
 *   logits[t, s] = k_scale[s] * sum_h w[t,h] * relu(q[t,h,:] . k[s,:])  for ks[t] <= s < ke[t].
 * Stands in for deep_gemm.fp8_mqa_logits(q_fp8, (k_fp8, k_scale), w, ks, ke) as
 * called at sparse_attn/DSA.py:343-345, 547-552, 654-659.
 *   q_fp8   [T, H, D] e4m3, contiguous, 16-byte aligned
 *   k_fp8   [S, D]    e4m3, contiguous, 16-byte aligned
 *   k_scale [S] fp32;  w [T, H] fp32 (DSA_W_F32) or bf16 (DSA_W_BF16), q scale folded in
 *   ks, ke  [T] int32 (ks may be NULL = 0)
 *   logits  [T, ld_logits] fp32, ld_logits >= S
 * Supported: H in {4,8,16,32,64} with D = 128, and H in {4,64} with D = 64.
 * clean != 0 also writes -inf to every column outside the window (the library
 * call's default); clean == 0 leaves columns that lie in fully masked 128-key
 * tiles untouched, which is all dsa_topk_select needs. */
int dsa_indexer_logits(const void* q_fp8, const void* k_fp8, const float* k_scale, const void* w, int w_dtype,
                       const int32_t* ks, const int32_t* ke, float* logits, int64_t ld_logits, int T, int S,
                       int H, int D, int clean, int32_t* status, void* stream);

/* Lightning-indexer logits for decode over a paged FP8 key cache: one query
 * token per sequence.  No counterpart call in the reference (it has no cache,
 * sparse_attn/DSA.py:475-477); same arithmetic as dsa_indexer_logits with
 * ks = 0, ke = ctx_len[b] and key s of sequence b stored at physical row
 * block_table[b, s/64]*64 + s%64.
 *   q_fp8 [B, H, 128] e4m3; w [B, H]; kcache [num_pages*64, 128] e4m3;
 *   kscale [num_pages*64] fp32; block_table [B, table_stride] int32;
 *   ctx_len [B] int32; logits [B, ld_logits] fp32, ld_logits >= max_ctx.
 * Columns >= ctx_len[b] inside a processed tile get -inf; beyond are untouched. */
int dsa_indexer_logits_paged(const void* q_fp8, const void* w, int w_dtype, const void* kcache,
                             const float* kscale, const int32_t* block_table, int64_t table_stride,
                             const int32_t* ctx_len, float* logits, int64_t ld_logits, int B, int H, int D,
                             int num_pages, int max_ctx, int32_t* status, void* stream);

/* Per-row top-k by radix select.  Stands in for logits.topk(k).indices at
 * sparse_attn/DSA.py:361, 567, 675-676.  Row t considers columns
 * [ks[t], min(ke[t], S)) only (ks NULL = 0, ke NULL = S) and writes k int32
 * column indices to out_idx[t, 0:k]: the indices of the k largest values,
 * unsorted, ties at the k-th value going to the lower column; when fewer than k
 * columns are in the window all of them are written followed by -1 padding.
 * Output is bit-identical from run to run. */
int dsa_topk_select(const float* logits, int64_t ld_logits, const int32_t* ks, const int32_t* ke, int T, int S,
                    int k, int32_t* out_idx, void* stream);

/* Indexer logits + top-k in one call (the whole of IndexerSimulator.logits_step,
 * sparse_attn/DSA.py:336-362).  `workspace` holds the fp32 logits of one chunk
 * of query rows; dsa_indexer_topk_workspace_bytes gives the size that does the
 * whole call in one chunk, smaller workspaces (>= one 256-row chunk) make it
 * loop. */
size_t dsa_indexer_topk_workspace_bytes(int T, int S);
int dsa_indexer_topk(const void* q_fp8, const void* k_fp8, const float* k_scale, const void* w, int w_dtype,
                     const int32_t* ks, const int32_t* ke, int T, int S, int H, int D, int k, int32_t* out_idx,
                     void* workspace, size_t workspace_bytes, int32_t* status, void* stream);

/* Token-sparse MLA attention, prefill (MQA over the shared latent KV):
 *   out[t,h,:] = sum_j softmax_j(scale * q[t,h,:576] . kv[idx[t,j],:576]) * kv[idx[t,j],:512]
 * over the slots with idx[t,j] >= 0; a row without any valid slot gives zeros.
 * Takes the place of the block-sparse attention stand-in reached through
 * register_sparse_fa().run (sparse_attn/DSA.py:208-249); the reference has no
 * sparse-MLA kernel of its own.
 *   q_bf16 [T, H, 576] bf16; kv_bf16 [S_kv, 576] bf16; idx [T, K] int32 positions
 *   into kv (negative = empty; >= S_kv is skipped and sets status 2);
 *   out_bf16 [T, H, 512] bf16.  All contiguous and 16-byte aligned.  K <= 2048; scale > 0.  Any H >= 1
 *   (heads are processed in groups of 128). */
int dsa_sparse_mla_prefill(const void* q_bf16, const void* kv_bf16, const int32_t* idx, void* out_bf16, int T, int H,
                           int S_kv, int K, float scale, int32_t* status, void* stream);

/* Block-sparse multi-head attention, the call behind register_sparse_fa().run
 * (sparse_attn/DSA.py:232-247: triton_block_sparse_attn_fwd_openai_prefetch(q, k, v, idx, num,
 * sm_scale) -> (out, _), whose source is not part of the reference).  Non-causal; 64-token blocks:
 *   out[b,s,h,:] = softmax_j(scale * q[b,s,h,:] . k[b,j,h,:]) v[b,j,h,:],  j over the key blocks
 *   lut[b,h,s/64,0..num[b,h,s/64]) of query block s/64.
 *   q, k, v, out [B, S, H, 128] bf16, contiguous, 16-byte aligned; S a multiple of 64;
 *   lut [B, H, S/64, topk] int32 key-block ids (an id outside [0, S/64) contributes nothing and
 *   sets status 2); num [B, H, S/64] int32, clamped to [0, topk]; scale > 0. */
int dsa_block_sparse_mha(const void* q_bf16, const void* k_bf16, const void* v_bf16, const int32_t* lut,
                         const int32_t* num, void* out_bf16, int B, int S, int H, int D, int topk, float scale,
                         int32_t* status, void* stream);

/* The same attention for decode over the paged FP8 latent cache (no counterpart
 * in the reference, which has no cache: sparse_attn/DSA.py:475-477).  One query
 * token per sequence; idx[b, j] is a logical position of sequence b, stored at
 * cache row block_table[b, pos/64]*64 + pos%64.  A cache row is 656 bytes:
 * 512 e4m3 latent values, 4 fp32 scales (one per 128 values), 64 bf16 rope
 * values; latent = e4m3 * scale is rounded to bf16 before the tensor-core math.
 *   q_bf16 [B, H, 576]; cache [num_pages*64, 656] bytes; block_table
 *   [B, table_stride] int32; idx [B, K] int32 (K <= 2048); out_bf16 [B, H, 512].
 * With few sequences the slot list of each is cut into parts that run on
 * different SMs and are merged by a second kernel; that needs `workspace` of
 * dsa_sparse_mla_decode_workspace_bytes(B, H, K) bytes (16-byte aligned).  With
 * workspace NULL or too small the call still works, one part per sequence. */
size_t dsa_sparse_mla_decode_workspace_bytes(int B, int H, int K);
int dsa_sparse_mla_decode_paged(const void* q_bf16, const void* cache, const int32_t* block_table,
                                int64_t table_stride, const int32_t* idx, void* out_bf16, int B, int H, int K,
                                int num_pages, int max_ctx, float scale, void* workspace, size_t workspace_bytes,
                                int32_t* status, void* stream);

/* dsa_indexer_topk without a caller-supplied workspace.  No counterpart in the
 * reference: it exists for hosts that cannot allocate device memory at the call
 * site (a runtime that owns the whole device heap and forbids allocation inside
 * its operator callbacks, a serving loop whose pool is frozen once it starts).
 * Same inputs, outputs and results as dsa_indexer_topk; the fp32 logits scratch
 * is a 64 MiB array built into the library, which every GPU that loads the
 * library keeps until the process exits.  Limits and rules:
 *   - min(T, 256) * round_up(S, 4) * 4 bytes must fit in 64 MiB (S <= 65536 when
 *     T >= 256); larger problems are refused with DSA_ERR_WORKSPACE.
 *   - The first call on each device looks up the array's device address, and
 *     that lookup is when the driver materialises the 64 MiB on that device (CUDA
 *     loads modules lazily): it can fail with DSA_ERR_CUDA "out of memory" on a
 *     GPU that is already full.  Make one warm-up call with T = 0 per device at
 *     start-up -- before the host freezes its pool and outside any stream
 *     capture; it launches nothing.
 *   - All calls on one device share the array, which keeps whatever the last
 *     call left there (every call overwrites what it reads).  Two calls whose
 *     kernels overlap on the GPU (different streams) race: serialise them.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine; after
 *     the warm-up call no device memory changes hands at all. */
size_t dsa_indexer_topk_static_max_bytes(void);
int dsa_indexer_topk_static(const void* q_fp8, const void* k_fp8, const float* k_scale, const void* w, int w_dtype,
                            const int32_t* ks, const int32_t* ke, int T, int S, int H, int D, int k,
                            int32_t* out_idx, int32_t* status, void* stream);

/* ---- test hooks ---------------------------------------------------------------
 * No counterpart in the reference.  They exist so that the parity tests can reach,
 * through this ABI, code paths that the normal entry points choose by themselves.
 *
 * dsa_test_indexer_logits_general: dsa_indexer_logits with 64 heads x 128 kept on
 *   the general kernel (the normal call takes the register-weight kernel for that
 *   shape); the two must agree bit for bit.
 * dsa_test_topk_select_two_pass: dsa_topk_select with every row on the two-pass
 *   radix path (the normal call takes the sampled single pass for long rows and
 *   falls back to this path when the sample misleads it); same sets, same order.
 * dsa_test_bounded_wait: launches one thread that waits, with the wait helper all
 *   pipeline roles use, on a barrier nobody arrives at; after poll_limit
 *   (1..65536) polls it must give up and write status 1 to *status. */
int dsa_test_indexer_logits_general(const void* q_fp8, const void* k_fp8, const float* k_scale, const void* w,
                                    int w_dtype, const int32_t* ks, const int32_t* ke, float* logits,
                                    int64_t ld_logits, int T, int S, int H, int D, int clean, int32_t* status,
                                    void* stream);
int dsa_test_topk_select_two_pass(const float* logits, int64_t ld_logits, const int32_t* ks, const int32_t* ke, int T,
                                  int S, int k, int32_t* out_idx, void* stream);
int dsa_test_bounded_wait(int poll_limit, int32_t* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* DSA_B200_H_ */
