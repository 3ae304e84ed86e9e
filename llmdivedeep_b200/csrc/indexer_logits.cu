// Lightning-indexer logits on sm_100a:
//   logits[t, s] = k_scale[s] * sum_h w[t, h] * relu(q[t, h, :] . k[s, :]),   ks[t] <= s < ke[t]
// Replaces the external call deep_gemm.fp8_mqa_logits(q_fp8, (k_fp8, k_scale), w, ks, ke)
// made at sparse_attn/DSA.py:343-345, 547-552 and 654-659 of the reference.
//
// One persistent CTA per SM.  A tile is 128 keys (the MMA M dimension, one TMEM
// lane per key) by N = NQ*H (token, head) pairs (the MMA N dimension, one TMEM
// column per pair).  FP8 e4m3 operands are fetched by TMA with the 128-byte (or
// 64-byte) swizzle the UMMA descriptors expect, tcgen05.mma accumulates in fp32
// in tensor memory, and two epilogue warpgroups drain alternate accumulator
// stages: every thread owns one key, walks the columns of its lane, applies
// ReLU, multiplies by the head weight (broadcast from shared memory) and sums
// the H heads of each token -- a purely thread-local reduction.  The sum order
// is fixed (even heads ascending, odd heads ascending, then even + odd), so
// results are bit-identical from run to run.
//
// Roles: warp 0 lane 0 = TMA producer, warp 1 lane 0 = MMA issuer (warp 1 owns
// the TMEM allocation), warps 4-7 and 8-11 = epilogue warpgroups 0 and 1.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <math_constants.h>

#include "dsa_common.cuh"
#include "dsa_host.h"

namespace dsa {

constexpr int kIdxThreads = 384;
constexpr int kTileKeys = 128;
constexpr int kChunkTiles = 64;        // key tiles per work unit
constexpr int kPageTokens = 64;

struct IndexerArgs {
  const float* k_scale;      // [S] (contiguous) or [num_pages*64] (paged), one per key
  const void* w;             // [T, H] fp32 or bf16
  const int32_t* ks;         // [T] or null (0)
  const int32_t* ke;         // [T]; paged: ctx_len [B]
  const int32_t* block_table;  // paged only: [B, table_stride]
  float* logits;             // [T, ld]
  int64_t ld;
  int64_t table_stride;
  int T;                     // query tokens (paged: sequences)
  int S;                     // keys (paged: max logical positions = pages_per_seq*64)
  int num_phys_rows;         // paged: rows of the cache
  int w_is_bf16;
  int* status;
};

template <int H, int D, int NQ, bool PAGED>
struct IdxCfg {
  static constexpr int N = H * NQ;
  static constexpr int KSTEPS = D / 32;
  static constexpr int K_TILE_BYTES = kTileKeys * D;
  static constexpr int Q_TILE_BYTES = N * D;
  static constexpr int STAGES = 6;
  static constexpr int TMEM_COLS = (2 * N < 32) ? 32 : 2 * N;
  static constexpr uint64_t SWZ = (D == 128) ? kSwz128 : kSwz64;
  static constexpr uint32_t SBO = 8 * D;                 // 8 rows of D bytes
  static constexpr int SMEM_BYTES = 1024 /*align slack*/ + STAGES * K_TILE_BYTES + 2 * Q_TILE_BYTES +
                                    8 * N * 4 + 16 * NQ * 4 + 256;
  static_assert(N % 16 == 0 && N >= 16 && N <= 256, "MMA N out of range");
  static_assert(D == 64 || D == 128, "head dim must be 64 or 128");
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM columns must be a power of two");
};

// [min ks, max ke) over the tokens of group g, computed by one full warp.
template <int NQ, bool PAGED>
__device__ __forceinline__ void group_window(const IndexerArgs& a, int g, int& lo, int& hi) {
  const int lane = threadIdx.x & 31;
  int mn = 0x7fffffff, mx = 0;
  for (int j = lane; j < NQ; j += 32) {
    const int t = g * NQ + j;
    if (t < a.T) {
      const int s0 = (!PAGED && a.ks) ? a.ks[t] : 0;
      const int s1 = a.ke[t];
      mn = min(mn, max(s0, 0));
      mx = max(mx, min(s1, a.S));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mn = min(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  lo = mn;
  hi = mx;
}

// key-tile range of work unit u (same answer in every role)
template <int NQ, bool PAGED>
__device__ __forceinline__ bool unit_tiles(const IndexerArgs& a, int u, int n_groups, int& g, int& t_lo,
                                           int& t_hi) {
  const int c = u / n_groups;
  g = u - c * n_groups;
  int lo, hi;
  group_window<NQ, PAGED>(a, g, lo, hi);
  if (hi <= lo) return false;
  t_lo = max(c * kChunkTiles, lo / kTileKeys);
  t_hi = min((c + 1) * kChunkTiles, (hi + kTileKeys - 1) / kTileKeys);
  return t_lo < t_hi;
}

template <int H, int D, int NQ, bool PAGED>
__global__ void __launch_bounds__(kIdxThreads, 1)
indexer_logits_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const IndexerArgs a, const int n_groups, const int n_units) {
  using C = IdxCfg<H, D, NQ, PAGED>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_s = smem;                                        // STAGES x [128 keys x D]
  uint8_t* q_s = k_s + C::STAGES * C::K_TILE_BYTES;           // 2 x [N rows x D]
  float* w_s = reinterpret_cast<float*>(q_s + 2 * C::Q_TILE_BYTES);   // 8 warps x N (private copies)
  int* win_s = reinterpret_cast<int*>(w_s + 8 * C::N);        // 8 warps x (ks[NQ], ke[NQ])
  uint64_t* bars = reinterpret_cast<uint64_t*>(win_s + 16 * NQ);
  uint64_t* k_full = bars;                  // [STAGES]
  uint64_t* k_empty = k_full + C::STAGES;   // [STAGES]
  uint64_t* q_full = k_empty + C::STAGES;   // [2]
  uint64_t* q_empty = q_full + 2;           // [2]
  uint64_t* acc_full = q_empty + 2;         // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < C::STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 4);       // one arrive per epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    uint32_t it = 0, nu = 0;
    for (int u = blockIdx.x; u < n_units && !*abort_flag; u += gridDim.x) {
      int g, t_lo, t_hi;
      if (!unit_tiles<NQ, PAGED>(a, u, n_groups, g, t_lo, t_hi)) continue;
      const int qs = nu & 1;
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait(&q_empty[qs], ((nu >> 1) & 1) ^ 1, abort_flag, a.status);
        if (ok) {
          mbar_expect_tx(&q_full[qs], C::Q_TILE_BYTES);
          tma_load_2d(q_s + qs * C::Q_TILE_BYTES, &tmap_q, 0, g * C::N, &q_full[qs]);
        }
      }
      ++nu;
      for (int kt = t_lo; kt < t_hi && ok; ++kt, ++it) {
        if (lane != 0) continue;
        const int st = it % C::STAGES;
        ok = mbar_wait(&k_empty[st], ((it / C::STAGES) & 1) ^ 1, abort_flag, a.status);
        if (!ok) break;
        uint8_t* dst = k_s + st * C::K_TILE_BYTES;
        if constexpr (!PAGED) {
          mbar_expect_tx(&k_full[st], C::K_TILE_BYTES);
          tma_load_2d(dst, &tmap_k, 0, kt * kTileKeys, &k_full[st]);
        } else {
          // two 64-token pages per tile; a missing or out-of-range page is skipped
          const int n_pages = (min(a.ke[g], a.S) + kPageTokens - 1) / kPageTokens;
          int rows[2];
          uint32_t bytes = 0;
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            const int page = kt * 2 + p;
            rows[p] = -1;
            if (page < n_pages) {
              const int phys = a.block_table[(int64_t)g * a.table_stride + page];
              if (phys >= 0 && (int64_t)(phys + 1) * kPageTokens <= a.num_phys_rows) {
                rows[p] = phys * kPageTokens;
                bytes += C::K_TILE_BYTES / 2;
              } else if (a.status) {
                atomicCAS(a.status, kStatusOk, kStatusBadIndex);
              }
            }
          }
          if (bytes) {
            mbar_expect_tx(&k_full[st], bytes);
#pragma unroll
            for (int p = 0; p < 2; ++p)
              if (rows[p] >= 0) tma_load_2d(dst + p * (C::K_TILE_BYTES / 2), &tmap_k, 0, rows[p], &k_full[st]);
          } else {
            mbar_arrive(&k_full[st]);
          }
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      it = __shfl_sync(0xffffffffu, it, 0);
      if (!ok) break;
    }
    // on abort, give copies already in flight a bounded chance to land
    if (lane == 0 && *abort_flag) {
      for (int st = 0; st < C::STAGES; ++st)
        for (uint32_t spin = 0; spin < (1u << 16) && !mbar_try_wait(&k_full[st], 0) &&
                                !mbar_try_wait(&k_full[st], 1); ++spin) {
        }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    constexpr uint32_t idesc = umma_idesc(0, 0, 0, 0, kTileKeys, C::N);
    uint32_t it = 0, nu = 0;
    for (int u = blockIdx.x; u < n_units && !*abort_flag; u += gridDim.x) {
      int g, t_lo, t_hi;
      if (!unit_tiles<NQ, PAGED>(a, u, n_groups, g, t_lo, t_hi)) continue;
      const int qs = nu & 1;
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait(&q_full[qs], (nu >> 1) & 1, abort_flag, a.status);
        const uint64_t qdesc = umma_smem_desc(smem_u32(q_s + qs * C::Q_TILE_BYTES), 16, C::SBO, C::SWZ);
        for (int kt = t_lo; kt < t_hi && ok; ++kt, ++it) {
          const int st = it % C::STAGES;
          const int acc = it & 1;
          ok = mbar_wait(&k_full[st], (it / C::STAGES) & 1, abort_flag, a.status) &&
               mbar_wait(&acc_empty[acc], ((it >> 1) & 1) ^ 1, abort_flag, a.status);
          if (!ok) break;
          tc_fence_after();
          const uint64_t kdesc = umma_smem_desc(smem_u32(k_s + st * C::K_TILE_BYTES), 16, C::SBO, C::SWZ);
#pragma unroll
          for (int k = 0; k < C::KSTEPS; ++k)
            umma_f8(tmem_base + acc * C::N, kdesc + (k * 32 >> 4), qdesc + (k * 32 >> 4), idesc, k > 0);
          umma_commit(&k_empty[st]);
          umma_commit(&acc_full[acc]);
        }
        if (ok) umma_commit(&q_empty[qs]);
      }
      ++nu;
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      it = __shfl_sync(0xffffffffu, it, 0);
      if (!ok) break;
    }
  } else if (warp >= 4) {
    // --------------------------- epilogue warpgroups ---------------------------
    const int wg = (warp - 4) >> 2;              // 0 or 1 = accumulator stage it drains
    const int wq = warp & 3;                     // TMEM lane quadrant of this warp
    const int row = wq * 32 + lane;              // key within the tile = TMEM lane
    float* my_w = w_s + (warp - 4) * C::N;       // each warp stages its own copy: no cross-warp sync
    int* my_ks = win_s + (warp - 4) * 2 * NQ;
    int* my_ke = my_ks + NQ;
    const uint32_t t_row = tmem_base + (uint32_t(wq * 32) << 16) + wg * C::N;
    uint32_t it = 0, n_mine = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
      int g, t_lo, t_hi;
      if (!unit_tiles<NQ, PAGED>(a, u, n_groups, g, t_lo, t_hi)) continue;
      bool staged = false;
      for (int kt = t_lo; kt < t_hi; ++kt, ++it) {
        if (int(it & 1) != wg) continue;
        if (!staged) {
          // stage this group's head weights and windows for the warp
          __syncwarp();
          for (int c = lane; c < C::N; c += 32) {
            const int t = g * NQ + c / H;
            float wv = 0.f;
            if (t < a.T) {
              const int64_t off = (int64_t)t * H + (c % H);
              wv = a.w_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.w)[off])
                               : reinterpret_cast<const float*>(a.w)[off];
            }
            my_w[c] = wv;
          }
          for (int j = lane; j < NQ; j += 32) {
            const int t = g * NQ + j;
            int s0 = 0, s1 = 0;
            if (t < a.T) {
              s0 = (!PAGED && a.ks) ? a.ks[t] : 0;
              s1 = min(a.ke[t], a.S);
            }
            my_ks[j] = s0;
            my_ke[j] = s1;
          }
          __syncwarp();
          staged = true;
        }
        const int s = kt * kTileKeys + row;      // logical key position
        float kscale = 0.f;
        if constexpr (!PAGED) {
          if (s < a.S) kscale = a.k_scale[s];
        } else {
          if (s < my_ke[0]) {
            const int phys = a.block_table[(int64_t)g * a.table_stride + s / kPageTokens];
            if (phys >= 0 && (int64_t)(phys + 1) * kPageTokens <= a.num_phys_rows)
              kscale = a.k_scale[(int64_t)phys * kPageTokens + (s % kPageTokens)];
          }
        }
        ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[wg], n_mine & 1, abort_flag, a.status));
        if (!ok) break;
        tc_fence_after();

        constexpr int CH = 32;                   // columns per TMEM load
        uint32_t v[2][CH];
        tmem_ld32(t_row, v[0]);
        uint64_t acc2 = 0;                       // (even heads, odd heads) running sums
#pragma unroll
        for (int c = 0; c < C::N; c += CH) {
          const int cur = (c / CH) & 1;
          tmem_wait_ld();
          if (c + CH < C::N) tmem_ld32(t_row + c + CH, v[cur ^ 1]);
#pragma unroll
          for (int i = 0; i < CH; i += 2) {
            const int col = c + i;
            if (col % H == 0) acc2 = 0;
            const float d0 = fmaxf(__uint_as_float(v[cur][i]), 0.f);
            const float d1 = fmaxf(__uint_as_float(v[cur][i + 1]), 0.f);
            const uint64_t wp = *reinterpret_cast<const uint64_t*>(my_w + col);
            acc2 = fma_f32x2(pack_f32x2(d0, d1), wp, acc2);
            if ((col + 2) % H == 0) {
              const int j = col / H;
              const int t = g * NQ + j;
              float e, o;
              unpack_f32x2(acc2, e, o);
              const float score = (e + o) * kscale;
              if (t < a.T && s < a.S) {
                const bool in = (s >= my_ks[j]) && (s < my_ke[j]);
                a.logits[(int64_t)t * a.ld + s] = in ? score : -CUDART_INF_F;
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[wg]);
        ++n_mine;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// -inf outside the tiles the main kernel wrote (the "clean logits" contract of the
// call being replaced): columns below the group's first tile and above its last.
template <int NQ>
__global__ void fill_masked_kernel(const IndexerArgs a, int n_groups) {
  const int t = blockIdx.x;
  if (t >= a.T) return;
  const int g = t / NQ;
  __shared__ int s_lo, s_hi;
  if (threadIdx.x < 32) {
    int lo, hi;
    group_window<NQ, false>(a, g, lo, hi);
    if (threadIdx.x == 0) {
      if (hi <= lo) { lo = 0; hi = 0; }
      s_lo = (lo / kTileKeys) * kTileKeys;
      s_hi = min(a.S, ((hi + kTileKeys - 1) / kTileKeys) * kTileKeys);
    }
  }
  __syncthreads();
  float* row = a.logits + (int64_t)t * a.ld;
  for (int s = threadIdx.x; s < s_lo; s += blockDim.x) row[s] = -CUDART_INF_F;
  for (int s = s_hi + threadIdx.x; s < a.S; s += blockDim.x) row[s] = -CUDART_INF_F;
}

// ------------------------------- host side ----------------------------------
static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

// 2-D byte tensor [rows, row_bytes] with a [box_rows, row_bytes] box, swizzled by row_bytes.
int make_tmap_2d_u8(CUtensorMap* m, const void* base, uint64_t rows, uint32_t row_bytes, uint64_t row_pitch,
                    uint32_t box_rows) {
  auto fn = encode_fn();
  if (!fn) return set_error(DSA_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  cuuint64_t dims[2] = {row_bytes, rows};
  cuuint64_t strides[1] = {row_pitch};
  cuuint32_t box[2] = {row_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapSwizzle sw = row_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                        : row_bytes == 64  ? CU_TENSOR_MAP_SWIZZLE_64B
                                           : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(DSA_ERR_CUDA, "cuTensorMapEncodeTiled failed (code %d)", (int)r);
  return DSA_OK;
}

template <int H, int D, int NQ, bool PAGED>
static int launch_indexer(const void* q, const void* k, const IndexerArgs& a, int clean, cudaStream_t stream) {
  using C = IdxCfg<H, D, NQ, PAGED>;
  if (a.T == 0 || a.S == 0) return DSA_OK;
  CUtensorMap tq, tk;
  int rc = make_tmap_2d_u8(&tq, q, (uint64_t)a.T * H, D, D, C::N);
  if (rc) return rc;
  rc = PAGED ? make_tmap_2d_u8(&tk, k, (uint64_t)a.num_phys_rows, D, D, kPageTokens)
             : make_tmap_2d_u8(&tk, k, (uint64_t)a.S, D, D, kTileKeys);
  if (rc) return rc;
  const int n_groups = (a.T + NQ - 1) / NQ;
  const int n_tiles = (a.S + kTileKeys - 1) / kTileKeys;
  const int n_chunks = (n_tiles + kChunkTiles - 1) / kChunkTiles;
  const int64_t n_units64 = (int64_t)n_groups * n_chunks;
  if (n_units64 > 0x7fffffff) return set_error(DSA_ERR_SHAPE, "indexer: too many work units");
  const int n_units = (int)n_units64;
  auto kern = indexer_logits_kernel<H, D, NQ, PAGED>;
  static bool attr_done = false;
  if (!attr_done) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
      return set_error(DSA_ERR_CUDA, "indexer: cannot raise dynamic shared memory to %d", C::SMEM_BYTES);
    attr_done = true;
  }
  const int grid = n_units < sm_count() ? n_units : sm_count();
  kern<<<grid, kIdxThreads, C::SMEM_BYTES, stream>>>(tq, tk, a, n_groups, n_units);
  if constexpr (!PAGED) {
    if (clean) fill_masked_kernel<NQ><<<a.T, 256, 0, stream>>>(a, n_groups);
  }
  return check_launch("indexer_logits");
}

int indexer_logits_dispatch(const void* q, const void* k, const IndexerArgs& a, int H, int D, int clean,
                            cudaStream_t stream) {
#define DSA_IDX_CASE(h, d)                                                    \
  if (H == h && D == d) return launch_indexer<h, d, 256 / h, false>(q, k, a, clean, stream);
  DSA_IDX_CASE(64, 128)
  DSA_IDX_CASE(32, 128)
  DSA_IDX_CASE(16, 128)
  DSA_IDX_CASE(8, 128)
  DSA_IDX_CASE(4, 128)
  DSA_IDX_CASE(64, 64)
  DSA_IDX_CASE(4, 64)
#undef DSA_IDX_CASE
  return set_error(DSA_ERR_SHAPE, "indexer: unsupported (heads=%d, head_dim=%d); heads in {4,8,16,32,64}, dim in {64,128}",
                   H, D);
}

int indexer_logits_paged_dispatch(const void* q, const void* kcache, const IndexerArgs& a, int H, int D,
                                  cudaStream_t stream) {
  if (H == 64 && D == 128) return launch_indexer<64, 128, 1, true>(q, kcache, a, 0, stream);
  if (H == 32 && D == 128) return launch_indexer<32, 128, 1, true>(q, kcache, a, 0, stream);
  if (H == 16 && D == 128) return launch_indexer<16, 128, 1, true>(q, kcache, a, 0, stream);
  return set_error(DSA_ERR_SHAPE, "paged indexer: unsupported (heads=%d, head_dim=%d)", H, D);
}

int indexer_logits_contiguous(const void* q, const void* k, const float* k_scale, const void* w, int w_dtype,
                              const int32_t* ks, const int32_t* ke, float* logits, int64_t ld, int T, int S,
                              int H, int D, int clean, int32_t* status, cudaStream_t stream) {
  IndexerArgs a{};
  a.k_scale = k_scale;
  a.w = w;
  a.ks = ks;
  a.ke = ke;
  a.block_table = nullptr;
  a.logits = logits;
  a.ld = ld;
  a.table_stride = 0;
  a.T = T;
  a.S = S;
  a.num_phys_rows = S;
  a.w_is_bf16 = (w_dtype == DSA_W_BF16);
  a.status = status;
  return indexer_logits_dispatch(q, k, a, H, D, clean, stream);
}

int indexer_logits_paged(const void* q, const void* w, int w_dtype, const void* kcache, const float* kscale,
                         const int32_t* block_table, int64_t table_stride, const int32_t* ctx_len, float* logits,
                         int64_t ld, int B, int H, int D, int num_pages, int max_ctx, int32_t* status,
                         cudaStream_t stream) {
  IndexerArgs a{};
  a.k_scale = kscale;
  a.w = w;
  a.ks = nullptr;
  a.ke = ctx_len;
  a.block_table = block_table;
  a.logits = logits;
  a.ld = ld;
  a.table_stride = table_stride;
  a.T = B;
  a.S = max_ctx;
  a.num_phys_rows = num_pages * kPageTokens;
  a.w_is_bf16 = (w_dtype == DSA_W_BF16);
  a.status = status;
  return indexer_logits_paged_dispatch(q, kcache, a, H, D, stream);
}

}  // namespace dsa
