// Lightning-indexer logits on sm_100a:
//   logits[t, s] = k_scale[s] * sum_h w[t, h] * relu(q[t, h, :] . k[s, :]),   ks[t] <= s < ke[t]
// Replaces the external call deep_gemm.fp8_mqa_logits(q_fp8, (k_fp8, k_scale), w, ks, ke)
// made at sparse_attn/DSA.py:343-345, 547-552 and 654-659 of the reference.
//
// One persistent CTA per SM.  A tile is 128 keys (the MMA M dimension, one TMEM
// lane per key) by N = NQ*H (token, head) pairs (the MMA N dimension, one TMEM
// column per pair).  FP8 e4m3 operands are fetched by TMA with the 128-byte (or
// 64-byte) swizzle the UMMA descriptors expect and tcgen05.mma accumulates in
// fp32 in tensor memory.  A work unit is a block of QB query groups against a
// chunk of 64 key tiles: every key tile fetched from L2 is multiplied with all
// QB resident query tiles, which divides the L2 -> shared-memory key traffic by
// QB (at QB = 1 that traffic, not the tensor pipe, bounds the kernel).
//
// Epilogue warpgroups drain alternate accumulator stages: every thread owns one
// key, walks the columns of its lane, applies ReLU, multiplies by the head
// weight (broadcast from shared memory) and sums the H heads of each token -- a
// purely thread-local reduction with a fixed order (head pair p of a token goes
// to chain p mod 2, score = (chain0.even + chain0.odd) + (chain1.even +
// chain1.odd)), so results are bit-identical from run to run.
//
// Roles: warp 0 = TMA producer, warp 1 = MMA issuer (owns the TMEM allocation),
// warp 2 = stages head weights and windows of the next unit, warps 4.. =
// epilogue.  All waits are bounded (see dsa_common.cuh).
#include <cuda.h>
#include <cudaTypedefs.h>
#include <math_constants.h>
#include <stdlib.h>

#include "dsa_common.cuh"
#include "dsa_host.h"

namespace dsa {

constexpr int kTileKeys = 128;         // keys per MMA (M); a paged work tile is two of these, see tile_keys()
constexpr int kChunkTiles = 64;        // most key tiles per work unit (launches with few units use fewer)
constexpr int kPageTokens = 64;
// Keys per pipeline tile.  The paged (decode) form has one query token per sequence, so a 128-key tile is little
// work (64 accumulator columns) against the fixed cost of its barrier hand-offs: it moves 256 keys (four pages)
// per tile, as two M=128 MMAs into adjacent accumulator columns.
template <bool PAGED>
__host__ __device__ constexpr int tile_keys() { return PAGED ? 4 * kTileKeys : kTileKeys; }

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
  int chunk_tiles;           // key tiles per work unit, <= kChunkTiles (set by the launcher)
  int* status;
};

// 4-byte asynchronous global -> shared copy (zero fill when !valid; src is then not read).  Unlike a load
// into a register it leaves no scoreboard entry, so a prefetch several tiles ahead never stalls a later move.
__device__ __forceinline__ void cp_async_f32(float* dst, const float* src, bool valid) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(valid ? 4 : 0)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int H, int D, int NQ, bool PAGED, int QB, int EPI>
struct IdxCfg {
  static constexpr int N = H * NQ;                       // accumulator columns = (token, head) pairs
  static constexpr int NTOK = NQ * QB;                   // query tokens per work unit
  static constexpr int KSTEPS = D / 32;
  static constexpr int TILE_KEYS = tile_keys<PAGED>();
  static constexpr int SUB = TILE_KEYS / kTileKeys;      // M=128 MMAs per tile
  static constexpr int PAGES = TILE_KEYS / kPageTokens;  // cache pages per tile (paged)
  static constexpr int ACC_COLS = N * SUB;               // accumulator columns per stage
  static constexpr int K_TILE_BYTES = TILE_KEYS * D;
  static constexpr int Q_TILE_BYTES = N * D;
  static constexpr int STAGES = PAGED ? 3 : 4;           // key tiles in flight (paged: 3 x 64 KB)
  static constexpr int TMEM_COLS = (2 * ACC_COLS < 32) ? 32 : 2 * ACC_COLS;
  static constexpr uint64_t SWZ = (D == 128) ? kSwz128 : kSwz64;
  static constexpr uint32_t SBO = 8 * D;                 // 8 rows of D bytes
  static constexpr int EPI_WARPS = EPI * 4;
  static constexpr int THREADS = 128 + EPI * 128;
  static constexpr int SPLIT = EPI / 2;                  // warpgroups sharing one accumulator stage
  static constexpr int COLS_PER_WG = N / SPLIT;
  static constexpr int CH = 16;                          // columns per TMEM load
  static constexpr int AHEAD = 2;                        // key tiles by which the k_scale prefetch runs ahead
  static constexpr int SMEM_BYTES = 1024 /*align slack*/ + STAGES * K_TILE_BYTES + 2 * QB * Q_TILE_BYTES +
                                    2 * QB * N * 4 + 2 * NTOK * 8 + 256 + (PAGED ? 4 * PAGES * kChunkTiles * 4 : 0) +
                                    AHEAD * SUB * EPI * 128 * 4;
  static_assert(EPI == 2 || EPI == 4, "two or four epilogue warpgroups");
  static_assert(N % 16 == 0 && N >= 16 && N <= 256, "MMA N out of range");
  static_assert(COLS_PER_WG % H == 0 && COLS_PER_WG % CH == 0, "a warpgroup must own whole tokens");
  static_assert(D == 64 || D == 128, "head dim must be 64 or 128");
  static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0, "TMEM columns must be a power of two");
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

// [min ks, max ke) over tokens [t0, t0 + ntok), computed by one full warp.
template <bool PAGED>
__device__ __forceinline__ void token_window(const IndexerArgs& a, int t0, int ntok, int& lo, int& hi) {
  const int lane = threadIdx.x & 31;
  int mn = 0x7fffffff, mx = 0;
  for (int j = lane; j < ntok; j += 32) {
    const int t = t0 + j;
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

// Work unit u -> query block qb, key-tile range [t_lo, t_hi), groups in the block nb.
// Called by a full warp; every role gets the same answer.
template <int NQ, int QB, bool PAGED>
__device__ __forceinline__ bool unit_tiles(const IndexerArgs& a, int u, int n_qblocks, int n_groups, int& qb,
                                           int& nb, int& t_lo, int& t_hi) {
  const int c = u / n_qblocks;
  qb = u - c * n_qblocks;
  nb = min(QB, n_groups - qb * QB);
  int lo, hi;
  token_window<PAGED>(a, qb * QB * NQ, nb * NQ, lo, hi);
  if (hi <= lo) return false;
  constexpr int TK = tile_keys<PAGED>();
  t_lo = max(c * a.chunk_tiles, lo / TK);
  t_hi = min((c + 1) * a.chunk_tiles, (hi + TK - 1) / TK);
  return t_lo < t_hi;
}

// One thread = one key.  Walks NCOLS accumulator columns starting at column COL0 of
// its TMEM lane.  Weights of chunk c+1 and its TMEM load are both requested before
// the math of chunk c, in that order: shared-memory loads queue behind a TMEM load
// issued earlier by the same warp, so the weights must go first to overlap.
template <int H, int NQ, int CH, int COL0, int NCOLS>
__device__ __forceinline__ void drain_columns(uint32_t t_lane, const float* __restrict__ w_s,
                                              const int2* __restrict__ win_s, float kscale, int s, bool s_ok,
                                              int n_tok, float* __restrict__ grp_base, uint32_t ld) {
  constexpr int NCH = 2;
  uint32_t v[2][CH];
  float4 wv[2][CH / 4];
  uint64_t chain[NCH];
#pragma unroll
  for (int i = 0; i < CH / 4; ++i) wv[0][i] = *reinterpret_cast<const float4*>(w_s + COL0 + 4 * i);
  tmem_ld16(t_lane + COL0, v[0]);
#pragma unroll
  for (int c = 0; c < NCOLS; c += CH) {
    const int cur = (c / CH) & 1;
    tmem_wait_ld();
    if (c + CH < NCOLS) {
#pragma unroll
      for (int i = 0; i < CH / 4; ++i)
        wv[cur ^ 1][i] = *reinterpret_cast<const float4*>(w_s + COL0 + c + CH + 4 * i);
      tmem_ld16(t_lane + COL0 + c + CH, v[cur ^ 1]);
    }
#pragma unroll
    for (int i = 0; i < CH; i += 4) {
      const int col = COL0 + c + i;                       // multiple of 4
      const float4 w4 = wv[cur][i / 4];
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        const int cp = col + 2 * p;                       // first column of this pair
        const int hp = (cp % H) / 2;                      // pair index inside the token
        const float d0 = fmaxf(__uint_as_float(v[cur][i + 2 * p]), 0.f);
        const float d1 = fmaxf(__uint_as_float(v[cur][i + 2 * p + 1]), 0.f);
        const uint64_t wp = p == 0 ? pack_f32x2(w4.x, w4.y) : pack_f32x2(w4.z, w4.w);
        if (hp < NCH) chain[hp % NCH] = 0;                // first use of the chain in this token
        chain[hp % NCH] = fma_f32x2(pack_f32x2(d0, d1), wp, chain[hp % NCH]);
        if (cp % H == H - 2) {                            // last pair of the token
          float score = 0.f;
#pragma unroll
          for (int q = 0; q < NCH; ++q) {
            float e, o;
            unpack_f32x2(chain[q], e, o);
            score += e + o;
          }
          const int j = cp / H;                           // token within the group
          const int2 win = win_s[j];                      // (ks, ke - ks)
          const bool in = static_cast<uint32_t>(s - win.x) < static_cast<uint32_t>(win.y);
          if (s_ok && j < n_tok) grp_base[static_cast<uint32_t>(j) * ld + static_cast<uint32_t>(s)] =
              in ? score * kscale : -CUDART_INF_F;
        }
      }
    }
  }
}

template <int H, int D, int NQ, bool PAGED, int QB, int EPI>
__global__ void __launch_bounds__(IdxCfg<H, D, NQ, PAGED, QB, EPI>::THREADS, 1)
indexer_logits_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                      const IndexerArgs a, const int n_groups, const int n_qblocks, const int n_units) {
  using C = IdxCfg<H, D, NQ, PAGED, QB, EPI>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_s = smem;                                        // STAGES x [128 keys x D]
  uint8_t* q_s = k_s + C::STAGES * C::K_TILE_BYTES;           // 2 x QB x [N rows x D]
  float* w_s = reinterpret_cast<float*>(q_s + 2 * QB * C::Q_TILE_BYTES);   // 2 x QB x N head weights
  int2* win_s = reinterpret_cast<int2*>(w_s + 2 * QB * C::N);              // 2 x NTOK (ks, ke - ks)
  uint64_t* bars = reinterpret_cast<uint64_t*>(win_s + 2 * C::NTOK);
  uint64_t* k_full = bars;                  // [STAGES]
  uint64_t* k_empty = k_full + C::STAGES;   // [STAGES]
  uint64_t* q_full = k_empty + C::STAGES;   // [2]
  uint64_t* q_empty = q_full + 2;           // [2]
  uint64_t* acc_full = q_empty + 2;         // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint64_t* w_full = acc_empty + 2;         // [2]
  uint64_t* w_empty = w_full + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* pages_s = const_cast<int*>(abort_flag) + 1;            // paged: first cache row of every page of the unit's chunk, per producer
  int* pagerow_s = pages_s + (PAGED ? 2 * C::PAGES * kChunkTiles : 0);   // paged: the same for the epilogue, 2 units deep (stager-written)
  float* ks_ring = reinterpret_cast<float*>(pagerow_s + (PAGED ? 2 * C::PAGES * kChunkTiles : 0));   // AHEAD x SUB x epilogue threads

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
      mbar_init(&acc_empty[i], 4 * C::SPLIT);   // one arrive per epilogue warp draining the stage
      mbar_init(&w_full[i], 1);
      mbar_init(&w_empty[i], C::EPI_WARPS);
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

  if (warp == 0 || (PAGED && warp == 3)) {
    // ------------------------------ TMA producer ------------------------------
    // paged: warps 0 and 3 each take every other tile (the per-copy issue latency of two threads overlaps)
    constexpr int PL = PAGED ? 2 : 1;
    const int pidx = warp == 0 ? 0 : 1;
    int* my_pages = pages_s + pidx * C::PAGES * kChunkTiles;
    uint32_t it = 0, nu = 0;
    for (int u = blockIdx.x; u < n_units && !*abort_flag; u += gridDim.x) {
      int qb, nb, t_lo, t_hi;
      if (!unit_tiles<NQ, QB, PAGED>(a, u, n_qblocks, n_groups, qb, nb, t_lo, t_hi)) continue;
      const int qs = nu & 1;
      bool ok = true;
      if constexpr (PAGED) {
        // the whole warp fetches the chunk's page ids at once (coalesced), so the issuing lane
        // never waits on a dependent global load per tile
        const int n_pages = (min(a.ke[qb], a.S) + kPageTokens - 1) / kPageTokens;
        __syncwarp();
        for (int i = lane; i < C::PAGES * (t_hi - t_lo); i += 32) {   // store the first cache row of each page, -1 = none
          const int page = C::PAGES * t_lo + i;
          int r = -1;
          if (page < n_pages) {
            const int phys = __ldg(a.block_table + (int64_t)qb * a.table_stride + page);
            if (phys >= 0 && (int64_t)(phys + 1) * kPageTokens <= a.num_phys_rows) r = phys * kPageTokens;
            else if (a.status) atomicCAS(a.status, kStatusOk, kStatusBadIndex);
          }
          my_pages[i] = r;
        }
        __syncwarp();
      }
      if (lane == 0 && pidx == 0) {
        ok = mbar_wait(&q_empty[qs], ((nu >> 1) & 1) ^ 1, abort_flag, a.status);
        if (ok) {
          mbar_expect_tx(&q_full[qs], nb * C::Q_TILE_BYTES);
          for (int b = 0; b < nb; ++b)
            tma_load_2d(q_s + (qs * QB + b) * C::Q_TILE_BYTES, &tmap_q, 0, (qb * QB + b) * C::N, &q_full[qs]);
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      // The whole warp walks the tiles; lane 0 waits and posts the byte count.  Paged: lanes 0..3 then issue
      // one page copy each in the same instruction, which costs the warp about what a single copy does.
      for (int kt = t_lo; kt < t_hi && ok; ++kt, ++it) {
        if (int(it % PL) != pidx) continue;
        const int st = it % C::STAGES;
        if (lane == 0) ok = mbar_wait(&k_empty[st], ((it / C::STAGES) & 1) ^ 1, abort_flag, a.status);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        uint8_t* dst = k_s + st * C::K_TILE_BYTES;
        if constexpr (!PAGED) {
          if (lane == 0) {
            mbar_expect_tx(&k_full[st], C::K_TILE_BYTES);
            tma_load_2d(dst, &tmap_k, 0, kt * C::TILE_KEYS, &k_full[st]);
          }
        } else {
          // four 64-token pages per tile; a missing or out-of-range page is skipped (rows validated above)
          const int r = lane < C::PAGES ? my_pages[C::PAGES * (kt - t_lo) + lane] : -1;
          const int n_valid = __popc(__ballot_sync(0xffffffffu, r >= 0));
          if (lane == 0) {
            if (n_valid) mbar_expect_tx(&k_full[st], n_valid * (C::K_TILE_BYTES / C::PAGES));
            else mbar_arrive(&k_full[st]);
          }
          __syncwarp();
          if (r >= 0) tma_load_2d(dst + lane * (C::K_TILE_BYTES / C::PAGES), &tmap_k, 0, r, &k_full[st]);
        }
      }
      ++nu;
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
    uint32_t it = 0, it2 = 0, nu = 0;
    for (int u = blockIdx.x; u < n_units && !*abort_flag; u += gridDim.x) {
      int qb, nb, t_lo, t_hi;
      if (!unit_tiles<NQ, QB, PAGED>(a, u, n_qblocks, n_groups, qb, nb, t_lo, t_hi)) continue;
      const int qs = nu & 1;
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait(&q_full[qs], (nu >> 1) & 1, abort_flag, a.status);
        for (int kt = t_lo; kt < t_hi && ok; ++kt, ++it) {
          const int st = it % C::STAGES;
          ok = mbar_wait(&k_full[st], (it / C::STAGES) & 1, abort_flag, a.status);
          const uint64_t kdesc = umma_smem_desc(smem_u32(k_s + st * C::K_TILE_BYTES), 16, C::SBO, C::SWZ);
          constexpr uint32_t kSubDesc = (kTileKeys * D) >> 4;     // descriptor step from one 128-key half to the next
          for (int b = 0; b < nb && ok; ++b, ++it2) {
            const int acc = it2 & 1;
            ok = mbar_wait(&acc_empty[acc], ((it2 >> 1) & 1) ^ 1, abort_flag, a.status);
            if (!ok) break;
            tc_fence_after();
            const uint64_t qdesc =
                umma_smem_desc(smem_u32(q_s + (qs * QB + b) * C::Q_TILE_BYTES), 16, C::SBO, C::SWZ);
#pragma unroll
            for (int sub = 0; sub < C::SUB; ++sub)
#pragma unroll
              for (int k = 0; k < C::KSTEPS; ++k)
                umma_f8(tmem_base + acc * C::ACC_COLS + sub * C::N, kdesc + sub * kSubDesc + (k * 32 >> 4),
                        qdesc + (k * 32 >> 4), idesc, k > 0);
            umma_commit(&acc_full[acc]);
          }
          if (ok) umma_commit(&k_empty[st]);
        }
        if (ok) umma_commit(&q_empty[qs]);
      }
      ++nu;
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      it = __shfl_sync(0xffffffffu, it, 0);
      it2 = __shfl_sync(0xffffffffu, it2, 0);
      if (!ok) break;
    }
  } else if (warp == 2) {
    // ------------------- stager: head weights and windows per unit -------------------
    uint32_t nu = 0;
    for (int u = blockIdx.x; u < n_units && !*abort_flag; u += gridDim.x) {
      int qb, nb, t_lo, t_hi;
      if (!unit_tiles<NQ, QB, PAGED>(a, u, n_qblocks, n_groups, qb, nb, t_lo, t_hi)) continue;
      const int ub = nu & 1;
      const bool ok = __all_sync(0xffffffffu, mbar_wait(&w_empty[ub], ((nu >> 1) & 1) ^ 1, abort_flag, a.status));
      if (!ok) break;
      float* wd = w_s + ub * QB * C::N;
      int2* wind = win_s + ub * C::NTOK;
      const int t0 = qb * QB * NQ;
      for (int c = lane; c < QB * C::N; c += 32) {
        const int t = t0 + c / H;
        float wvv = 0.f;
        if (t < a.T) {
          const int64_t off = (int64_t)t * H + (c % H);
          wvv = a.w_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.w)[off])
                            : reinterpret_cast<const float*>(a.w)[off];
        }
        wd[c] = wvv;
      }
      for (int j = lane; j < C::NTOK; j += 32) {
        const int t = t0 + j;
        int s0 = 0, s1 = 0;
        if (t < a.T) {
          s0 = (!PAGED && a.ks) ? max(a.ks[t], 0) : 0;
          s1 = min(a.ke[t], a.S);
        }
        wind[j] = make_int2(s0, max(s1 - s0, 0));
      }
      if constexpr (PAGED) {
        // first cache row of each page of the chunk (-1 = none), so that the epilogue's k_scale fetch is one load
        int* pr = pagerow_s + ub * C::PAGES * kChunkTiles;
        const int n_pages = (min(a.ke[qb], a.S) + kPageTokens - 1) / kPageTokens;
        for (int i = lane; i < C::PAGES * (t_hi - t_lo); i += 32) {
          const int page = C::PAGES * t_lo + i;
          int r = -1;
          if (page < n_pages) {
            const int phys = __ldg(a.block_table + (int64_t)qb * a.table_stride + page);
            if (phys >= 0 && (int64_t)(phys + 1) * kPageTokens <= a.num_phys_rows) r = phys * kPageTokens;
          }
          pr[i] = r;
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&w_full[ub]);
      ++nu;
    }
  } else if (warp >= 4) {
    // --------------------------- epilogue warpgroups ---------------------------
    const int ew = warp - 4;                     // epilogue warp index
    const int wg = ew >> 2;                      // warpgroup
    const int stage = wg & 1;                    // accumulator stage it drains
    const int part = wg >> 1;                    // which share of the columns (SPLIT > 1)
    const int wq = warp & 3;                     // TMEM lane quadrant of this warp
    const int row = wq * 32 + lane;              // key within the tile = TMEM lane
    const uint32_t t_lane = tmem_base + (uint32_t(wq * 32) << 16) + stage * C::ACC_COLS;
    uint32_t it2 = 0, n_mine = 0, nu = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
      int qb, nb, t_lo, t_hi;
      if (!unit_tiles<NQ, QB, PAGED>(a, u, n_qblocks, n_groups, qb, nb, t_lo, t_hi)) continue;
      const int ub = nu & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&w_full[ub], (nu >> 1) & 1, abort_flag, a.status));
      if (!ok) break;
      // k_scale of the tile AHEAD tiles on travels global -> shared asynchronously into this thread's own slot
      // (paged: its cache row comes from the page rows the stager wrote, so it is a single fetch)
      float* my_ring = ks_ring + (threadIdx.x - 128);
      const int* pr = pagerow_s + ub * C::PAGES * kChunkTiles;
      auto prefetch_kscale = [&](int tile) {
        if (tile < t_hi) {
#pragma unroll
          for (int sub = 0; sub < C::SUB; ++sub) {
            const int sk = tile * C::TILE_KEYS + sub * kTileKeys + row;
            const float* src = a.k_scale;
            bool valid;
            if constexpr (!PAGED) {
              valid = sk < a.S;
              if (valid) src += sk;
            } else {
              const int r = pr[C::PAGES * (tile - t_lo) + 2 * sub + (row >> 6)];
              valid = r >= 0;
              if (valid) src += r + (row & (kPageTokens - 1));
            }
            cp_async_f32(my_ring + ((tile % C::AHEAD) * C::SUB + sub) * (EPI * 128), src, valid);
          }
        }
        cp_async_commit();                       // one group per tile, empty past the end of the unit
      };
      const uint32_t ld32 = static_cast<uint32_t>(a.ld);
#pragma unroll
      for (int i = 0; i < C::AHEAD; ++i) prefetch_kscale(t_lo + i);
      for (int kt = t_lo; kt < t_hi && ok; ++kt) {
        cp_async_wait<C::AHEAD - 1>();           // this tile's group has landed
        float kscale[C::SUB];
#pragma unroll
        for (int sub = 0; sub < C::SUB; ++sub) kscale[sub] = my_ring[((kt % C::AHEAD) * C::SUB + sub) * (EPI * 128)];
        prefetch_kscale(kt + C::AHEAD);          // reuses the slots just read
        for (int b = 0; b < nb; ++b, ++it2) {
          if (int(it2 & 1) != stage) continue;
          const int g = qb * QB + b;
          const float* my_w = w_s + (ub * QB + b) * C::N;
          const int2* my_win = win_s + ub * C::NTOK + b * NQ;
          float* grp_base = a.logits + (int64_t)g * NQ * a.ld;   // 32-bit offsets from here: NQ * ld < 2^31
          const int n_tok = min(NQ, a.T - g * NQ);
          ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[stage], n_mine & 1, abort_flag, a.status));
          if (!ok) break;
          tc_fence_after();
#pragma unroll
          for (int sub = 0; sub < C::SUB; ++sub) {
            const int s = kt * C::TILE_KEYS + sub * kTileKeys + row;    // logical key position
            const uint32_t t_sub = t_lane + sub * C::N;
            if constexpr (C::SPLIT == 1) {
              drain_columns<H, NQ, C::CH, 0, C::N>(t_sub, my_w, my_win, kscale[sub], s, s < a.S, n_tok, grp_base, ld32);
            } else {
              if (part == 0)
                drain_columns<H, NQ, C::CH, 0, C::COLS_PER_WG>(t_sub, my_w, my_win, kscale[sub], s, s < a.S, n_tok,
                                                               grp_base, ld32);
              else
                drain_columns<H, NQ, C::CH, C::COLS_PER_WG, C::COLS_PER_WG>(t_sub, my_w, my_win, kscale[sub], s,
                                                                            s < a.S, n_tok, grp_base, ld32);
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&acc_empty[stage]);
          ++n_mine;
        }
      }
      cp_async_wait<0>();                        // nothing of this unit may land in a slot of the next
      __syncwarp();
      if (lane == 0) mbar_arrive(&w_empty[ub]);
      ++nu;
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
// call being replaced): columns below the query block's first tile and above its last.
template <int NTOK>
__global__ void fill_masked_kernel(const IndexerArgs a) {
  const int t = blockIdx.x;
  if (t >= a.T) return;
  __shared__ int s_lo, s_hi;
  if (threadIdx.x < 32) {
    int lo, hi;
    token_window<false>(a, (t / NTOK) * NTOK, NTOK, lo, hi);
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

// ---------------------------------------------------------------------------------------------------
// Register-weight form for 64 heads x 128 dims over contiguous keys (the prefill shape).
// The epilogue of the general kernel is bound by delivering head weights from shared memory: every thread
// needs all 256 weights of a tile, 128 KB per tile through a 128 B/clk port.  Here a tile is still 128 keys x
// (4 query tokens x 64 heads), but each of FOUR epilogue warpgroups owns ONE token of the group: its 64
// weights stay in registers (32 packed pairs) for the whole work unit, and per tile a thread walks only the
// 64 accumulator columns of its token.  No shared-memory traffic in the inner loop at all.  The price: a unit
// holds one query group (not two), so a key tile fetched from L2 serves 4 query tokens instead of 8.
// Summation order per (token, key) is the same as in the general kernel: the two forms agree bit for bit.
struct RwCfg {
  static constexpr int H = 64, D = 128, NQ = 4, N = 256, KSTEPS = 4;
  static constexpr int K_TILE_BYTES = kTileKeys * D, Q_TILE_BYTES = N * D;
  static constexpr int STAGES = 6;
  static constexpr int EPI_WG = 4, EPI_WARPS = 16, THREADS = 128 + EPI_WG * 128;
  static constexpr uint32_t SBO = 8 * D;
  static constexpr int SMEM_BYTES = 1024 + STAGES * K_TILE_BYTES + 2 * Q_TILE_BYTES + 2 * N * 4 + 2 * NQ * 8 + 256;
  static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

__global__ void __launch_bounds__(RwCfg::THREADS, 1)
indexer_logits_rw_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                         const IndexerArgs a, const int n_groups, const int n_units) {
  using C = RwCfg;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* k_s = smem;                                        // STAGES x [128 keys x D]
  uint8_t* q_s = k_s + C::STAGES * C::K_TILE_BYTES;           // 2 x [N rows x D]
  float* w_s = reinterpret_cast<float*>(q_s + 2 * C::Q_TILE_BYTES);   // 2 x N head weights
  int2* win_s = reinterpret_cast<int2*>(w_s + 2 * C::N);              // 2 x NQ (ks, ke - ks)
  uint64_t* bars = reinterpret_cast<uint64_t*>(win_s + 2 * C::NQ);
  uint64_t* k_full = bars;                  // [STAGES]
  uint64_t* k_empty = k_full + C::STAGES;   // [STAGES]
  uint64_t* q_full = k_empty + C::STAGES;   // [2]
  uint64_t* q_empty = q_full + 2;           // [2]
  uint64_t* acc_full = q_empty + 2;         // [2]
  uint64_t* acc_empty = acc_full + 2;       // [2]
  uint64_t* w_full = acc_empty + 2;         // [2]
  uint64_t* w_empty = w_full + 2;           // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_empty + 2);
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
      mbar_init(&acc_empty[i], C::EPI_WARPS);     // every epilogue warp drains a share of every stage
      mbar_init(&w_full[i], 1);
      mbar_init(&w_empty[i], C::EPI_WARPS);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
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
      int g, nb, t_lo, t_hi;
      if (!unit_tiles<C::NQ, 1, false>(a, u, n_groups, n_groups, g, nb, t_lo, t_hi)) continue;
      const int qs = nu & 1;
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait(&q_empty[qs], ((nu >> 1) & 1) ^ 1, abort_flag, a.status);
        if (ok) {
          mbar_expect_tx(&q_full[qs], C::Q_TILE_BYTES);
          tma_load_2d(q_s + qs * C::Q_TILE_BYTES, &tmap_q, 0, g * C::N, &q_full[qs]);
        }
        for (int kt = t_lo; kt < t_hi && ok; ++kt, ++it) {
          const int st = it % C::STAGES;
          ok = mbar_wait(&k_empty[st], ((it / C::STAGES) & 1) ^ 1, abort_flag, a.status);
          if (!ok) break;
          mbar_expect_tx(&k_full[st], C::K_TILE_BYTES);
          tma_load_2d(k_s + st * C::K_TILE_BYTES, &tmap_k, 0, kt * kTileKeys, &k_full[st]);
        }
      }
      ++nu;
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      it = __shfl_sync(0xffffffffu, it, 0);
      if (!ok) break;
    }
    if (lane == 0 && *abort_flag) {               // on abort, give copies already in flight a bounded chance to land
      for (int st = 0; st < C::STAGES; ++st)
        for (uint32_t spin = 0; spin < (1u << 16) && !mbar_try_wait(&k_full[st], 0) && !mbar_try_wait(&k_full[st], 1); ++spin) {
        }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    constexpr uint32_t idesc = umma_idesc(0, 0, 0, 0, kTileKeys, C::N);
    uint32_t it = 0, nu = 0;
    for (int u = blockIdx.x; u < n_units && !*abort_flag; u += gridDim.x) {
      int g, nb, t_lo, t_hi;
      if (!unit_tiles<C::NQ, 1, false>(a, u, n_groups, n_groups, g, nb, t_lo, t_hi)) continue;
      const int qs = nu & 1;
      bool ok = true;
      if (lane == 0) {
        ok = mbar_wait(&q_full[qs], (nu >> 1) & 1, abort_flag, a.status);
        const uint64_t qdesc = umma_smem_desc(smem_u32(q_s + qs * C::Q_TILE_BYTES), 16, C::SBO, kSwz128);
        for (int kt = t_lo; kt < t_hi && ok; ++kt, ++it) {
          const int st = it % C::STAGES, acc = it & 1;
          ok = mbar_wait(&k_full[st], (it / C::STAGES) & 1, abort_flag, a.status) &&
               mbar_wait(&acc_empty[acc], ((it >> 1) & 1) ^ 1, abort_flag, a.status);
          if (!ok) break;
          tc_fence_after();
          const uint64_t kdesc = umma_smem_desc(smem_u32(k_s + st * C::K_TILE_BYTES), 16, C::SBO, kSwz128);
#pragma unroll
          for (int k = 0; k < C::KSTEPS; ++k)
            umma_f8(tmem_base + acc * C::N, kdesc + (k * 32 >> 4), qdesc + (k * 32 >> 4), idesc, k > 0);
          umma_commit(&acc_full[acc]);
          umma_commit(&k_empty[st]);
        }
        if (ok) umma_commit(&q_empty[qs]);
      }
      ++nu;
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      it = __shfl_sync(0xffffffffu, it, 0);
      if (!ok) break;
    }
  } else if (warp == 2) {
    // ------------------- stager: head weights and windows of the next unit -------------------
    uint32_t nu = 0;
    for (int u = blockIdx.x; u < n_units && !*abort_flag; u += gridDim.x) {
      int g, nb, t_lo, t_hi;
      if (!unit_tiles<C::NQ, 1, false>(a, u, n_groups, n_groups, g, nb, t_lo, t_hi)) continue;
      const int ub = nu & 1;
      const bool ok = __all_sync(0xffffffffu, mbar_wait(&w_empty[ub], ((nu >> 1) & 1) ^ 1, abort_flag, a.status));
      if (!ok) break;
      float* wd = w_s + ub * C::N;
      const int t0 = g * C::NQ;
      for (int c = lane; c < C::N; c += 32) {
        const int t = t0 + c / C::H;
        float wvv = 0.f;
        if (t < a.T) {
          const int64_t off = (int64_t)t * C::H + (c % C::H);
          wvv = a.w_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.w)[off])
                            : reinterpret_cast<const float*>(a.w)[off];
        }
        wd[c] = wvv;
      }
      if (lane < C::NQ) {
        const int t = t0 + lane;
        int s0 = 0, s1 = 0;
        if (t < a.T) {
          s0 = a.ks ? max(a.ks[t], 0) : 0;
          s1 = min(a.ke[t], a.S);
        }
        win_s[ub * C::NQ + lane] = make_int2(s0, max(s1 - s0, 0));
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&w_full[ub]);
      ++nu;
    }
  } else if (warp >= 4) {
    // ------------- epilogue: warpgroup = query token of the group, thread = key of the tile -------------
    const int ew = warp - 4;
    const int tok = ew >> 2;                     // token within the group = 64-column slice of the accumulator
    const int wq = warp & 3;                     // TMEM lane quadrant of this warp
    const int row = wq * 32 + lane;              // key within the tile = TMEM lane
    const uint32_t t_lane = tmem_base + (uint32_t(wq * 32) << 16) + tok * C::H;
    uint32_t it = 0, nu = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
      int g, nb, t_lo, t_hi;
      if (!unit_tiles<C::NQ, 1, false>(a, u, n_groups, n_groups, g, nb, t_lo, t_hi)) continue;
      const int ub = nu & 1;
      ok = __all_sync(0xffffffffu, mbar_wait(&w_full[ub], (nu >> 1) & 1, abort_flag, a.status));
      if (!ok) break;
      uint64_t wreg[C::H / 2];                   // this token's 64 head weights as 32 packed pairs, for the whole unit
      {
        const float4* src = reinterpret_cast<const float4*>(w_s + ub * C::N + tok * C::H);
#pragma unroll
        for (int i = 0; i < C::H / 4; ++i) {
          const float4 w4 = src[i];
          wreg[2 * i] = pack_f32x2(w4.x, w4.y);
          wreg[2 * i + 1] = pack_f32x2(w4.z, w4.w);
        }
      }
      const int2 win = win_s[ub * C::NQ + tok];  // (ks, ke - ks)
      __syncwarp();
      if (lane == 0) mbar_arrive(&w_empty[ub]);  // weights and window are in registers
      const int t_tok = g * C::NQ + tok;
      float* out_row = a.logits + (int64_t)t_tok * a.ld;
      for (int kt = t_lo; kt < t_hi && ok; ++kt, ++it) {
        const int stage = it & 1;
        // k_scale is only needed for the last multiply of the tile: a plain load requested here has the whole
        // tile's work to arrive (the array is L2-resident), and nothing is carried from tile to tile
        const int s = kt * kTileKeys + row;              // key position
        const float kscale = s < a.S ? __ldg(a.k_scale + s) : 0.f;
        ok = __all_sync(0xffffffffu, mbar_wait(&acc_full[stage], (it >> 1) & 1, abort_flag, a.status));
        if (!ok) break;
        tc_fence_after();
        const uint32_t t_acc = t_lane + stage * C::N;
        uint32_t v[2][16];
        uint64_t chain[2];
        tmem_ld16(t_acc, v[0]);
#pragma unroll
        for (int c = 0; c < C::H; c += 16) {
          const int cur = (c >> 4) & 1;
          tmem_wait_ld();
          if (c + 16 < C::H) tmem_ld16(t_acc + c + 16, v[cur ^ 1]);
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            const int hp = (c + i) >> 1;               // head pair
            const float d0 = fmaxf(__uint_as_float(v[cur][i]), 0.f);
            const float d1 = fmaxf(__uint_as_float(v[cur][i + 1]), 0.f);
            if (hp < 2) chain[hp] = 0;
            chain[hp & 1] = fma_f32x2(pack_f32x2(d0, d1), wreg[hp], chain[hp & 1]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[stage]);   // the accumulator slice is in registers
        float e0, o0, e1, o1;
        unpack_f32x2(chain[0], e0, o0);
        unpack_f32x2(chain[1], e1, o1);
        const float score = (0.f + (e0 + o0)) + (e1 + o1);
        if (s < a.S && t_tok < a.T) {
          const bool in = static_cast<uint32_t>(s - win.x) < static_cast<uint32_t>(win.y);
          out_row[s] = in ? score * kscale : -CUDART_INF_F;
        }
      }
      ++nu;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
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

// 2-D byte tensor [rows, inner_bytes] (row pitch in bytes) with a [box_rows, box_bytes] box whose
// shared-memory image is swizzled by the box width (128 or 64 bytes).  The map is declared with
// 4-byte elements (every size here is a multiple of 4), so the x coordinate of a copy counts
// 4-byte units; the swizzle works on 16-byte chunks and does not depend on the element type.
int make_tmap_2d_bytes(CUtensorMap* m, const void* base, uint64_t rows, uint64_t inner_bytes, uint64_t row_pitch,
                       uint32_t box_bytes, uint32_t box_rows) {
  auto fn = encode_fn();
  if (!fn) return set_error(DSA_ERR_CUDA, "cuTensorMapEncodeTiled entry point not found");
  if ((inner_bytes | box_bytes) & 3) return set_error(DSA_ERR_SHAPE, "tensor map: sizes must be multiples of 4 bytes");
  cuuint64_t dims[2] = {inner_bytes / 4, rows};
  cuuint64_t strides[1] = {row_pitch};
  cuuint32_t box[2] = {box_bytes / 4, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUtensorMapSwizzle sw = box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                        : box_bytes == 64  ? CU_TENSOR_MAP_SWIZZLE_64B
                                           : CU_TENSOR_MAP_SWIZZLE_NONE;
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(DSA_ERR_CUDA, "cuTensorMapEncodeTiled failed (code %d)", (int)r);
  return DSA_OK;
}

int make_tmap_2d_u8(CUtensorMap* m, const void* base, uint64_t rows, uint32_t row_bytes, uint64_t row_pitch,
                    uint32_t box_rows) {
  return make_tmap_2d_bytes(m, base, rows, row_bytes, row_pitch, row_bytes, box_rows);
}

template <int H, int D, int NQ, bool PAGED, int QB, int EPI>
static int launch_indexer(const void* q, const void* k, const IndexerArgs& args, int clean, cudaStream_t stream) {
  using C = IdxCfg<H, D, NQ, PAGED, QB, EPI>;
  if (args.T == 0 || args.S == 0) return DSA_OK;
  IndexerArgs a = args;
  CUtensorMap tq, tk;
  int rc = make_tmap_2d_u8(&tq, q, (uint64_t)a.T * H, D, D, C::N);
  if (rc) return rc;
  rc = PAGED ? make_tmap_2d_u8(&tk, k, (uint64_t)a.num_phys_rows, D, D, kPageTokens)
             : make_tmap_2d_u8(&tk, k, (uint64_t)a.S, D, D, kTileKeys);
  if (rc) return rc;
  const int n_groups = (a.T + NQ - 1) / NQ;
  const int n_qblocks = (n_groups + QB - 1) / QB;
  const int n_tiles = (a.S + C::TILE_KEYS - 1) / C::TILE_KEYS;
  // Units are dealt to the CTAs round-robin: keep at least six rounds of them so that the last, partly
  // filled round costs little, by cutting the key range finer when there are few query blocks.
  a.chunk_tiles = kChunkTiles;
  while (a.chunk_tiles > 8 &&
         (int64_t)n_qblocks * ((n_tiles + a.chunk_tiles - 1) / a.chunk_tiles) < 6LL * sm_count())
    a.chunk_tiles /= 2;
  const int n_chunks = (n_tiles + a.chunk_tiles - 1) / a.chunk_tiles;
  const int64_t n_units64 = (int64_t)n_qblocks * n_chunks;
  if (n_units64 > 0x7fffffff) return set_error(DSA_ERR_SHAPE, "indexer: too many work units");
  const int n_units = (int)n_units64;
  auto kern = indexer_logits_kernel<H, D, NQ, PAGED, QB, EPI>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
    return set_error(DSA_ERR_CUDA, "indexer: cannot raise dynamic shared memory to %d", C::SMEM_BYTES);
  const int grid = n_units < sm_count() ? n_units : sm_count();
  kern<<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(tq, tk, a, n_groups, n_qblocks, n_units);
  if constexpr (!PAGED) {
    if (clean) fill_masked_kernel<C::NTOK><<<a.T, 256, 0, stream>>>(a);
  }
  return check_launch("indexer_logits");
}


static int launch_indexer_rw(const void* q, const void* k, const IndexerArgs& args, int clean, cudaStream_t stream) {
  using C = RwCfg;
  if (args.T == 0 || args.S == 0) return DSA_OK;
  IndexerArgs a = args;
  CUtensorMap tq, tk;
  int rc = make_tmap_2d_u8(&tq, q, (uint64_t)a.T * C::H, C::D, C::D, C::N);
  if (rc) return rc;
  rc = make_tmap_2d_u8(&tk, k, (uint64_t)a.S, C::D, C::D, kTileKeys);
  if (rc) return rc;
  const int n_groups = (a.T + C::NQ - 1) / C::NQ;
  const int n_tiles = (a.S + kTileKeys - 1) / kTileKeys;
  a.chunk_tiles = kChunkTiles;                      // same rule as the general form: at least six rounds of units
  while (a.chunk_tiles > 8 && (int64_t)n_groups * ((n_tiles + a.chunk_tiles - 1) / a.chunk_tiles) < 6LL * sm_count())
    a.chunk_tiles /= 2;
  const int64_t n_units64 = (int64_t)n_groups * ((n_tiles + a.chunk_tiles - 1) / a.chunk_tiles);
  if (n_units64 > 0x7fffffff) return set_error(DSA_ERR_SHAPE, "indexer: too many work units");
  const int n_units = (int)n_units64;
  if (cudaFuncSetAttribute(indexer_logits_rw_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES) != cudaSuccess)
    return set_error(DSA_ERR_CUDA, "indexer: cannot raise dynamic shared memory to %d", C::SMEM_BYTES);
  const int grid = n_units < sm_count() ? n_units : sm_count();
  indexer_logits_rw_kernel<<<grid, C::THREADS, C::SMEM_BYTES, stream>>>(tq, tk, a, n_groups, n_units);
  if (clean) fill_masked_kernel<C::NQ><<<a.T, 256, 0, stream>>>(a);
  return check_launch("indexer_logits");
}

// general != 0 keeps 64 heads x 128 on the general kernel (the test hook that compares the two forms)
int indexer_logits_dispatch(const void* q, const void* k, const IndexerArgs& a, int H, int D, int clean, int general,
                            cudaStream_t stream) {
  if (H == 64 && D == 128 && !general) return launch_indexer_rw(q, k, a, clean, stream);
#define DSA_IDX_CASE(h, d) \
  if (H == h && D == d) return launch_indexer<h, d, 256 / h, false, 2, 2>(q, k, a, clean, stream);
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
  if (H == 64 && D == 128) return launch_indexer<64, 128, 1, true, 1, 2>(q, kcache, a, 0, stream);
  if (H == 32 && D == 128) return launch_indexer<32, 128, 1, true, 1, 2>(q, kcache, a, 0, stream);
  if (H == 16 && D == 128) return launch_indexer<16, 128, 1, true, 1, 2>(q, kcache, a, 0, stream);
  return set_error(DSA_ERR_SHAPE, "paged indexer: unsupported (heads=%d, head_dim=%d)", H, D);
}

int indexer_logits_contiguous(const void* q, const void* k, const float* k_scale, const void* w, int w_dtype,
                              const int32_t* ks, const int32_t* ke, float* logits, int64_t ld, int T, int S,
                              int H, int D, int clean, int general, int32_t* status, cudaStream_t stream) {
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
  return indexer_logits_dispatch(q, k, a, H, D, clean, general, stream);
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
