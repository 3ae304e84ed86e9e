// Block-sparse multi-head attention on sm_100a: the call the reference reaches through
// register_sparse_fa().run (sparse_attn/DSA.py:232-247), i.e.
//   triton_block_sparse_attn_fwd_openai_prefetch(q, k, v, idx, num, sm_scale) -> (out, _)
// q, k, v, out [B, S, H, 128] bf16; 64-token blocks; idx [B, H, S/64, topk] int32 lists, for every query
// block, the key blocks it attends to (the first num[b, h, qb] entries count); non-causal.
//   out[b, s, h, :] = softmax_j(scale * q[b, s, h, :] . k[b, j, h, :]) v[b, j, h, :],  j over the listed blocks
//
// Persistent CTAs, two per SM, each walking units (batch, head, query block).  A query block is 64 rows, so
// the MMAs are M = 64: their accumulator rows sit in lanes 0-15 of each 32-lane quadrant of tensor memory,
// and each of the four softmax warps works on 16 rows.  Barrier stages and phases follow from running
// counters, so the producers load the next unit's Q, K and V while the current unit is still in its tail.
//   * warps 0 and 2: TMA producers (Q and K; V).  Q [64 x 128] once per unit, then per listed key block K and
//     V [64 x 128], each as two 128-byte-swizzled panels of 64 dims, into a 3-stage K ring and a 2-stage V ring;
//     32 list entries are read at a time, one per lane.
//   * warp 1: owns the tensor memory; lane 0 issues S = Q K^T (8 tcgen05.mma kind::f16, K-major
//     operands) into one of two score buffers, up to two blocks ahead of the softmax, and O += P V
//     (4 MMAs; P from shared memory, V read through an MN-major descriptor, so the [key][dim] tile needs
//     no transpose).  It polls "next K landed and its score buffer read" and "this block's P and V
//     ready" together, so neither a late K tile nor a slow softmax leaves the tensor pipe idle.
//   * warps 4-7: online softmax.  Scores come from tensor memory; a row (lanes 0-15 of the quadrant) is
//     split over a lane pair -- lane r keeps columns 0-31, lane r+16 receives 32-63 by shuffle -- so all
//     32 lanes compute; P goes to one of two shared-memory buffers as bf16 in the K-major swizzled
//     layout; the running maximum is raised (and O rescaled in tensor memory) only when it grows by
//     more than 8 in log2 units.
// Every wait is bounded (dsa_common.cuh).
#include <cuda.h>
#include <cudaTypedefs.h>
#include <math_constants.h>

#include "dsa_common.cuh"
#include "dsa_host.h"

namespace dsa {

constexpr int kBsBlk = 64;                         // tokens per query / key block
constexpr int kBsD = 128;                          // head dim
constexpr int kBsPanelBytes = kBsBlk * 128;        // [64 rows x 64 dims] bf16
constexpr int kBsTileBytes = 2 * kBsPanelBytes;    // [64 rows x 128 dims]
constexpr int kBsKStages = 3;                      // K tiles in flight: a K stage is free once its scores are computed
constexpr int kBsVStages = 2;                      // V tiles in flight: needed one softmax later, freed after P.V
constexpr int kBsThreads = 256;
constexpr int kBsSmemBytes = kBsTileBytes /*Q*/ + (kBsKStages + kBsVStages) * kBsTileBytes /*K,V*/ +
                             2 * kBsPanelBytes /*P, double-buffered*/ + 256 /*barriers*/;
static_assert(2 * (kBsSmemBytes + 1024) <= 228 * 1024, "two CTAs per SM (1 KB per CTA is reserved by the system)");
constexpr uint32_t kBsColO = 0, kBsColS = 128 /* two score buffers of 64 columns */, kBsTmemCols = 256;

struct BsArgs {
  const int32_t* lut;          // [B, H, nqb, topk]
  const int32_t* num;          // [B, H, nqb]
  __nv_bfloat16* out;          // [B, S, H, 128]
  int B, S, H, nqb, topk;
  float scale_log2e;
  int* status;
};

__device__ __forceinline__ uint32_t bs_pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float bs_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

__global__ void __launch_bounds__(kBsThreads, 2)
block_sparse_mha_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const BsArgs a, const int n_units) {
  extern __shared__ __align__(1024) uint8_t smem[];           // the swizzled tiles need 1024-byte alignment
  uint8_t* q_s = smem;                                        // 2 panels [64 rows x 128 B]
  uint8_t* k_s = q_s + kBsTileBytes;                          // stages x 2 panels
  uint8_t* v_s = k_s + kBsKStages * kBsTileBytes;             // stages x 2 panels
  uint8_t* p_s = v_s + kBsVStages * kBsTileBytes;             // 2 x [64 rows x 64 keys] bf16, one panel each
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + 2 * kBsPanelBytes);
  uint64_t* q_full = bars + 0;                                // TMA -> MMA, once per unit
  uint64_t* q_empty = bars + 1;                               // the unit's last scores are issued: Q may be replaced
  uint64_t* k_full = bars + 2;                                // [3] TMA -> MMA
  uint64_t* k_free = bars + 5;                                // [3] the scores of the block are computed
  uint64_t* v_full = bars + 8;                                // [2] TMA -> MMA
  uint64_t* v_free = bars + 10;                               // [2] P.V of the block finished
  uint64_t* s_full = bars + 12;                               // [2] MMA -> softmax
  uint64_t* s_free = bars + 14;                               // [2] softmax has read that score buffer
  uint64_t* p_full = bars + 16;                               // [2] softmax -> MMA
  uint64_t* pv_done = bars + 18;                              // [2] P.V of a block finished: O quiescent, that P buffer free
  uint64_t* o_final = bars + 20;                              // the unit's last P.V finished
  uint64_t* o_free = bars + 21;                               // the unit's O has been read out
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 22);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nkb = a.S / kBsBlk;
  const int list_cap = a.topk;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_empty, 1);
    mbar_init(o_final, 1);
    mbar_init(o_free, 128);
    for (int i = 0; i < kBsKStages; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_free[i], 1);
      mbar_init(&pv_done[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 128);
      mbar_init(&p_full[i], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (smem_u32(smem) & 1023u) {                               // never seen; the tiles would be mis-swizzled: refuse, do not compute
    if (threadIdx.x == 0 && a.status) atomicCAS(a.status, kStatusOk, kStatusWaitTimeout);
    return;
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kBsTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  // A CTA walks units u = blockIdx.x, blockIdx.x + gridDim.x, ...; unit = (batch, head, query block), query block
  // fastest, so that neighbouring CTAs share K/V blocks in L2.  Every role walks the same sequence and keeps its own
  // running counters (units with a non-empty list: nq; key blocks: jt), from which barrier stages and phases follow;
  // the producers run ahead into the next unit while the current one is still being worked on.
  auto unit_len = [&](int u) { return min(max(__ldg(a.num + u), 0), list_cap); };
  auto decode = [&](int u, int& b, int& h, int& qb) {
    qb = u % a.nqb;
    const int bh = u / a.nqb;
    h = bh % a.H;
    b = bh / a.H;
  };

  if (warp == 0 || warp == 2) {
    // ----------- TMA producers: warp 0 = Q and K, warp 2 = V.  The whole warp walks the lists; lane 0 waits and
    // posts the byte count, lanes 0 and 1 issue the two panel copies of a tile in one instruction. -----------
    const bool is_k = warp == 0;
    uint32_t nq = 0, jt = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
      const int n = unit_len(u);
      if (n == 0) continue;
      int b, h, qb;
      decode(u, b, h, qb);
      const int x0 = h * (kBsD / 2);                          // TMA x coordinate in 4-byte units: head h, dim 0
      if (is_k) {
        if (lane == 0) {
          ok = mbar_wait(q_empty, (nq & 1) ^ 1, abort_flag, a.status);
          if (ok) mbar_expect_tx(q_full, kBsTileBytes);
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        if (lane < 2) tma_load_2d(q_s + lane * kBsPanelBytes, &tmap_q, x0 + lane * 32, b * a.S + qb * kBsBlk, q_full);
      }
      const int32_t* list = a.lut + (int64_t)u * a.topk;
      for (int j0 = 0; j0 < n && ok; j0 += 32) {
        int e = (j0 + lane < n) ? __ldg(list + j0 + lane) : 0;     // 32 list entries at a time, one per lane
        if (e < 0 || e >= nkb) {
          if (is_k && a.status) atomicCAS(a.status, kStatusOk, kStatusBadIndex);
          e = 0;                                              // a bad entry reads block 0 (defined data); its scores are masked
        }
        const int jn = min(32, n - j0);
        for (int jj = 0; jj < jn && ok; ++jj, ++jt) {
          const int kb = __shfl_sync(0xffffffffu, e, jj);
          if (is_k) {
            const int st = jt % kBsKStages;
            if (lane == 0) ok = mbar_wait(&k_free[st], ((jt / kBsKStages) & 1) ^ 1, abort_flag, a.status);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (lane == 0) mbar_expect_tx(&k_full[st], kBsTileBytes);
            __syncwarp();
            if (lane < 2)
              tma_load_2d(k_s + st * kBsTileBytes + lane * kBsPanelBytes, &tmap_k, x0 + lane * 32, b * a.S + kb * kBsBlk, &k_full[st]);
          } else {
            const int st = jt & 1;
            if (lane == 0) ok = mbar_wait(&v_free[st], ((jt >> 1) & 1) ^ 1, abort_flag, a.status);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            if (lane == 0) mbar_expect_tx(&v_full[st], kBsTileBytes);
            __syncwarp();
            if (lane < 2)
              tma_load_2d(v_s + st * kBsTileBytes + lane * kBsPanelBytes, &tmap_v, x0 + lane * 32, b * a.S + kb * kBsBlk, &v_full[st]);
          }
        }
      }
      ++nq;
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(1, 1, 0, 0, 64, kBsBlk);
      constexpr uint32_t idesc_pv = umma_idesc(1, 1, 0, 1, 64, kBsD);
      const uint64_t qdesc = umma_smem_desc(smem_u32(q_s), 16, 1024, kSwz128);
      const uint64_t pdesc = umma_smem_desc(smem_u32(p_s), 16, 1024, kSwz128);
      const uint64_t kdesc0 = umma_smem_desc(smem_u32(k_s), 16, 1024, kSwz128);
      const uint64_t vdesc0 = umma_smem_desc(smem_u32(v_s), kBsPanelBytes, 1024, kSwz128);
      constexpr uint64_t kStage = kBsTileBytes >> 4, kPanel = kBsPanelBytes >> 4;
      uint32_t nq = 0, jt = 0;                                // jt: running index of the unit's first block
      bool ok = true;
      // Scores run up to two blocks ahead of the softmax (two score buffers in tensor memory): block t is issued
      // as soon as its K tile has landed and the softmax has read block t-2 out of the same buffer.
      auto qk_ready = [&](uint32_t t) -> bool {
        return mbar_try_wait(&k_full[t % kBsKStages], (t / kBsKStages) & 1) &&
               (t < 2 || mbar_try_wait(&s_free[t & 1], ((t >> 1) - 1) & 1));
      };
      auto issue_qk = [&](uint32_t t) {                       // both waits have succeeded
        const int st = t % kBsKStages;
        tc_fence_after();
#pragma unroll
        for (int p = 0; p < 2; ++p)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16_ss(tmem + kBsColS + (t & 1) * kBsBlk, qdesc + p * kPanel + 2 * ks,
                        kdesc0 + st * kStage + p * kPanel + 2 * ks, idesc_qk, (p | ks) != 0);
        umma_commit(&s_full[t & 1]);
        umma_commit(&k_free[st]);
      };
      for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
        const int n = unit_len(u);
        if (n == 0) continue;
        ok = mbar_wait(q_full, nq & 1, abort_flag, a.status);
        if (ok && nq > 0) ok = mbar_wait(o_free, (nq - 1) & 1, abort_flag, a.status);   // the previous unit's O is read out
        uint32_t qk_next = jt;                                // next block whose scores are to be issued
        const uint32_t unit_end = jt + n;
        for (int j = 0; j < n && ok; ++j) {
          const uint32_t t = jt + j;
          const int st = t & 1;
          // issue scores ahead while waiting for this block's P (and V): never stall P.V behind a late K tile,
          // never leave the tensor pipe idle while one is there
          bool have_p = false;
          for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
            if (qk_next < unit_end && qk_next <= t + 2 && qk_ready(qk_next)) {
              issue_qk(qk_next);
              if (++qk_next == unit_end) umma_commit(q_empty);   // those were the unit's last scores: Q may be replaced
              continue;
            }
            if (qk_next > t && mbar_try_wait(&v_full[st], (t >> 1) & 1) && mbar_try_wait(&p_full[t & 1], (t >> 1) & 1)) {
              have_p = true;
              break;
            }
            if (spin > kFastSpins) {
              if (*abort_flag) break;
              __nanosleep(40);
            }
          }
          if (!have_p) {
            if (!*abort_flag) {
              *abort_flag = 1;
              if (a.status) atomicCAS(a.status, kStatusOk, kStatusWaitTimeout);
            }
            ok = false;
            break;
          }
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < kBsBlk / 16; ++ks)    // 16 keys per step: 32 B along P's rows, 16 rows x 128 B into each V panel
            umma_f16_ss(tmem + kBsColO, pdesc + (t & 1) * kPanel + 2 * ks, vdesc0 + st * kStage + ks * (2048 >> 4), idesc_pv,
                        (j | ks) != 0);
          umma_commit(&v_free[st]);
          umma_commit(&pv_done[t & 1]);
          if (j == n - 1) umma_commit(o_final);
        }
        jt += n;
        ++nq;
      }
    }
  } else if (warp >= 4) {
    // ---------------------- softmax and output (lanes 0-15 of each warp hold rows) ----------------------
    const int quad = warp - 4;
    const bool active = lane < 16;
    const int row = quad * 16 + (lane & 15);                  // query row of the block (lanes 16-31 shadow lanes 0-15)
    const uint32_t t_row = tmem + (uint32_t(quad * 32) << 16);
    uint32_t nq = 0, jt = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
      const int n = unit_len(u);
      int b, h, qb;
      decode(u, b, h, qb);
      __nv_bfloat16* orow = a.out + (((int64_t)b * a.S + qb * kBsBlk + row) * a.H + h) * kBsD;
      if (n == 0) {                                           // nothing listed: zero rows
        if (active)
          for (int c = 0; c < kBsD * 2 / 16; ++c) reinterpret_cast<uint4*>(orow)[c] = make_uint4(0, 0, 0, 0);
        continue;
      }
      const int32_t* list = a.lut + (int64_t)u * a.topk;
      float m = -CUDART_INF_F, l = 0.f;
      for (int j = 0; j < n && ok; ++j, ++jt) {
        const int kb = __ldg(list + j);                       // requested before the wait: only its validity is needed
        ok = __all_sync(0xffffffffu, mbar_wait(&s_full[jt & 1], (jt >> 1) & 1, abort_flag, a.status));
        if (!ok) break;
        tc_fence_after();
        uint32_t sv[kBsBlk];
        tmem_ld32(t_row + kBsColS + (jt & 1) * kBsBlk, *reinterpret_cast<uint32_t(*)[32]>(sv));
        tmem_ld32(t_row + kBsColS + (jt & 1) * kBsBlk + 32, *reinterpret_cast<uint32_t(*)[32]>(sv + 32));
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&s_free[jt & 1]);
        const bool listed = kb >= 0 && kb < nkb;
        // An M = 64 accumulator keeps its rows in lanes 0-15 of the quadrant, so lanes 16-31 would idle (and
        // pay for 64 exponentials of garbage).  Each row is split instead: lane r keeps columns 0-31, lane
        // r + 16 receives columns 32-63 by shuffle; maximum and sum are combined across the pair.
        float x[kBsBlk / 2];                           // raw scores; the (positive) scale is folded into the exponent's FMA
        float bmax = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < kBsBlk / 2; ++i) {
          const uint32_t hi = __shfl_sync(0xffffffffu, sv[kBsBlk / 2 + i], lane & 15);
          x[i] = __uint_as_float(active ? sv[i] : hi);
          bmax = fmaxf(bmax, x[i]);
        }
        if (!listed) {                                 // a bad list entry (uniform, rare): the whole block is masked
#pragma unroll
          for (int i = 0; i < kBsBlk / 2; ++i) x[i] = -CUDART_INF_F;
          bmax = -CUDART_INF_F;
        }
        bmax = fmaxf(bmax, __shfl_xor_sync(0xffffffffu, bmax, 16)) * a.scale_log2e;
        const float m_new = fmaxf(m, bmax);
        const bool grow = m_new - m > 8.f;             // also true when m is still -inf and m_new is finite
        if (__any_sync(0xffffffffu, grow)) {
          const float alpha = grow ? bs_exp2(m - m_new) : 1.f;
          if (grow) m = m_new;
          l *= alpha;
          if (j > 0) {                                 // O must be quiescent: P.V of the previous block complete
            ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(jt - 1) & 1], ((jt - 1) >> 1) & 1, abort_flag, a.status));
            if (!ok) break;
            tc_fence_after();
#pragma unroll 1
            for (int c = 0; c < kBsD; c += 32) {       // lanes 0-15 scale their rows; the shadow lanes' rows are unused
              uint32_t ov[32];
              tmem_ld32(t_row + kBsColO + c, ov);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
              tmem_st32(t_row + kBsColO + c, ov);
            }
            tmem_wait_st();
          }
        }
        const float m_eff = (m == -CUDART_INF_F) ? 0.f : m;
        uint32_t pk[kBsBlk / 4];
        float psum = 0.f;
#pragma unroll
        for (int i = 0; i < kBsBlk / 2; i += 2) {
          const float p0 = bs_exp2(fmaf(x[i], a.scale_log2e, -m_eff)), p1 = bs_exp2(fmaf(x[i + 1], a.scale_log2e, -m_eff));
          psum += p0 + p1;
          pk[i >> 1] = bs_pack_bf16x2(p0, p1);
        }
        psum += __shfl_xor_sync(0xffffffffu, psum, 16);
        l += psum;
        if (jt > 1) {                                  // two P buffers: P.V of block jt-2 (of any unit) read this one
          ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[jt & 1], ((jt >> 1) - 1) & 1, abort_flag, a.status));
          if (!ok) break;
        }
        {                                              // this lane's half row of P: 64 bytes, K-major, 128-byte swizzle
          uint8_t* dst = p_s + (jt & 1) * kBsPanelBytes + row * 128;
          const int c0 = (lane >> 4) * 4;              // first 16-byte chunk: columns 0-31 or 32-63
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(dst + (((c0 + c) ^ (row & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
        }
        fence_async_smem();                            // visible to the tensor core's reads
        tc_fence_before();
        mbar_arrive(&p_full[jt & 1]);
      }
      if (ok) ok = __all_sync(0xffffffffu, mbar_wait(o_final, nq & 1, abort_flag, a.status));
      if (!ok) break;
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
      for (int c = 0; c < kBsD; c += 32) {
        uint32_t ov[32];
        tmem_ld32(t_row + kBsColO + c, ov);
        tmem_wait_ld();
        if (active) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = bs_pack_bf16x2(__uint_as_float(ov[i + 0]) * inv, __uint_as_float(ov[i + 1]) * inv);
            w.y = bs_pack_bf16x2(__uint_as_float(ov[i + 2]) * inv, __uint_as_float(ov[i + 3]) * inv);
            w.z = bs_pack_bf16x2(__uint_as_float(ov[i + 4]) * inv, __uint_as_float(ov[i + 5]) * inv);
            w.w = bs_pack_bf16x2(__uint_as_float(ov[i + 6]) * inv, __uint_as_float(ov[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c + i) = w;
          }
        }
      }
      tc_fence_before();
      mbar_arrive(o_free);                             // the next unit's first P.V may overwrite O
      ++nq;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kBsTmemCols);
  }
}

int make_tmap_2d_bytes(CUtensorMap* m, const void* base, uint64_t rows, uint64_t inner_bytes, uint64_t row_pitch,
                       uint32_t box_bytes, uint32_t box_rows);

int block_sparse_mha_launch(const void* q, const void* k, const void* v, const int32_t* lut, const int32_t* num,
                            void* out, int B, int S, int H, int topk, float scale, int32_t* status,
                            cudaStream_t stream) {
  if (B == 0 || S == 0 || H == 0) return DSA_OK;
  CUtensorMap tq, tk, tv;
  const uint64_t pitch = (uint64_t)H * kBsD * 2;
  int rc = make_tmap_2d_bytes(&tq, q, (uint64_t)B * S, pitch, pitch, 128, kBsBlk);
  if (!rc) rc = make_tmap_2d_bytes(&tk, k, (uint64_t)B * S, pitch, pitch, 128, kBsBlk);
  if (!rc) rc = make_tmap_2d_bytes(&tv, v, (uint64_t)B * S, pitch, pitch, 128, kBsBlk);
  if (rc) return rc;
  BsArgs a{};
  a.lut = lut; a.num = num; a.out = static_cast<__nv_bfloat16*>(out);
  a.B = B; a.S = S; a.H = H; a.nqb = S / kBsBlk; a.topk = topk;
  a.scale_log2e = scale * 1.4426950408889634f;
  a.status = status;
  if (cudaFuncSetAttribute(block_sparse_mha_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kBsSmemBytes) != cudaSuccess)
    return set_error(DSA_ERR_CUDA, "block_sparse_mha: cannot raise dynamic shared memory to %d", kBsSmemBytes);
  const int64_t n_units64 = (int64_t)B * H * a.nqb;
  if (n_units64 > 0x7fffffff) return set_error(DSA_ERR_SHAPE, "block_sparse_mha: too many query blocks");
  const int n_units = (int)n_units64;
  const int grid = n_units < 2 * sm_count() ? n_units : 2 * sm_count();   // persistent: two CTAs per SM
  block_sparse_mha_kernel<<<grid, kBsThreads, kBsSmemBytes, stream>>>(tq, tk, tv, a, n_units);
  return check_launch("block_sparse_mha");
}

}  // namespace dsa
