// Block-sparse multi-head attention on sm_100a: the call the reference reaches through
// register_sparse_fa().run (sparse_attn/DSA.py:232-247), i.e.
//   triton_block_sparse_attn_fwd_openai_prefetch(q, k, v, idx, num, sm_scale) -> (out, _)
// q, k, v, out [B, S, H, 128] bf16; 64-token blocks; idx [B, H, S/64, topk] int32 lists, for every query
// block, the key blocks it attends to (the first num[b, h, qb] entries count); non-causal.
//   out[b, s, h, :] = softmax_j(scale * q[b, s, h, :] . k[b, j, h, :]) v[b, j, h, :],  j over the listed blocks
//
// One CTA per (batch, head, query block); two CTAs share an SM.  A query block is 64 rows, so the MMAs
// are M = 64: their accumulator rows sit in lanes 0-15 of each 32-lane quadrant of tensor memory, and
// each of the four softmax warps works on 16 rows.
//   * warp 0 lane 0: TMA producer.  Q [64 x 128] once, then per listed key block K and V [64 x 128]
//     each as two 128-byte-swizzled panels of 64 dims, into a two-stage ring.
//   * warp 1: owns the tensor memory; lane 0 issues S = Q K^T (8 tcgen05.mma kind::f16, K-major
//     operands) and O += P V (4 MMAs; P from shared memory, V read through an MN-major descriptor, so
//     the [key][dim] tile needs no transpose).
//   * warps 4-7: online softmax, thread = query row.  Scores come from tensor memory, P goes to shared
//     memory as bf16 in the K-major swizzled layout; the running maximum is raised (and O rescaled in
//     tensor memory) only when it grows by more than 8 in log2 units.
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
constexpr int kBsMaxList = 1024;                   // listed key blocks per query block held in shared memory
constexpr int kBsSmemBytes = 1024 + kBsTileBytes /*Q*/ + (kBsKStages + kBsVStages) * kBsTileBytes /*K,V*/ +
                             kBsPanelBytes /*P*/ + 256 /*barriers*/ + kBsMaxList * 4;
static_assert(2 * kBsSmemBytes <= 227 * 1024, "two CTAs per SM");
constexpr uint32_t kBsColO = 0, kBsColS = 128, kBsTmemCols = 256;

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
                        const __grid_constant__ CUtensorMap tmap_v, const BsArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                                        // 2 panels [64 rows x 128 B]
  uint8_t* k_s = q_s + kBsTileBytes;                          // stages x 2 panels
  uint8_t* v_s = k_s + kBsKStages * kBsTileBytes;             // stages x 2 panels
  uint8_t* p_s = v_s + kBsVStages * kBsTileBytes;             // [64 rows x 64 keys] bf16, one panel
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + kBsPanelBytes);
  uint64_t* q_full = bars + 0;
  uint64_t* o_final = bars + 1;
  uint64_t* k_full = bars + 2;                                // [3] TMA -> MMA
  uint64_t* k_free = bars + 5;                                // [3] the scores of the block are computed
  uint64_t* v_full = bars + 8;                                // [2] TMA -> MMA
  uint64_t* v_free = bars + 10;                               // [2] P.V of the block finished
  uint64_t* s_full = bars + 12;                               // MMA -> softmax
  uint64_t* s_free = bars + 13;                               // softmax has read S
  uint64_t* p_full = bars + 14;                               // softmax -> MMA
  uint64_t* pv_done = bars + 15;                              // [2] P.V of block j finished: O quiescent, P free
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* lut_s = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int nkb = a.S / kBsBlk;
  const int64_t unit = ((int64_t)b * a.H + h) * a.nqb + qb;
  const int n = min(max(a.num[unit], 0), min(a.topk, kBsMaxList));

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(o_final, 1);
    for (int i = 0; i < kBsKStages; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_free[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_free[i], 1);
      mbar_init(&pv_done[i], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(s_free, 128);
    mbar_init(p_full, 128);
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  for (int j = threadIdx.x; j < n; j += kBsThreads) {         // the list, validated once
    int kb = a.lut[unit * a.topk + j];
    if (kb < 0 || kb >= nkb) {
      if (a.status) atomicCAS(a.status, kStatusOk, kStatusBadIndex);
      kb = -1;                                                // its scores are masked: contributes nothing
    }
    lut_s[j] = kb;
  }
  if (n == 0) {                                               // nothing listed: zero rows
    if (threadIdx.x < kBsBlk) {
      uint4* o = reinterpret_cast<uint4*>(a.out + (((int64_t)b * a.S + qb * kBsBlk + threadIdx.x) * a.H + h) * kBsD);
      for (int c = 0; c < kBsD * 2 / 16; ++c) o[c] = make_uint4(0, 0, 0, 0);
    }
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
  const int x0 = h * (kBsD / 2);                              // TMA x coordinate in 4-byte units: head h, dim 0

  if (warp == 0) {
    // ------------------------------ K producer (and Q) ------------------------------
    // The whole warp walks the list; lane 0 waits and posts the byte count, then lanes 0 and 1 issue the two
    // panel copies in one instruction (a copy costs its issuing thread several hundred cycles whatever its size).
    if (lane == 0) {
      mbar_expect_tx(q_full, kBsTileBytes);
      for (int p = 0; p < 2; ++p)
        tma_load_2d(q_s + p * kBsPanelBytes, &tmap_q, x0 + p * 32, b * a.S + qb * kBsBlk, q_full);
    }
    bool ok = true;
    for (int j = 0; j < n && ok; ++j) {
      const int st = j % kBsKStages;
      if (lane == 0) ok = mbar_wait(&k_free[st], ((j / kBsKStages) & 1) ^ 1, abort_flag, a.status);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      const int kb = max(lut_s[j], 0);                        // a bad entry reads block 0 (defined data); its scores are masked
      if (lane == 0) mbar_expect_tx(&k_full[st], kBsTileBytes);
      __syncwarp();
      if (lane < 2)
        tma_load_2d(k_s + st * kBsTileBytes + lane * kBsPanelBytes, &tmap_k, x0 + lane * 32, b * a.S + kb * kBsBlk, &k_full[st]);
    }
  } else if (warp == 2) {
    // --------------------------------- V producer ---------------------------------
    bool ok = true;
    for (int j = 0; j < n && ok; ++j) {
      const int st = j & 1;
      if (lane == 0) ok = mbar_wait(&v_free[st], ((j >> 1) & 1) ^ 1, abort_flag, a.status);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      const int kb = max(lut_s[j], 0);
      if (lane == 0) mbar_expect_tx(&v_full[st], kBsTileBytes);
      __syncwarp();
      if (lane < 2)
        tma_load_2d(v_s + st * kBsTileBytes + lane * kBsPanelBytes, &tmap_v, x0 + lane * 32, b * a.S + kb * kBsBlk, &v_full[st]);
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
      bool ok = mbar_wait(q_full, 0, abort_flag, a.status);
      auto issue_qk = [&](int j) -> bool {
        const int st = j % kBsKStages;
        if (!mbar_wait(&k_full[st], (j / kBsKStages) & 1, abort_flag, a.status)) return false;
        if (j > 0 && !mbar_wait(s_free, (j - 1) & 1, abort_flag, a.status)) return false;
        tc_fence_after();
#pragma unroll
        for (int p = 0; p < 2; ++p)
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16_ss(tmem + kBsColS, qdesc + p * kPanel + 2 * ks, kdesc0 + st * kStage + p * kPanel + 2 * ks, idesc_qk,
                        (p | ks) != 0);
        umma_commit(s_full);
        umma_commit(&k_free[st]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n && ok; ++j) {
        const int st = j & 1;
        bool qk_done = j + 1 >= n;
        if (!qk_done && mbar_try_wait(&k_full[(j + 1) % kBsKStages], ((j + 1) / kBsKStages) & 1)) {   // next scores while this softmax runs
          ok = issue_qk(j + 1);
          qk_done = true;
        }
        if (!ok) break;
        ok = mbar_wait(&v_full[st], (j >> 1) & 1, abort_flag, a.status) && mbar_wait(p_full, j & 1, abort_flag, a.status);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < kBsBlk / 16; ++ks)      // 16 keys per step: 32 B along P's rows, 16 rows x 128 B into each V panel
          umma_f16_ss(tmem + kBsColO, pdesc + 2 * ks, vdesc0 + st * kStage + ks * (2048 >> 4), idesc_pv, (j | ks) != 0);
        umma_commit(&v_free[st]);
        umma_commit(&pv_done[j & 1]);
        if (j == n - 1) umma_commit(o_final);
        if (!qk_done) ok = issue_qk(j + 1);
      }
    }
  } else if (warp >= 4) {
    // ---------------------- softmax and output (lanes 0-15 of each warp hold rows) ----------------------
    const int quad = warp - 4;
    const bool active = lane < 16;
    const int row = quad * 16 + (lane & 15);                  // query row of the block (lanes 16-31 shadow lanes 0-15)
    const uint32_t t_row = tmem + (uint32_t(quad * 32) << 16);
    float m = -CUDART_INF_F, l = 0.f;
    bool ok = true;
    for (int j = 0; j < n && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(s_full, j & 1, abort_flag, a.status));
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[kBsBlk];
      tmem_ld32(t_row + kBsColS, *reinterpret_cast<uint32_t(*)[32]>(sv));
      tmem_ld32(t_row + kBsColS + 32, *reinterpret_cast<uint32_t(*)[32]>(sv + 32));
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(s_free);
      const bool listed = lut_s[j] >= 0;
      float s[kBsBlk];
      float bmax = -CUDART_INF_F;
#pragma unroll
      for (int i = 0; i < kBsBlk; ++i) {
        s[i] = (listed && active) ? __uint_as_float(sv[i]) * a.scale_log2e : -CUDART_INF_F;
        bmax = fmaxf(bmax, s[i]);
      }
      const float m_new = fmaxf(m, bmax);
      const bool grow = m_new - m > 8.f;               // also true when m is still -inf and m_new is finite
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = grow ? bs_exp2(m - m_new) : 1.f;
        if (grow) m = m_new;
        l *= alpha;
        if (j > 0) {                                   // O must be quiescent: P.V of the previous block complete
          ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, a.status));
          if (!ok) break;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < kBsD; c += 32) {
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
      uint32_t pk[kBsBlk / 2];
      float psum = 0.f;
#pragma unroll
      for (int i = 0; i < kBsBlk; i += 2) {
        const float p0 = bs_exp2(s[i] - m_eff), p1 = bs_exp2(s[i + 1] - m_eff);
        psum += p0 + p1;
        pk[i >> 1] = bs_pack_bf16x2(p0, p1);
      }
      l += psum;
      if (j > 0) {                                     // P is single-buffered: P.V of the previous block must be done
        ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, a.status));
        if (!ok) break;
      }
      if (active) {                                    // this row of P: 128 bytes, K-major, 128-byte swizzle
        uint8_t* dst = p_s + row * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<uint4*>(dst + ((c ^ (row & 7)) << 4)) = make_uint4(pk[4 * c], pk[4 * c + 1], pk[4 * c + 2], pk[4 * c + 3]);
      }
      fence_async_smem();                              // visible to the tensor core's reads
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(o_final, 0, abort_flag, a.status));
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = a.out + (((int64_t)b * a.S + qb * kBsBlk + row) * a.H + h) * kBsD;
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
  const dim3 grid(a.nqb, H, B);
  block_sparse_mha_kernel<<<grid, kBsThreads, kBsSmemBytes, stream>>>(tq, tk, tv, a);
  return check_launch("block_sparse_mha");
}

}  // namespace dsa
