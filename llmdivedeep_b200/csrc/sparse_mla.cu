// Token-sparse MLA attention on sm_100a (MQA over the shared 576-dim latent KV, 512-dim V):
//   o[t, h, :] = sum_j softmax_j(scale * q[t, h, :] . kv[idx[t, j], :]) * kv[idx[t, j], :512]
// Takes the place of the block-sparse stand-in the reference reaches through
// register_sparse_fa() (sparse_attn/DSA.py:208-249); the reference itself has no sparse-MLA
// kernel, no latent cache and no decode path (sparse_attn/DSA.py:475-477).
//
// One CTA per (query token, half of the V dimension, group of up to 128 heads).
//   * Q [128 heads x 576] arrives by TMA as nine 128-byte-swizzled K-major panels (A operand).
//   * The selected KV rows are gathered 64 at a time into nine [64 keys x 64 dims] panels with
//     the same swizzle: cp.async from the bf16 KV, or -- for the paged FP8 latent cache of
//     decode -- 16-byte loads, e4m3 -> bf16 with the per-128 group scale, 16-byte stores.
//     A panel is the K-major B operand of S = Q K^T and, read with an MN-major descriptor, the
//     B operand of O += P V: the rows are gathered once and used twice.
//   * tcgen05.mma kind::f16 (bf16 in, fp32 out): S [128 x 64] and O [128 x 256] live in tensor
//     memory; P is written back to tensor memory as packed bf16 and is the A operand of P V.
//   * Online softmax with one thread per head (= TMEM lane): the row maximum and sum are
//     thread-local; O is rescaled in tensor memory only when the running maximum grows by more
//     than 8 (in log2 units), which keeps every exponent <= 2^8.
// The two CTAs of a token each recompute S (the 512 fp32 columns of a full O would fill tensor
// memory on their own); they share nothing and need no cluster.
//
// Roles: warps 0-3 softmax / output (thread = head), warp 4 lane 0 MMA issuer (warp 4 owns the
// TMEM allocation), warps 5-8 gather.  Every wait is bounded (dsa_common.cuh).
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_fp8.h>
#include <math_constants.h>

#include "dsa_common.cuh"
#include "dsa_host.h"

namespace dsa {

constexpr int kMlaDqk = 576;
constexpr int kMlaDv = 512;
constexpr int kMlaDvHalf = 256;
#ifndef DSA_MLA_BLK
#define DSA_MLA_BLK 64
#define DSA_MLA_BUFS 2
#endif
constexpr int kMlaBlk = DSA_MLA_BLK;              // keys per block
constexpr int kMlaBufs = DSA_MLA_BUFS;            // KV buffers in shared memory
constexpr int kMlaPanels = kMlaDqk / 64;          // 9 panels of 64 dims (128 bytes)
constexpr int kMlaQTmemPanels = 5;                // Q panels kept in tensor memory as the A operand
constexpr int kMlaQSmemPanels = kMlaPanels - kMlaQTmemPanels;   // the remaining 4 stay in shared memory
constexpr int kMlaQPanelBytes = 128 * 128;        // 128 heads x 128 B
constexpr int kMlaKPanelBytes = kMlaBlk * 128;    // 32 keys x 128 B
constexpr int kMlaQBytes = kMlaPanels * kMlaQPanelBytes;   // 147456
constexpr int kMlaKBytes = kMlaPanels * kMlaKPanelBytes;   // 36864 per buffer
constexpr int kMlaThreads = 288;
constexpr int kMlaGatherThreads = 128;
constexpr int kMlaMaxK = 2048;                    // selected slots per query (row ids staged in shared memory)
constexpr int kMlaQSmemBytes = kMlaQSmemPanels * kMlaQPanelBytes;   // 65536
constexpr int kMlaSmemBytes = 1024 + kMlaQSmemBytes + kMlaBufs * kMlaKBytes + 1024 + kMlaMaxK * 4;
static_assert(kMlaBufs <= 2, "descriptor selection assumes one or two KV buffers");
static_assert(kMlaBufs * kMlaKBytes >= kMlaQTmemPanels * kMlaQPanelBytes, "the KV buffers double as the staging area of the TMEM-bound Q panels");
constexpr int kLatentTokenBytes = 656;            // 512 e4m3 + 4 fp32 scales + 64 bf16 rope
constexpr int kLatentPage = 64;
// tensor-memory columns
constexpr uint32_t kColO = 0, kColS = 256, kColP = kColS + kMlaBlk, kColQ = kColP + kMlaBlk / 2, kMlaTmemCols = 512;
static_assert(kColQ + kMlaQTmemPanels * 32 <= kMlaTmemCols, "tensor memory budget: O 256, S Blk, P Blk/2, Q 32 per panel");

struct MlaArgs {
  const __nv_bfloat16* kv;        // prefill: [S_kv, 576] bf16
  const uint8_t* cache;           // decode: [num_pages*64, 656] bytes
  const int32_t* block_table;     // decode: [B, table_stride]
  const int32_t* idx;             // [T, K] selected key positions (negative = empty)
  __nv_bfloat16* out;             // [T, H, 512]
  int64_t table_stride;
  int T, H, K;
  int S_kv;                       // prefill: rows of kv; decode: logical positions per sequence
  int num_phys_rows;              // decode: rows of the cache
  float scale_log2e;              // softmax scale * log2(e)
  int* status;
  int n_split;                    // > 1: each query's slot list is cut into n_split parts (decode with few queries)
  float* part_o;                  // [T * n_split, H, 512] fp32 normalised partial outputs
  float* part_lse;                // [T * n_split, H] log2-sum-exp of each part (-inf = empty part)
};

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t n = valid ? 16u : 0u;            // 0 source bytes = zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float fast_exp2(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}

// Gather one block of selected rows into the nine swizzled panels of a buffer.  Thread g of 128.
// rows_s: the block's row ids (prefill: kv row; decode: physical cache row), -1 = empty slot.
template <bool FP8_PAGED>
__device__ __forceinline__ void gather_block(const MlaArgs& a, const int* __restrict__ rows_s, uint8_t* kv_s, int g) {
  if constexpr (!FP8_PAGED) {
    // rows x 72 chunks of 16 bytes
#pragma unroll 4
    for (int q = g; q < kMlaBlk * 72; q += kMlaGatherThreads) {
      const int r = q / 72, cc = q - r * 72;
      const int p = cc >> 3, c = cc & 7;
      const int row = rows_s[r];
      const uint8_t* src = reinterpret_cast<const uint8_t*>(a.kv) + (int64_t)max(row, 0) * (kMlaDqk * 2) + cc * 16;
      cp_async16(kv_s + p * kMlaKPanelBytes + r * 128 + ((c ^ (r & 7)) << 4), src, row >= 0);
    }
    cp_async_wait_all();
  } else {
    // latent: rows x 32 chunks of 16 e4m3 -> two 16-byte bf16 chunks each; rope: rows x 8 chunks.
    // Every load of the block (rope, latent, scales) is issued before the first use: the cache does not
    // fit L2, and this way a block pays one DRAM round trip instead of three.
    constexpr int kRope = kMlaBlk * 8 / kMlaGatherThreads;     // rope chunks per thread
    uint4 rope[kRope];
#pragma unroll
    for (int u = 0; u < kRope; ++u) {
      const int q = g + u * kMlaGatherThreads;
      const int row = rows_s[q >> 3];
      rope[u] = make_uint4(0, 0, 0, 0);
      if (row >= 0) rope[u] = __ldg(reinterpret_cast<const uint4*>(a.cache + (int64_t)row * kLatentTokenBytes + kMlaDv + 16) + (q & 7));
    }
    constexpr int kBatch = 16;
    static_assert((kMlaBlk * 32) % (kMlaGatherThreads * kBatch) == 0, "latent chunks per thread must be a multiple of the batch");
    for (int q0 = g; q0 < kMlaBlk * 32; q0 += kMlaGatherThreads * kBatch) {
      uint4 raw[kBatch];
      float sc[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int q = q0 + u * kMlaGatherThreads;
        const int r = q >> 5, cc = q & 31;           // cc: 16-element chunk of the 512 latent dims
        const int row = rows_s[r];
        raw[u] = make_uint4(0, 0, 0, 0);
        sc[u] = 0.f;
        if (row >= 0) {
          const uint8_t* rec = a.cache + (int64_t)row * kLatentTokenBytes;
          raw[u] = __ldg(reinterpret_cast<const uint4*>(rec + cc * 16));
          sc[u] = __ldg(reinterpret_cast<const float*>(rec + kMlaDv) + (cc >> 3));
        }
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int q = q0 + u * kMlaGatherThreads;
        const int r = q >> 5, cc = q & 31;
        const uint32_t w[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
        uint32_t outw[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const __nv_fp8x2_storage_t pr = static_cast<__nv_fp8x2_storage_t>((w[i] >> (16 * hh)) & 0xffffu);
            const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(pr, __NV_E4M3);
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
            outw[i * 2 + hh] = pack_bf16x2(f.x * sc[u], f.y * sc[u]);
          }
        }
        const int d0 = cc * 16;                        // first latent dim of this chunk
        const int p = d0 >> 6, c = (d0 & 63) >> 3;     // panel, 16-byte chunk inside the 128-byte row (even)
        uint8_t* base = kv_s + p * kMlaKPanelBytes + r * 128;
        *reinterpret_cast<uint4*>(base + ((c ^ (r & 7)) << 4)) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
        *reinterpret_cast<uint4*>(base + (((c + 1) ^ (r & 7)) << 4)) = make_uint4(outw[4], outw[5], outw[6], outw[7]);
      }
    }
#pragma unroll
    for (int u = 0; u < kRope; ++u) {
      const int q = g + u * kMlaGatherThreads;
      const int r = q >> 3, c = q & 7;
      *reinterpret_cast<uint4*>(kv_s + 8 * kMlaKPanelBytes + r * 128 + ((c ^ (r & 7)) << 4)) = rope[u];
    }
  }
  fence_async_smem();          // make the panel writes visible to the tensor core's reads
}

template <bool FP8_PAGED>
__global__ void __launch_bounds__(kMlaThreads, 1)
sparse_mla_kernel(const __grid_constant__ CUtensorMap tmap_q, const MlaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                               // Q panels 5..8 [128 heads x 128 B]
  uint8_t* kv_s = q_s + kMlaQSmemBytes;              // KV buffers x 9 panels [Blk keys x 128 B]; first: staging of Q panels 0..4
  uint64_t* bars = reinterpret_cast<uint64_t*>(kv_s + kMlaBufs * kMlaKBytes);
  uint64_t* q_full = bars + 0;
  uint64_t* o_final = bars + 1;
  uint64_t* kv_full = bars + 2;                      // [2] gather -> MMA
  uint64_t* kv_free = bars + 4;                      // [2] P.V of the block finished: its KV buffer is free
  uint64_t* s_full = bars + 6;                       // [2] MMA -> softmax
  uint64_t* p_full = bars + 8;                       // [2] softmax -> MMA
  uint64_t* pv_done = bars + 10;                     // [2] P.V of block j finished: O is quiescent, P is free
  uint64_t* s_free = bars + 12;                      // softmax has read S into registers
  uint64_t* q_moved = bars + 13;                     // Q panels 0..4 are in tensor memory, the staging area is free
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 14);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_s = const_cast<int*>(abort_flag) + 1;
  int* rows_all = reinterpret_cast<int*>(kv_s + kMlaBufs * kMlaKBytes + 1024);   // [kMlaMaxK] row id per slot, -1 = empty

  const int t = blockIdx.x / a.n_split, split = blockIdx.x % a.n_split, vhalf = blockIdx.y, hg = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_per = ((a.K + a.n_split - 1) / a.n_split + kMlaBlk - 1) / kMlaBlk * kMlaBlk;   // slots per part
  const int k_lo = min(a.K, split * k_per), k_cnt = min(a.K, k_lo + k_per) - k_lo;
  const int32_t* idx_row = a.idx + (int64_t)t * a.K + k_lo;
  const int heads_here = min(128, a.H - hg * 128);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(o_final, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&kv_full[b], kMlaGatherThreads);
      mbar_init(&kv_free[b], 1);
      mbar_init(&s_full[b], 1);
      mbar_init(&p_full[b], 128);
      mbar_init(&pv_done[b], 1);
    }
    mbar_init(s_free, 128);
    mbar_init(q_moved, 128);
    *abort_flag = 0;
    *last_s = -1;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_q);
  }
  __syncthreads();
  {  // translate every slot to a row id once; the last non-empty slot decides the number of key blocks
    int last = -1;
    const int k_pad = (k_cnt + kMlaBlk - 1) / kMlaBlk * kMlaBlk;
    for (int j = threadIdx.x; j < k_pad; j += kMlaThreads) {
      int r = -1;
      const int pos = j < k_cnt ? idx_row[j] : -1;
      if (pos >= 0) {
        if (pos >= a.S_kv) {
          if (a.status) atomicCAS(a.status, kStatusOk, kStatusBadIndex);
        } else if constexpr (!FP8_PAGED) {
          r = pos;
        } else {
          const int phys = a.block_table[(int64_t)t * a.table_stride + pos / kLatentPage];
          if (phys >= 0 && (int64_t)(phys + 1) * kLatentPage <= a.num_phys_rows) r = phys * kLatentPage + pos % kLatentPage;
          else if (a.status) atomicCAS(a.status, kStatusOk, kStatusBadIndex);
        }
      }
      rows_all[j] = r;
      if (r >= 0) last = j;
    }
    if (last >= 0) atomicMax(last_s, last);
  }
  __syncthreads();
  const int nblk = (*last_s + kMlaBlk) / kMlaBlk;
  if (nblk == 0) {   // nothing selected: the output row is zero (a part: weight zero in the combine)
    if (threadIdx.x < 128 && threadIdx.x < heads_here) {
      if (a.n_split == 1) {
        uint4* o = reinterpret_cast<uint4*>(a.out + ((int64_t)t * a.H + hg * 128 + threadIdx.x) * kMlaDv + vhalf * kMlaDvHalf);
        for (int c = 0; c < kMlaDvHalf * 2 / 16; ++c) o[c] = make_uint4(0, 0, 0, 0);
      } else {
        const int64_t prow = (int64_t)blockIdx.x * a.H + hg * 128 + threadIdx.x;
        float4* o = reinterpret_cast<float4*>(a.part_o + prow * kMlaDv + vhalf * kMlaDvHalf);
        for (int c = 0; c < kMlaDvHalf / 4; ++c) o[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (vhalf == 0) a.part_lse[prow] = -CUDART_INF_F;
      }
    }
    return;
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, kMlaTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 4) {
    // ------------------------------- MMA issuer -------------------------------
    // Issue order: QK(0), then per block j: QK(j+1) (so the next scores are computed while
    // the softmax of block j runs), wait for P(j), PV(j).  MMAs complete in issue order.
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(1, 1, 0, 0, 128, kMlaBlk);
      constexpr uint32_t idesc_pv = umma_idesc(1, 1, 0, 1, 128, kMlaDvHalf);
      mbar_expect_tx(q_full, kMlaQBytes);
      for (int p = 0; p < kMlaPanels; ++p)          // panels 0..4 into the staging area, 5..8 to their place; x in 4-byte units
        tma_load_2d(p < kMlaQTmemPanels ? kv_s + p * kMlaQPanelBytes : q_s + (p - kMlaQTmemPanels) * kMlaQPanelBytes,
                    &tmap_q, p * 32, t * a.H + hg * 128, q_full);
      bool ok = mbar_wait(q_full, 0, abort_flag, a.status) && mbar_wait(q_moved, 0, abort_flag, a.status);
      // The issuing thread is a single lane: every instruction between two MMAs delays the tensor pipe
      // (a 64-key MMA takes ~48 cycles), so descriptors are built once and the 36 MMAs of a block are
      // straight-line code with compile-time offsets.
      uint64_t qdesc[kMlaQSmemPanels];
#pragma unroll
      for (int p = 0; p < kMlaQSmemPanels; ++p)
        qdesc[p] = umma_smem_desc(smem_u32(q_s + p * kMlaQPanelBytes), 16, 1024, kSwz128);
      uint64_t kdesc[kMlaBufs], vdesc_b[kMlaBufs];
#pragma unroll
      for (int b = 0; b < kMlaBufs; ++b) {
        kdesc[b] = umma_smem_desc(smem_u32(kv_s + b * kMlaKBytes), 16, 1024, kSwz128);
        vdesc_b[b] = umma_smem_desc(smem_u32(kv_s + b * kMlaKBytes + vhalf * 4 * kMlaKPanelBytes), kMlaKPanelBytes, 1024, kSwz128);
      }
      auto issue_qk = [&](int j) -> bool {
        const int kvb = j % kMlaBufs;
        if (!mbar_wait(&kv_full[kvb], (j / kMlaBufs) & 1, abort_flag, a.status)) return false;
        if (j > 0 && !mbar_wait(s_free, (j - 1) & 1, abort_flag, a.status)) return false;   // S of block j-1 was read
        tc_fence_after();
        const uint64_t kd0 = kMlaBufs == 1 ? kdesc[0] : (kvb ? kdesc[kMlaBufs - 1] : kdesc[0]);
#pragma unroll
        for (int p = 0; p < kMlaPanels; ++p) {
          const uint64_t kd = kd0 + uint64_t((p * kMlaKPanelBytes) >> 4);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            if (p < kMlaQTmemPanels)                 // A operand from tensor memory: no shared-memory read for Q
              umma_f16_ts(tmem + kColS, tmem + kColQ + p * 32 + 8 * ks, kd + 2 * ks, idesc_qk, (p | ks) != 0);
            else
              umma_f16_ss(tmem + kColS, qdesc[p < kMlaQTmemPanels ? 0 : p - kMlaQTmemPanels] + 2 * ks, kd + 2 * ks, idesc_qk, 1);
          }
        }
        umma_commit(s_full);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < nblk && ok; ++j) {
        const int b = j & 1, kvb = j % kMlaBufs;
        // next scores first only if their keys have already landed; never stall P.V behind a gather
        bool qk_done = j + 1 >= nblk;
        if (!qk_done && kMlaBufs > 1 && mbar_try_wait(&kv_full[(j + 1) % kMlaBufs], ((j + 1) / kMlaBufs) & 1)) {
          ok = issue_qk(j + 1);
          qk_done = true;
        }
        if (!ok) break;
        ok = mbar_wait(p_full, j & 1, abort_flag, a.status);
        if (!ok) break;
        tc_fence_after();
        const uint64_t vdesc = kMlaBufs == 1 ? vdesc_b[0] : (kvb ? vdesc_b[kMlaBufs - 1] : vdesc_b[0]);
#pragma unroll
        for (int ks = 0; ks < kMlaBlk / 16; ++ks)     // 16 keys per step: 16 rows x 128 B further into each panel
          umma_f16_ts(tmem + kColO, tmem + kColP + 8 * ks, vdesc + ks * (2048 >> 4), idesc_pv,
                      (j | ks) != 0);
        umma_commit(&kv_free[kvb]);
        umma_commit(&pv_done[j & 1]);
        if (j == nblk - 1) umma_commit(o_final);
        if (!qk_done) ok = issue_qk(j + 1);
      }
    }
  } else if (warp >= 5) {
    // --------------------------------- gather ---------------------------------
    const int g = threadIdx.x - 160;
    mbar_wait(q_moved, 0, abort_flag, a.status);      // the buffers hold Q panels until they are in tensor memory
    for (int j = 0; j < nblk; ++j) {
      const int kvb = j % kMlaBufs;
      mbar_wait(&kv_free[kvb], ((j / kMlaBufs) & 1) ^ 1, abort_flag, a.status);
      gather_block<FP8_PAGED>(a, rows_all + j * kMlaBlk, kv_s + kvb * kMlaKBytes, g);
      mbar_arrive(&kv_full[kvb]);
      if (*abort_flag) break;
    }
  } else {
    // ------------------------- softmax and output (thread = head) -------------------------
    const int row = threadIdx.x;                       // 0..127 = TMEM lane
    const uint32_t t_row = tmem + (uint32_t(warp * 32) << 16);
    float m = -CUDART_INF_F, l = 0.f;
    bool ok = __all_sync(0xffffffffu, mbar_wait(q_full, 0, abort_flag, a.status));
    if (ok) {
      // this head's row of Q panels 0..4: swizzled shared memory -> packed bf16 pairs in tensor memory
#pragma unroll 1
      for (int p = 0; p < kMlaQTmemPanels; ++p) {
        uint32_t qv[32];
        const uint8_t* src = kv_s + p * kMlaQPanelBytes + row * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const uint4 w = *reinterpret_cast<const uint4*>(src + ((c ^ (row & 7)) << 4));
          qv[4 * c + 0] = w.x; qv[4 * c + 1] = w.y; qv[4 * c + 2] = w.z; qv[4 * c + 3] = w.w;
        }
        tmem_st32(t_row + kColQ + p * 32, qv);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(q_moved);
    }
    for (int j = 0; j < nblk && ok; ++j) {
      ok = __all_sync(0xffffffffu, mbar_wait(s_full, j & 1, abort_flag, a.status));
      if (!ok) break;
      tc_fence_after();
      uint32_t sv[kMlaBlk];
#pragma unroll
      for (int c = 0; c < kMlaBlk; c += 32)
        tmem_ld32(t_row + kColS + c, *reinterpret_cast<uint32_t(*)[32]>(sv + c));
      tmem_wait_ld();
      tc_fence_before();
      mbar_arrive(s_free);                             // the next block's scores may overwrite S now
      float s[kMlaBlk];                                // raw scores; the (positive) scale is folded into the exponent's FMA
      float bmax = -CUDART_INF_F;
      const int* vrow = rows_all + j * kMlaBlk;
#pragma unroll
      for (int i = 0; i < kMlaBlk; ++i) {
        s[i] = vrow[i] >= 0 ? __uint_as_float(sv[i]) : -CUDART_INF_F;
        bmax = fmaxf(bmax, s[i]);
      }
      bmax *= a.scale_log2e;
      const float m_new = fmaxf(m, bmax);
      const bool grow = m_new - m > 8.f;               // also true when m is still -inf and m_new is finite
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = grow ? fast_exp2(m - m_new) : 1.f;
        if (grow) m = m_new;
        l *= alpha;
        if (j > 0) {
          // O must be quiescent: P.V of the previous block has to be complete
          ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, a.status));
          if (!ok) break;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < kMlaDvHalf; c += 32) {
            uint32_t ov[32];
            tmem_ld32(t_row + kColO + c, ov);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
            tmem_st32(t_row + kColO + c, ov);
          }
        }
      }
      const float m_eff = (m == -CUDART_INF_F) ? 0.f : m;
      uint32_t pk[kMlaBlk / 2];
      float psum = 0.f;
#pragma unroll
      for (int i = 0; i < kMlaBlk; i += 2) {
        const float p0 = fast_exp2(fmaf(s[i], a.scale_log2e, -m_eff)), p1 = fast_exp2(fmaf(s[i + 1], a.scale_log2e, -m_eff));
        psum += p0 + p1;
        pk[i >> 1] = pack_bf16x2(p0, p1);
      }
      l += psum;
      if (j > 0) {                                     // P is single-buffered: P.V of the previous block must be done
        ok = __all_sync(0xffffffffu, mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, a.status));
        if (!ok) break;
        tc_fence_after();
      }
#pragma unroll
      for (int c = 0; c < kMlaBlk / 2; c += 16)
        tmem_st16(t_row + kColP + c, *reinterpret_cast<uint32_t(*)[16]>(pk + c));
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(o_final, 0, abort_flag, a.status));
    if (ok) {
      tc_fence_after();
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = a.out + ((int64_t)t * a.H + hg * 128 + row) * kMlaDv + vhalf * kMlaDvHalf;
      const int64_t prow = (int64_t)blockIdx.x * a.H + hg * 128 + row;
      if (a.n_split > 1 && vhalf == 0 && row < heads_here)
        a.part_lse[prow] = l > 0.f ? m + log2f(l) : -CUDART_INF_F;
#pragma unroll 1
      for (int c = 0; c < kMlaDvHalf; c += 32) {
        uint32_t ov[32];
        tmem_ld32(t_row + kColO + c, ov);
        tmem_wait_ld();
        if (row < heads_here && a.n_split > 1) {
          float4* po = reinterpret_cast<float4*>(a.part_o + prow * kMlaDv + vhalf * kMlaDvHalf + c);
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            po[i >> 2] = make_float4(__uint_as_float(ov[i]) * inv, __uint_as_float(ov[i + 1]) * inv,
                                     __uint_as_float(ov[i + 2]) * inv, __uint_as_float(ov[i + 3]) * inv);
        } else if (row < heads_here) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(ov[i + 0]) * inv, __uint_as_float(ov[i + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(ov[i + 2]) * inv, __uint_as_float(ov[i + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(ov[i + 4]) * inv, __uint_as_float(ov[i + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(ov[i + 6]) * inv, __uint_as_float(ov[i + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c + i) = w;
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem, kMlaTmemCols);
  }
}

// out[t,h,:] = sum_s 2^(lse_s - M) o_s / sum_s 2^(lse_s - M): merges the parts of a split slot list.
__global__ void __launch_bounds__(128) sparse_mla_combine_kernel(const MlaArgs a) {
  const int t = blockIdx.x, h = blockIdx.y;
  float wgt[16];
  float mx = -CUDART_INF_F, den = 0.f;
  for (int sp = 0; sp < a.n_split; ++sp) {
    wgt[sp] = a.part_lse[((int64_t)t * a.n_split + sp) * a.H + h];
    mx = fmaxf(mx, wgt[sp]);
  }
  for (int sp = 0; sp < a.n_split; ++sp) {
    wgt[sp] = (mx == -CUDART_INF_F) ? 0.f : exp2f(wgt[sp] - mx);
    den += wgt[sp];
  }
  const float inv = den > 0.f ? 1.f / den : 0.f;
  const int d = threadIdx.x * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int sp = 0; sp < a.n_split; ++sp) {
    const float4 v = *reinterpret_cast<const float4*>(a.part_o + (((int64_t)t * a.n_split + sp) * a.H + h) * kMlaDv + d);
    acc.x += wgt[sp] * v.x; acc.y += wgt[sp] * v.y; acc.z += wgt[sp] * v.z; acc.w += wgt[sp] * v.w;
  }
  uint2 o;
  o.x = pack_bf16x2(acc.x * inv, acc.y * inv);
  o.y = pack_bf16x2(acc.z * inv, acc.w * inv);
  *reinterpret_cast<uint2*>(a.out + ((int64_t)t * a.H + h) * kMlaDv + d) = o;
}

int make_tmap_2d_bytes(CUtensorMap* m, const void* base, uint64_t rows, uint64_t inner_bytes, uint64_t row_pitch,
                       uint32_t box_bytes, uint32_t box_rows);

template <bool FP8_PAGED>
static int launch_mla(const void* q, const MlaArgs& a, cudaStream_t stream) {
  if (a.T == 0 || a.H == 0) return DSA_OK;
  CUtensorMap tq;
  int rc = make_tmap_2d_bytes(&tq, q, (uint64_t)a.T * a.H, kMlaDqk * 2, kMlaDqk * 2, 128, 128);
  if (rc) return rc;
  auto kern = sparse_mla_kernel<FP8_PAGED>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmemBytes) != cudaSuccess)
    return set_error(DSA_ERR_CUDA, "sparse_mla: cannot raise dynamic shared memory to %d", kMlaSmemBytes);
  const dim3 grid(a.T * a.n_split, 2, (a.H + 127) / 128);
  kern<<<grid, kMlaThreads, kMlaSmemBytes, stream>>>(tq, a);
  if (a.n_split > 1) sparse_mla_combine_kernel<<<dim3(a.T, a.H), 128, 0, stream>>>(a);
  return check_launch("sparse_mla");
}

int sparse_mla_prefill_launch(const void* q, const void* kv, const int32_t* idx, void* out, int T, int H, int S_kv,
                              int K, float scale, int32_t* status, cudaStream_t stream) {
  MlaArgs a{};
  a.kv = static_cast<const __nv_bfloat16*>(kv);
  a.idx = idx;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.T = T; a.H = H; a.K = K; a.S_kv = S_kv;
  a.scale_log2e = scale * 1.4426950408889634f;
  a.status = status;
  a.n_split = 1;
  return launch_mla<false>(q, a, stream);
}

// With few queries (decode) one CTA pair per query leaves most SMs idle and walks 2048 slots serially:
// cut the slot list into parts of >= 256 slots while the grid still fits the GPU in one wave.  More
// parts than that lose: every part pays the CTA set-up again and writes an fp32 partial output that
// the combine kernel reads back (batch 64 at 8 parts: 233 us; unsplit: 140 us; batch 8: 36 vs 116 us).
int mla_decode_splits(int B, int H, int K) {
  const int ctas = B * 2 * ((H + 127) / 128);
  int ns = 1;
  while (ns < 8 && ctas * ns * 2 <= sm_count() && K / (ns * 2) >= 256) ns *= 2;
  return ns;
}
size_t mla_decode_workspace_bytes(int B, int H, int K) {
  const int ns = mla_decode_splits(B, H, K);
  if (ns <= 1) return 0;
  return (size_t)B * ns * H * (kMlaDv + 1) * sizeof(float);
}

int sparse_mla_decode_launch(const void* q, const void* cache, const int32_t* block_table, int64_t table_stride,
                             const int32_t* idx, void* out, int B, int H, int K, int num_pages, int max_ctx,
                             float scale, void* workspace, size_t workspace_bytes, int32_t* status,
                             cudaStream_t stream) {
  MlaArgs a{};
  a.n_split = mla_decode_splits(B, H, K);
  if (a.n_split > 1 && workspace && workspace_bytes >= mla_decode_workspace_bytes(B, H, K)) {
    a.part_o = static_cast<float*>(workspace);
    a.part_lse = a.part_o + (size_t)B * a.n_split * H * kMlaDv;
  } else {
    a.n_split = 1;
  }
  a.cache = static_cast<const uint8_t*>(cache);
  a.block_table = block_table;
  a.table_stride = table_stride;
  a.idx = idx;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.T = B; a.H = H; a.K = K; a.S_kv = max_ctx;
  a.num_phys_rows = num_pages * kLatentPage;
  a.scale_log2e = scale * 1.4426950408889634f;
  a.status = status;
  return launch_mla<true>(q, a, stream);
}

}  // namespace dsa
