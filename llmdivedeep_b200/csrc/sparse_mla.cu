// Token-sparse MLA attention on sm_100a (MQA over the shared 576-dim latent KV, 512-dim V):
//   o[t, h, :] = sum_j softmax_j(scale * q[t, h, :] . kv[idx[t, j], :]) * kv[idx[t, j], :512]
// Takes the place of the block-sparse stand-in the reference reaches through
// register_sparse_fa() (sparse_attn/DSA.py:208-249); the reference itself has no sparse-MLA
// kernel, no latent cache and no decode path (sparse_attn/DSA.py:475-477).
//
// One CLUSTER of two CTAs per (query token, group of up to 128 heads).  The 576-dim row splits
// into nine 64-dim panels: eight latent panels (they are also V) and the rope panel.  CTA c of the
// pair owns latent panels 4c..4c+3 -- its half of V -- and half of the rope panel's contraction:
//   * it gathers only those five panels of every selected row (40 KB per 64-key block instead of
//     72 KB, four blocks in flight): TMA tile::gather4 from the bf16 KV, or -- for the paged FP8
//     latent cache of decode -- cp.async of the raw rows into two shared-memory stages, two blocks
//     ahead, and a shared -> shared conversion e4m3 x group scale -> bf16 (three KV buffers; the
//     fourth one's space holds the raw stages);
//   * its five Q panels live in tensor memory as the A operand, so Q.K^T reads no shared memory for
//     Q, and it computes a PARTIAL score tile S_c = Q_c K_c^T (18 tcgen05.mma kind::f16 of N = 64
//     instead of 36: back-to-back MMAs into one accumulator complete ~130 cycles apart whatever
//     their N, and that chain is what bounded the kernel that computed all of S in both CTAs);
//   * the two partial tiles ([128 heads x 64 keys], rounded to fp16: 16 KB) are exchanged through
//     distributed shared memory with one bulk copy per block and direction, double-buffered, issued
//     by a warp of its own (the copy queues behind the gather on the SM's TMA unit, and the lane that
//     issues it stalls for hundreds of cycles);
//     S = fp16(S_0) + fp16(S_1), summed in fp32, is the same number, bit for bit, on both sides, so
//     both run the same online softmax and hold the same P, which is the A operand (from tensor
//     memory) of O_c += P V_c with the gathered panels read through an MN-major descriptor.  fp16
//     partials carry 11 significant bits each: an error below the bf16 rounding of P for scores
//     within +-65504; they halve the copy, which shares the TMA unit with the gather.
// O is rescaled in tensor memory only when the running maximum grows by more than 8 (log2 units).
//
// Roles: warps 0-7 exchange + softmax + output, warp 8 lane 0 MMA issuer (warp 8 owns the TMEM
// allocation), warps 9-12 gather, warp 13 lane 0 issues the tile copies.  A thread of warps 0-7 owns one head (TMEM lane) and HALF of a
// block's keys (warp w: lanes 32 (w % 4).., keys 32 (w / 4)..): with one thread per head and all 64
// keys the softmax, not the tensor pipe, paced the kernel.  Per block n such a warp first moves its
// part of the partial scores of block n out of tensor memory and on to the peer, then
// runs the softmax of block n-1, whose peer tile arrived while the scores of block n were computed;
// the two threads of a head agree on the block maximum through shared memory (rounded up to bf16:
// any common reference point is exact for a softmax) and keep separate partial row sums.
// Every wait is bounded (dsa_common.cuh); the two CTAs leave together through a cluster barrier.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <math_constants.h>

#include "dsa_common.cuh"
#include "dsa_host.h"

namespace dsa {

constexpr int kMlaDqk = 576;
constexpr int kMlaDv = 512;
constexpr int kMlaDvHalf = 256;
constexpr int kMlaBlk = 64;                        // keys per block
constexpr int kMlaPanels = 5;                      // panels per CTA: four latent (its V half) + rope
constexpr int kMlaBufs = 4;                        // KV buffers in shared memory
constexpr int kMlaQPanelBytes = 128 * 128;         // 128 heads x 128 B
constexpr int kMlaKPanelBytes = kMlaBlk * 128;     // 64 keys x 128 B
constexpr int kMlaKBytes = kMlaPanels * kMlaKPanelBytes;      // 40960 per buffer
constexpr int kMlaXBytes = 128 * kMlaBlk * 2;      // one partial score tile, fp16: 16384
constexpr int kMlaXStages = 2;                     // exchange buffers (send and receive) per CTA
constexpr int kMlaRing = 2;                        // row-id slots: read only by the gather warps, inside the call that staged them
constexpr int kMlaMaskRing = 8;                    // validity masks (64 bits per block) for the softmax: >= blocks in flight
// Gather warps: four for prefill (the TMA unit, not the issuing warps, bounds that gather: more do not help), eight for
// decode, where the warps convert the FP8 rows themselves and four of them take longer per block than the score chain.
template <bool FP8_PAGED>
struct MlaCfg {
  static constexpr int kGatherWarps = FP8_PAGED ? 8 : 4;
  static constexpr int kGatherThreads = kGatherWarps * 32;
  static constexpr int kCopyWarp = 9 + kGatherWarps;          // issues the copies of the partial score tiles
  static constexpr int kThreads = 288 + kGatherThreads + 32;
};
constexpr int kMlaBarBytes = 256;                  // mbarriers and a few words
constexpr int kMlaPairBytes = 2 * 2 * 128 * 2;     // block maxima of the two key halves, double-buffered, bf16 (reused for the row sums, fp32)
constexpr int kMlaSmemBytes = 1024 + kMlaBufs * kMlaKBytes + 2 * kMlaXStages * kMlaXBytes + kMlaBarBytes +
                              kMlaRing * kMlaBlk * 4 + kMlaMaskRing * 2 * 4 + kMlaPairBytes;
static_assert(kMlaSmemBytes <= 232448, "shared memory budget of one CTA");
static_assert(2 * kMlaKBytes == kMlaPanels * kMlaQPanelBytes, "Q staging: the five panels fill the last two KV buffers");
constexpr int kLatentTokenBytes = 656;             // 512 e4m3 + 4 fp32 scales + 64 bf16 rope
constexpr int kLatentPage = 64;
// tensor-memory columns: O 256, S 64, P 32, Q 5 x 32
constexpr uint32_t kColO = 0, kColS = 256, kColP = kColS + kMlaBlk, kColQ = kColP + kMlaBlk / 2, kMlaTmemCols = 512;
static_assert(kColQ + kMlaPanels * 32 <= kMlaTmemCols, "tensor memory budget");

struct MlaArgs {
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
  int tma_out;                    // the output tensor map is valid: full 128-head groups leave through TMA stores
};

// ---- cluster helpers ----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t mapa_u32(uint32_t addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
  return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_wait() {
  cluster_arrive();
  cluster_wait();
}
// Arrive on the peer's barrier to say "I have READ the tile".  Relaxed on purpose: a release at cluster scope
// costs a memory fence of thousands of cycles per block, and nothing written by this thread has to become
// visible -- the loads it orders were consumed by arithmetic that issued before this instruction, so they
// have returned.
__device__ __forceinline__ void mbar_arrive_remote_relaxed(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// this CTA's shared memory -> the peer's, completion counted on the peer's mbarrier.  Tried instead and dropped:
// 16-byte st.async from registers straight into the peer's buffer (no staging, no acknowledgement with four receive
// stages, but the stores drain at about half the rate of this copy and hold up the warps that issue them), and part
// of the row gather by cp.async -- the load/store path moves rows no faster than gather4 and slows the softmax.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_cluster, const void* src, uint32_t bytes, uint32_t bar_cluster) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst_cluster), "r"(smem_u32(src)), "r"(bytes), "r"(bar_cluster) : "memory");
}
// four rows of a [rows, 576] bf16 tensor map (box 64 elements x 1 row), one 64-dim panel each -> 512 B of shared memory
__device__ __forceinline__ void tma_gather4(void* dst, const void* tmap, int x, int r0, int r1, int r2, int r3, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.tile::gather4.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "r"(smem_u32(bar))
      : "memory");
}

// one [rows x 128 B] panel, shared memory (128-B swizzle) -> global, tracked by the thread's bulk group
__device__ __forceinline__ void tma_store_2d(const void* tmap, const void* src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
               ::"l"(reinterpret_cast<uint64_t>(tmap)), "r"(x), "r"(y), "r"(smem_u32(src)) : "memory");
}
__device__ __forceinline__ void bulk_commit_and_wait_read() {      // shared memory may be reused / released afterwards
  asm volatile("cp.async.bulk.commit_group;\n\tcp.async.bulk.wait_group.read 0;" ::: "memory");
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
__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {      // out-of-range values saturate to +-65504
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// fp32 sums of two fp16 pairs, exact before the one rounding of each sum (mixed-precision adds: no separate conversions)
__device__ __forceinline__ float2 add_f16x2_f32(uint32_t a, uint32_t b) {
  float2 r;
  asm("{\n\t.reg .b16 al, ah, bl, bh;\n\t.reg .f32 t0, t1;\n\t"
      "mov.b32 {al, ah}, %2;\n\tmov.b32 {bl, bh}, %3;\n\t"
      "add.rn.f32.f16 t0, al, 0f00000000;\n\tadd.rn.f32.f16 t1, ah, 0f00000000;\n\t"
      "add.rn.f32.f16 %0, bl, t0;\n\tadd.rn.f32.f16 %1, bh, t1;\n\t}"
      : "=f"(r.x), "=f"(r.y) : "r"(a), "r"(b));
  return r;
}
// A partial score tile is [2 key halves][128 heads][32 keys] fp16: 64 bytes per thread of warps 0-7, 2 KB contiguous per
// warp.  16-byte chunk c (0..3) of a thread's 64 bytes: the chunk order is rotated by the lane pair so that the eight lanes
// of a quarter-warp hit different banks.
__device__ __forceinline__ int xchg_off(int half, int row, int c) {
  return half * (kMlaXBytes / 2) + row * 64 + (((c ^ (row >> 1)) & 3) << 4);
}
// fp32 -> bf16 bits, rounded towards +infinity
__device__ __forceinline__ uint32_t bf16_bits_round_up(float x) {
  const uint32_t b = __float_as_uint(x);
  return ((b >> 31) || (b & 0x7fffffffu) >= 0x7f800000u) ? (b >> 16) : ((b + 0xffffu) >> 16);
}

// ---- paged FP8 latent cache (decode) ------------------------------------------------------------
// A block's rows travel global -> shared memory as raw bytes with cp.async (asynchronous, two blocks ahead, no registers
// held), and are converted shared -> shared.  A raw row is this CTA's 256 e4m3 values followed by the row's four scales.
constexpr int kRawRow = kMlaDvHalf + 16;
constexpr int kRawStage = kMlaBlk * kRawRow;         // 17408 bytes
static_assert(2 * kRawStage <= kMlaKBytes, "the two raw stages take the place of the fourth KV buffer");
__device__ __forceinline__ void cp_async_16(void* dst, const void* src, int src_bytes) {      // src_bytes 0: zero fill
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// e4m3 -> bf16 with the per-128 group scale, raw stage -> this CTA's four latent panels of a KV buffer.  Thread g of
// GT gather threads; an empty slot was zero-filled (values and scales), so it converts to zeros.  (Tried and dropped:
// decode's latent MMAs in fp16, so that e4m3 x scale is one conversion and one packed multiply per two values -- a third
// of the instructions, and 9 % slower end to end: the conversion is not what paces the decode kernel.)
template <int GT>
__device__ __forceinline__ void convert_block(const uint8_t* stage, uint8_t* kv_s, int g, int cta) {
  constexpr int kLat = kMlaBlk * 16 / GT;          // 16-value chunks per thread
#pragma unroll
  for (int u = 0; u < kLat; ++u) {
    const int q = g + u * GT;
    const int r = q >> 4, cc = q & 15;              // row, chunk inside this CTA's 256 latent dims
    const uint4 raw = *reinterpret_cast<const uint4*>(stage + r * kRawRow + cc * 16);
    const float sc = *reinterpret_cast<const float*>(stage + r * kRawRow + kMlaDvHalf + (cta * 2 + (cc >> 3)) * 4);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t outw[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const __nv_fp8x2_storage_t pr = static_cast<__nv_fp8x2_storage_t>((w[i >> 1] >> (16 * (i & 1))) & 0xffffu);
      const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(pr, __NV_E4M3);
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
      outw[i] = pack_bf16x2(f.x * sc, f.y * sc);
    }
    const int p = cc >> 2, c = (cc & 3) * 2;        // local panel, 16-byte chunk inside the 128-byte row (even)
    uint8_t* base = kv_s + p * kMlaKPanelBytes + r * 128;
    *reinterpret_cast<uint4*>(base + ((c ^ (r & 7)) << 4)) = make_uint4(outw[0], outw[1], outw[2], outw[3]);
    *reinterpret_cast<uint4*>(base + (((c + 1) ^ (r & 7)) << 4)) = make_uint4(outw[4], outw[5], outw[6], outw[7]);
  }
}

template <bool FP8_PAGED>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(MlaCfg<FP8_PAGED>::kThreads, 1)
sparse_mla_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                  const __grid_constant__ CUtensorMap tmap_o, const MlaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  constexpr int NB = FP8_PAGED ? kMlaBufs - 1 : kMlaBufs;      // KV buffers in use (decode: the fourth holds the raw stages)
  // Whether a warp tells the peer that it has read a received tile before the peer may send into that stage again.  The
  // order of a warp's work makes the acknowledgement redundant (see where the tile is written); prefill runs 1.3 % faster
  // without it, decode -- at 96 registers per thread -- 4 % slower (the variant without it spills), so decode keeps it.
  constexpr bool kAck = FP8_PAGED;
  constexpr int kMlaGatherWarps = MlaCfg<FP8_PAGED>::kGatherWarps, kMlaGatherThreads = MlaCfg<FP8_PAGED>::kGatherThreads;
  constexpr int kMlaCopyWarp = MlaCfg<FP8_PAGED>::kCopyWarp, kMlaThreads = MlaCfg<FP8_PAGED>::kThreads;
  uint8_t* kv_s = smem;                                        // four buffers x five panels [64 keys x 128 B]
  uint8_t* send_s = kv_s + kMlaBufs * kMlaKBytes;              // [2] this CTA's partial score tiles
  uint8_t* recv_s = send_s + kMlaXStages * kMlaXBytes;         // [2] the peer's
  uint64_t* bars = reinterpret_cast<uint64_t*>(recv_s + kMlaXStages * kMlaXBytes);
  uint64_t* q_full = bars + 0;
  uint64_t* q_moved = bars + 1;                      // Q is in tensor memory, its staging areas are free
  uint64_t* o_final = bars + 2;
  uint64_t* s_full = bars + 3;                       // MMA -> warps 0-7
  uint64_t* s_free = bars + 4;                       // warps 0-7 have read S into registers
  uint64_t* p_full = bars + 5;                       // softmax -> MMA
  uint64_t* pv_done = bars + 6;                      // P.V of a block finished: O is quiescent, P is free
  uint64_t* send_full = bars + 7;                    // [2] this CTA's partial tile is in send_s[stage]
  uint64_t* recv_full = bars + 9;                    // [2] the peer's partial tile has landed in recv_s[stage]
  uint64_t* xchg_free = bars + 11;                   // [2] the peer has read what this CTA sent into that stage
  uint64_t* kv_full = bars + 13;                     // [4] gather -> MMA
  uint64_t* kv_free = bars + 17;                     // [4] P.V of the block finished: its KV buffer is free
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* last_s = const_cast<int*>(abort_flag) + 1;
  int* ring = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(bars) + kMlaBarBytes);     // [kMlaRing][64] row id per slot, -1 = empty
  uint32_t* masks = reinterpret_cast<uint32_t*>(ring + kMlaRing * kMlaBlk);        // [kMlaMaskRing][2] bit s = slot s of the block is in use
  uint8_t* pair_s = reinterpret_cast<uint8_t*>(masks + kMlaMaskRing * 2);          // what the two threads of a head tell each other

  const int cta = blockIdx.x & 1, peer = cta ^ 1;              // rank in the cluster = V half = contraction part
  const int unit = blockIdx.x >> 1;
  const int t = unit / a.n_split, split = unit % a.n_split, hg = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int k_per = ((a.K + a.n_split - 1) / a.n_split + kMlaBlk - 1) / kMlaBlk * kMlaBlk;   // slots per part
  const int k_lo = min(a.K, split * k_per), k_cnt = min(a.K, k_lo + k_per) - k_lo;
  const int32_t* idx_row = a.idx + (int64_t)t * a.K + k_lo;
  const int heads_here = min(128, a.H - hg * 128);
  // the five Q panels wait in the last two KV buffers for their move into tensor memory
  auto q_stage = [&](int lp) -> uint8_t* { return kv_s + (NB - 2) * kMlaKBytes + lp * kMlaQPanelBytes; };

  // ---- set-up, arranged so that nothing waits for anything it does not need ------------------------------------
  // every thread requests its share of the slot list first (the scan below decides the number of key blocks) ...
  constexpr int kScan = 8;
  int pos[kScan];
#pragma unroll
  for (int u = 0; u < kScan; ++u) {
    const int j = threadIdx.x + u * kMlaThreads;
    pos[u] = j < k_cnt ? __ldg(idx_row + j) : -1;
  }
  // ... while warp 0 initialises the barriers (one per lane) and sends for Q (one panel per lane) and warp 8 allocates
  // tensor memory
  if (warp == 0) {
    if (lane < 21) {
      const uint32_t count = (lane == 1 || lane == 4 || lane == 5) ? 8u             // q_moved, s_free, p_full: lane 0 of warps 0-7
                             : (lane == 7 || lane == 8) ? 8u                         // send_full: lane 0 of warps 0-7
                             : (lane == 11 || lane == 12) ? 8u                       // xchg_free: lane 0 of the peer's warps 0-7
                             : (lane >= 13 && lane <= 16) ? (FP8_PAGED ? uint32_t(kMlaGatherThreads) : uint32_t(kMlaGatherWarps))
                                                          : 1u;                      // q_full, o_final, s_full, pv_done, recv_full, kv_free
      mbar_init(bars + lane, count);
      mbar_fence_init();
    }
    if (lane == 0) {
      *abort_flag = 0;
      *last_s = -1;
    }
    __syncwarp();
    if (lane == 0) mbar_expect_tx(q_full, kMlaPanels * kMlaQPanelBytes);
    __syncwarp();
    // Q is on its way before anything else happens: into this CTA's own shared memory, counted on its own barrier
    if (lane < kMlaPanels)                             // x in 4-byte units: 32 per panel
      tma_load_2d(q_stage(lane), &tmap_q, (lane < 4 ? cta * 4 + lane : 8) * 32, t * a.H + hg * 128, q_full);
    if (lane == kMlaPanels && !FP8_PAGED) tma_prefetch_desc(&tmap_kv);
    if (lane == kMlaPanels + 1 && a.tma_out) tma_prefetch_desc(&tmap_o);
  } else if (warp == 8) {
    tmem_alloc(tmem_slot, kMlaTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  {  // the last usable slot decides the number of key blocks (the same number in both CTAs of the pair)
    int last = -1;
#pragma unroll
    for (int u = 0; u < kScan; ++u)
      if (pos[u] >= 0 && pos[u] < a.S_kv) last = threadIdx.x + u * kMlaThreads;
    for (int j = threadIdx.x + kScan * kMlaThreads; j < k_cnt; j += kMlaThreads) {      // slot lists beyond 3584: rare
      const int p = idx_row[j];
      if (p >= 0 && p < a.S_kv) last = j;
    }
    if (last >= 0) atomicMax(last_s, last);
  }
  __syncthreads();
  const int nblk = (*last_s + kMlaBlk) / kMlaBlk;
  if (nblk == 0) {   // nothing selected: the output row is zero (a part: weight zero in the combine); no cluster traffic yet
    if (threadIdx.x < 128 && threadIdx.x < heads_here) {
      if (a.n_split == 1) {
        uint4* o = reinterpret_cast<uint4*>(a.out + ((int64_t)t * a.H + hg * 128 + threadIdx.x) * kMlaDv + cta * kMlaDvHalf);
        for (int c = 0; c < kMlaDvHalf * 2 / 16; ++c) o[c] = make_uint4(0, 0, 0, 0);
      } else {
        const int64_t prow = (int64_t)unit * a.H + hg * 128 + threadIdx.x;
        float4* o = reinterpret_cast<float4*>(a.part_o + prow * kMlaDv + cta * kMlaDvHalf);
        for (int c = 0; c < kMlaDvHalf / 4; ++c) o[c] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (cta == 0) a.part_lse[prow] = -CUDART_INF_F;
      }
    }
    // an index that is out of range is still reported
    for (int j = threadIdx.x; j < k_cnt; j += kMlaThreads)
      if (idx_row[j] >= a.S_kv && a.status) atomicCAS(a.status, kStatusOk, kStatusBadIndex);
    if (threadIdx.x == 0) mbar_wait(q_full, 0, abort_flag, a.status);     // the Q copy must have landed before the CTA goes
    if (warp == 8) tmem_dealloc(*tmem_slot, kMlaTmemCols);
    return;
  }
  const uint32_t tmem = *tmem_slot;
  // The peer's barriers must be initialised before anything is sent to it.  Every thread arrives here; the warps that
  // talk to the peer (0-7, copy) wait before their first remote access, the others only before they leave, so that the
  // round trip through the cluster barrier is off the path to the first MMA.
  cluster_arrive();

  if (warp == 8) {
    // ------------------------------- MMA issuer -------------------------------
    // The partial scores of a block travel to the peer and through the softmax while the next blocks are scored: P.V of a
    // block is issued about two blocks after its scores.  MMAs complete in issue order.
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc(1, 1, 0, 0, 128, kMlaBlk);
      constexpr uint32_t idesc_pv = umma_idesc(1, 1, 0, 1, 128, kMlaDvHalf);
      bool ok = mbar_wait(q_moved, 0, abort_flag, a.status);
      uint64_t kdesc[kMlaBufs], vdesc[kMlaBufs];
#pragma unroll
      for (int b = 0; b < kMlaBufs; ++b) {
        kdesc[b] = umma_smem_desc(smem_u32(kv_s + b * kMlaKBytes), 16, 1024, kSwz128);
        vdesc[b] = umma_smem_desc(smem_u32(kv_s + b * kMlaKBytes), kMlaKPanelBytes, 1024, kSwz128);
      }
      auto pick = [&](const uint64_t (&d)[kMlaBufs], int b) { return b == 0 ? d[0] : b == 1 ? d[1] : b == 2 ? d[2] : d[3]; };
      const uint32_t rope_ks = 2 * cta;              // this CTA's two K-steps of the rope panel
      // P.V of block j: four MMAs (N = 256) and the commits that release the block's KV buffer, P and O.  They go as a
      // group: alternated one by one with the MMAs of a score chain they cost far more (167 ms against 116 for the 128K
      // prefill).  With A in tensor memory every MMA of this kernel costs its full ~137-cycle latency whether or not it
      // depends on the one before (sixteen independent N = 64 MMAs in place of these four: +137 cycles each), so the
      // block time is the number of MMA instructions, 18 + 4, times that.
      auto pv_mmas = [&](int j) {
        tc_fence_after();
        const uint64_t vd = pick(vdesc, j % NB);
#pragma unroll
        for (int ks = 0; ks < kMlaBlk / 16; ++ks)     // 16 keys per step: 16 rows x 128 B further into each panel
          umma_f16_ts(tmem + kColO, tmem + kColP + 8 * ks, vd + ks * (2048 >> 4), idesc_pv, (j | ks) != 0);
        umma_commit(&kv_free[j % NB]);
        umma_commit(pv_done);
        if (j == nblk - 1) umma_commit(o_final);
      };
      // Partial scores of block i.  The 18 MMAs form one dependent chain (about 130 cycles apart), so the tensor pipe
      // idles three quarters of the time: P.V of block `pv`, if its P arrives while this chain is issued, is slipped in
      // at the next panel boundary.
      int qk = 0, pv = 0;                              // next block to score, next block to accumulate
      auto pv_ready = [&]() { return pv < qk && mbar_try_wait(p_full, pv & 1); };
      auto issue_qk = [&](int i) {
        tc_fence_after();
        const uint64_t kd0 = pick(kdesc, i % NB);
#pragma unroll
        for (int lp = 0; lp < 4; ++lp) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16_ts(tmem + kColS, tmem + kColQ + lp * 32 + 8 * ks, kd0 + uint64_t((lp * kMlaKPanelBytes) >> 4) + 2 * ks,
                        idesc_qk, (lp | ks) != 0);
          if (pv_ready()) pv_mmas(pv++);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
          umma_f16_ts(tmem + kColS, tmem + kColQ + 4 * 32 + 8 * (rope_ks + u),
                      kd0 + uint64_t((4 * kMlaKPanelBytes) >> 4) + 2 * (rope_ks + u), idesc_qk, 1);
        umma_commit(s_full);
      };
      // Whatever is ready goes: the scores of the next block (its rows gathered, S read out by warps 0-7), else P.V of the
      // oldest block whose P is there.  Blocking on one of the two while the other could run used to pace the kernel.
      // (Tried and dropped: P.V only inside a chain -- four P.V MMAs cost the pipe about 600 cycles wherever they go.)
      // The start of the next chain is what the block time hangs on, so the accumulator's release is polled first and
      // the arrival of the gathered rows, once seen, is not polled again (a poll costs 100-150 cycles even on a barrier
      // that is complete).
      uint32_t idle = 0;
      bool rows_there = false;
      while (ok && pv < nblk) {
        if (qk < nblk && !rows_there) rows_there = mbar_try_wait(&kv_full[qk % NB], (qk / NB) & 1);
        if (rows_there && (qk == 0 || mbar_try_wait(s_free, (qk - 1) & 1))) {
          issue_qk(qk);
          ++qk;
          rows_there = false;
          idle = 0;
        } else if (pv_ready()) {
          pv_mmas(pv++);
          idle = 0;
        } else if (++idle > kFastSpins) {              // bounded like every other wait (dsa_common.cuh)
          if (*abort_flag) ok = false;
          else if (idle > kSpinLimit) {
            *abort_flag = 1;
            if (a.status) atomicCAS(a.status, kStatusOk, kStatusWaitTimeout);
            ok = false;
          } else __nanosleep(40);
        }
      }
    }
  } else if (warp == kMlaCopyWarp) {
    // ------------------- partial score tiles: this CTA's send_s[stage] -> the peer's recv_s[stage] -------------------
    cluster_wait();
    if (lane == 0) {
      const uint32_t peer_recv = mapa_u32(smem_u32(recv_s), peer), peer_recv_full = mapa_u32(smem_u32(recv_full), peer);
      for (int n = 0; n < nblk; ++n) {
        const int st = n & 1, ph = (n >> 1) & 1;
        if (!mbar_wait(&send_full[st], ph, abort_flag, a.status)) break;    // all eight warps have written their parts of block n
        // warps 0-7 consumed the peer's block n-2 before they wrote block n: this CTA's receive stage can be armed again
        mbar_expect_tx(&recv_full[st], kMlaXBytes);
        bulk_copy_to_peer(peer_recv + st * kMlaXBytes, send_s + st * kMlaXBytes, kMlaXBytes, peer_recv_full + st * 8);
      }
    }
  } else if (warp >= 9) {
    // ----------------------------- gather of the selected rows -----------------------------
    const int g = threadIdx.x - 288;                  // 0..kMlaGatherThreads-1
    const int w4 = warp - 9;
    // Row ids travel two blocks ahead of their use, so that no global-memory latency sits in the loop below: `pos_nxt` is the
    // selected position of this thread's slot in the block after the next gather, `row_cur` the row id (for decode: the
    // physical cache row, through the block table) of its slot in the next gather.  Threads 0..63 of the group.
    auto load_pos = [&](int blk) -> int {
      const int j = blk * kMlaBlk + g;
      return (g < kMlaBlk && blk < nblk && j < k_cnt) ? __ldg(idx_row + j) : -1;
    };
    auto translate = [&](int pos) -> int {             // -1 = empty slot; bad positions and page ids are flagged and skipped
      if (pos < 0) return -1;
      if (pos >= a.S_kv) {
        if (a.status) atomicCAS(a.status, kStatusOk, kStatusBadIndex);
        return -1;
      }
      if constexpr (!FP8_PAGED) {
        return pos;
      } else {
        const int phys = __ldg(a.block_table + (int64_t)t * a.table_stride + pos / kLatentPage);
        if (phys >= 0 && (int64_t)(phys + 1) * kLatentPage <= a.num_phys_rows) return phys * kLatentPage + pos % kLatentPage;
        if (a.status) atomicCAS(a.status, kStatusOk, kStatusBadIndex);
        return -1;
      }
    };
    bool ok = true;
    if constexpr (!FP8_PAGED) {
      int row_cur = translate(load_pos(0)), pos_nxt = load_pos(1);
      // stage the row ids of block i and fill its KV buffer; called for i = 0, 1, 2, ... in order
      auto gather = [&](int i) -> bool {
        const int kvb = i % NB;
        int* rows_s = ring + (i % kMlaRing) * kMlaBlk;
        if (i >= NB) mbar_wait(&kv_free[kvb], ((i / NB) - 1) & 1, abort_flag, a.status);
        if (g < kMlaBlk) {
          rows_s[g] = row_cur;
          const uint32_t used = __ballot_sync(0xffffffffu, row_cur >= 0);       // warps 9 and 10: 32 slots each
          if (lane == 0) masks[(i % kMlaMaskRing) * 2 + w4] = used;
        }
        row_cur = translate(pos_nxt);
        pos_nxt = load_pos(i + 2);
        // ids staged; every thread of the group takes the same way out of a failed wait
        if (named_bar_or(2, kMlaGatherThreads, *abort_flag != 0)) return false;
        uint8_t* dst = kv_s + kvb * kMlaKBytes;
        // warp w4 fetches kRowsPerWarp consecutive rows: lane = 5 * (group of four rows) + panel, one gather4 each
        constexpr int kRowsPerWarp = kMlaBlk / kMlaGatherWarps, kLanes = kRowsPerWarp / 4 * kMlaPanels;
        if (lane == 0) mbar_expect_tx(&kv_full[kvb], kLanes * 512);
        __syncwarp();
        if (lane < kLanes) {
          const int rg = lane / kMlaPanels, lp = lane - rg * kMlaPanels;
          const int r0 = w4 * kRowsPerWarp + rg * 4;
          const int x = (lp < 4 ? cta * 4 + lp : 8) * 32;             // in the map's 4-byte elements
          // an empty slot reads the row just past the end of the tensor: TMA fills it with zeros
          auto rid = [&](int r) { const int v = rows_s[r]; return v >= 0 ? v : a.S_kv; };
          tma_gather4(dst + lp * kMlaKPanelBytes + r0 * 128, &tmap_kv, x, rid(r0), rid(r0 + 1), rid(r0 + 2), rid(r0 + 3),
                      &kv_full[kvb]);
        }
        return true;
      };
      // Up to four blocks are in flight: the wait on kv_free inside gather() is what paces this loop.  The last two
      // buffers hold the Q panels until Q is in tensor memory.
      for (int i = 0; i < nblk && ok; ++i) {
        if (i == NB - 2) mbar_wait(q_moved, 0, abort_flag, a.status);      // a failure shows in abort_flag inside gather()
        ok = gather(i);
      }
    } else {
      // Decode.  Block b's raw rows are requested two blocks ahead with cp.async into one of two raw stages (the space of
      // the fourth KV buffer), its rope halves with plain loads into registers; block b is converted into its KV buffer
      // while blocks b+1 and b+2 are on their way.  The page-table entry of a slot is requested one call before it is
      // examined, its position one call before that, so that no global-memory latency sits in the loop.
      uint8_t* raw_s = kv_s + NB * kMlaKBytes;
      auto table_entry = [&](int pos) -> int {
        return (pos >= 0 && pos < a.S_kv) ? __ldg(a.block_table + (int64_t)t * a.table_stride + pos / kLatentPage) : -1;
      };
      auto cache_row = [&](int pos, int phys) -> int {   // -1 = empty slot; bad positions and page ids are flagged and skipped
        if (pos < 0) return -1;
        if (pos < a.S_kv && phys >= 0 && (int64_t)(phys + 1) * kLatentPage <= a.num_phys_rows)
          return phys * kLatentPage + pos % kLatentPage;
        if (a.status) atomicCAS(a.status, kStatusOk, kStatusBadIndex);
        return -1;
      };
      constexpr int kRopePer = kMlaBlk * 4 / kMlaGatherThreads;      // 16-byte rope chunks per thread and block
      uint4 rope_e[kRopePer], rope_o[kRopePer];        // rope chunks of the even / odd block in flight
      // request block b: stage its row ids (and the validity mask for the softmax), then issue the copies
      auto fetch = [&](int b, int row, uint4 (&rope)[kRopePer]) {
        int* rows_s = ring + (b & 1) * kMlaBlk;
        if (g < kMlaBlk) {
          rows_s[g] = row;
          const uint32_t used = __ballot_sync(0xffffffffu, row >= 0);            // warps 9 and 10: 32 slots each
          if (lane == 0) masks[(b % kMlaMaskRing) * 2 + w4] = used;
        }
        named_bar_sync(2, kMlaGatherThreads);            // ids staged; everyone is done with the raw stage that is overwritten next
        if (b < nblk) {
          uint8_t* stage = raw_s + (b & 1) * kRawStage;
          constexpr int kCopies = kMlaBlk * 17;          // 16 value chunks + the scales, per row
#pragma unroll
          for (int u = 0; u < (kCopies + kMlaGatherThreads - 1) / kMlaGatherThreads; ++u) {
            const int q = g + u * kMlaGatherThreads;
            if (q < kCopies) {
              const int r = q / 17, c = q - r * 17;
              const int rr = rows_s[r];
              const uint8_t* rec = a.cache + (int64_t)(rr >= 0 ? rr : 0) * kLatentTokenBytes;
              cp_async_16(stage + r * kRawRow + c * 16, rec + (c < 16 ? cta * kMlaDvHalf + c * 16 : kMlaDv), rr >= 0 ? 16 : 0);
            }
          }
#pragma unroll
          for (int u = 0; u < kRopePer; ++u) {           // this CTA's two K-steps of the rope panel: 64 bytes per row
            const int q = g + u * kMlaGatherThreads;
            const int rr = rows_s[q >> 2];
            rope[u] = make_uint4(0, 0, 0, 0);
            if (rr >= 0)
              rope[u] = __ldg(reinterpret_cast<const uint4*>(a.cache + (int64_t)rr * kLatentTokenBytes + kMlaDv + 16) + cta * 4 + (q & 3));
          }
        }
        cp_async_commit();                               // one group per call, empty or not: the counting below relies on it
      };
      int P2, T2, P3;                                    // position / table entry of this thread's slot in block i+2, position in block i+3
      {
        const int p0 = load_pos(0), p1 = load_pos(1);
        P2 = load_pos(2);
        P3 = load_pos(3);
        const int t0 = table_entry(p0), t1 = table_entry(p1);
        T2 = table_entry(P2);
        fetch(0, cache_row(p0, t0), rope_e);
        fetch(1, cache_row(p1, t1), rope_o);
      }
      auto step = [&](int i, uint4 (&rope)[kRopePer]) -> bool {
        const int kvb = i % NB;
        if (i == NB - 2) mbar_wait(q_moved, 0, abort_flag, a.status);    // buffers NB-2 and NB-1 held the Q panels
        if (i >= NB) mbar_wait(&kv_free[kvb], ((i / NB) - 1) & 1, abort_flag, a.status);
        cp_async_wait<1>();                              // this thread's copies of block i have landed (block i+1 may be in flight)
        // ... and everyone else's; every thread of the group takes the same way out of a failed wait
        if (named_bar_or(2, kMlaGatherThreads, *abort_flag != 0)) return false;
        uint8_t* dst = kv_s + kvb * kMlaKBytes;
        convert_block<kMlaGatherThreads>(raw_s + (i & 1) * kRawStage, dst, g, cta);
#pragma unroll
        for (int u = 0; u < kRopePer; ++u) {
          const int q = g + u * kMlaGatherThreads;
          const int r = q >> 2, c = cta * 4 + (q & 3);
          *reinterpret_cast<uint4*>(dst + 4 * kMlaKPanelBytes + r * 128 + ((c ^ (r & 7)) << 4)) = rope[u];
        }
        fence_async_smem();                              // make the panel writes visible to the tensor core's reads
        mbar_arrive(&kv_full[kvb]);
        const int row = cache_row(P2, T2);               // block i+2
        P2 = P3;
        T2 = table_entry(P2);
        P3 = load_pos(i + 4);
        fetch(i + 2, row, rope);
        return true;
      };
      for (int i = 0; i < nblk && ok; i += 2) {
        ok = step(i, rope_e);
        if (ok && i + 1 < nblk) ok = step(i + 1, rope_o);
      }
      cp_async_wait<0>();                                // nothing of this thread's is in flight into shared memory when it leaves
    }
  } else {
    // ------------- partial-score exchange, softmax and output: thread = (head, half of a block's keys) -------------
    const int qd = warp & 3, half = warp >> 2;
    const int row = qd * 32 + lane;                    // head = TMEM lane
    const uint32_t t_row = tmem + (uint32_t(qd * 32) << 16);
    const uint32_t peer_xchg_free = mapa_u32(smem_u32(xchg_free), peer);      // [2], 8 bytes apart
    uint16_t* max_s = reinterpret_cast<uint16_t*>(pair_s);                    // [2 buffers][2 halves][128 heads] bf16 bits
    float m = -CUDART_INF_F, l = 0.f;                  // l: this thread's keys only
    bool ok = __all_sync(0xffffffffu, mbar_wait(q_full, 0, abort_flag, a.status));
    if (ok) {
      // this head's row of the five Q panels, swizzled shared memory -> packed bf16 pairs in tensor memory: the ten
      // half-panels (64 B) alternate between the two threads of the head
#pragma unroll 1
      for (int hp = half; hp < 2 * kMlaPanels; hp += 2) {
        uint32_t qv[16];
        const uint8_t* src = q_stage(hp >> 1) + row * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint4 w = *reinterpret_cast<const uint4*>(src + ((((hp & 1) * 4 + c) ^ (row & 7)) << 4));
          qv[4 * c + 0] = w.x; qv[4 * c + 1] = w.y; qv[4 * c + 2] = w.z; qv[4 * c + 3] = w.w;
        }
        tmem_st16(t_row + kColQ + hp * 16, qv);
      }
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_moved);             // one arrival per warp: 256 arrivals on one barrier queue up
    }
    cluster_wait();
    // Per iteration n: first half of the softmax of block n-1 (its peer tile arrived while this warp did other things:
    // scores, block maximum), then -- as soon as the scores of block n are complete -- their read-out and hand-over, then
    // the second half (exponentials, P).  The read-out sits in the middle so that the first half fills the time this warp
    // would otherwise wait for the chain, and P of block n-1 is ready early enough to be queued right behind chain n+1.
    float s[32];                                       // raw scores of block n-1; the (positive) scale is folded into the exponent's FMA
    float bmax = 0.f;                                  // block maximum over all 64 keys, in log2 units
    for (int n = 0; n <= nblk && ok; ++n) {
      const int j = n - 1;
      if (n > 0) {
        const int st = j & 1, ph = (j >> 1) & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(&recv_full[st], ph, abort_flag, a.status));
        if (!ok) break;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int off = st * kMlaXBytes + xchg_off(half, row, c);
          const uint4 mine = *reinterpret_cast<const uint4*>(send_s + off);       // what this thread wrote itself
          const uint4 theirs = *reinterpret_cast<const uint4*>(recv_s + off);
          const uint32_t mw[4] = {mine.x, mine.y, mine.z, mine.w}, tw[4] = {theirs.x, theirs.y, theirs.z, theirs.w};
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 x = add_f16x2_f32(mw[k], tw[k]);
            s[8 * c + 2 * k] = x.x;
            s[8 * c + 2 * k + 1] = x.y;
          }
        }
        if constexpr (kAck) {
          __syncwarp();
          if (lane == 0) mbar_arrive_remote_relaxed(peer_xchg_free + st * 8);    // the peer may send into this stage again
        }
        const uint32_t used = masks[(j % kMlaMaskRing) * 2 + half];
        if (used != 0xffffffffu) {                       // empty slots (the tail of a short row, holes): warp-uniform
#pragma unroll
          for (int i = 0; i < 32; ++i) s[i] = (used >> i) & 1u ? s[i] : -CUDART_INF_F;
        }
        float bm[4] = {s[0], s[1], s[2], s[3]};          // four independent chains
#pragma unroll
        for (int i = 4; i < 32; ++i) bm[i & 3] = fmaxf(bm[i & 3], s[i]);
        // the block maximum over all 64 keys: the two threads of a head exchange theirs, rounded up to bf16
        uint16_t* mx = max_s + (j & 1) * 256;
        const uint32_t mine_bits = bf16_bits_round_up(fmaxf(fmaxf(bm[0], bm[1]), fmaxf(bm[2], bm[3])) * a.scale_log2e);
        mx[half * 128 + row] = static_cast<uint16_t>(mine_bits);
        named_bar_sync(3 + qd, 64);
        bmax = fmaxf(__uint_as_float(mine_bits << 16), __uint_as_float(uint32_t(mx[(half ^ 1) * 128 + row]) << 16));
      }
      if (n < nblk) {
        // ---- partial scores of block n: tensor memory -> registers -> fp16 in send_s[stage]; the copy warp takes it from there
        const int st = n & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(s_full, n & 1, abort_flag, a.status));
        if (!ok) break;
        tc_fence_after();
        uint32_t sv[32];
        tmem_ld32(t_row + kColS + 32 * half, sv);
        tmem_wait_ld();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);            // the next block's scores may overwrite S now
        // The peer must have read block n-2, the last user of this stage (which also means that that copy is complete).
        // That is already so without asking: this thread has seen the peer's block n-1 arrive (first half of the softmax
        // above), the peer sent it only after all of its warps had written their parts, and each of them wrote its part
        // after it had read this CTA's block n-2.  The same holds the other way round.
        if constexpr (kAck) {
          if (n >= kMlaXStages) ok = __all_sync(0xffffffffu, mbar_wait(&xchg_free[st], ((n >> 1) & 1) ^ 1, abort_flag, a.status));
          if (!ok) break;
        }
        uint8_t* send = send_s + st * kMlaXBytes;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          auto h2 = [&](int k) { return pack_f16x2(__uint_as_float(sv[8 * c + 2 * k]), __uint_as_float(sv[8 * c + 2 * k + 1])); };
          *reinterpret_cast<uint4*>(send + xchg_off(half, row, c)) = make_uint4(h2(0), h2(1), h2(2), h2(3));
        }
        fence_async_smem();                            // the bulk copy reads the tile through the async proxy
        __syncwarp();
        if (lane == 0) mbar_arrive(&send_full[st]);
      }
      if (n > 0) {
        const float m_new = fmaxf(m, bmax);
        const bool grow = m_new - m > 8.f;               // also true when m is still -inf and m_new is finite
        bool waited_pv = false;
        if (__any_sync(0xffffffffu, grow)) {
          const float alpha = grow ? fast_exp2(m - m_new) : 1.f;
          if (grow) m = m_new;
          l *= alpha;
          if (j > 0) {
            // O must be quiescent: P.V of the previous block has to be complete.  This thread scales its half of the columns.
            ok = __all_sync(0xffffffffu, mbar_wait(pv_done, (j - 1) & 1, abort_flag, a.status));
            if (!ok) break;
            waited_pv = true;
            tc_fence_after();
#pragma unroll 1
            for (int c = half * (kMlaDvHalf / 2); c < (half + 1) * (kMlaDvHalf / 2); c += 32) {
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
        uint32_t pk[16];
        float ps[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = fast_exp2(fmaf(s[i], a.scale_log2e, -m_eff)), p1 = fast_exp2(fmaf(s[i + 1], a.scale_log2e, -m_eff));
          ps[(i >> 1) & 3] += p0 + p1;
          pk[i >> 1] = pack_bf16x2(p0, p1);
        }
        l += (ps[0] + ps[1]) + (ps[2] + ps[3]);
        if (j > 0 && !waited_pv) {                       // P is single-buffered: P.V of the previous block must be done
          ok = __all_sync(0xffffffffu, mbar_wait(pv_done, (j - 1) & 1, abort_flag, a.status));
          if (!ok) break;
          tc_fence_after();
        }
        tmem_st16(t_row + kColP + 16 * half, pk);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
      }
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(o_final, 0, abort_flag, a.status));
    // A full group of 128 heads leaves through shared memory and TMA stores: four [128 heads x 128 B] panels in the
    // (now idle) first two KV buffers, written asynchronously in whole lines.  16-byte stores from the threads -- every
    // lane its own 1 KB-strided row -- cost about 4 % of the kernel.
    const bool by_tma = a.tma_out && a.n_split == 1 && heads_here == 128;
    if (ok) {
      tc_fence_after();
      // the row sum over all keys: the two threads of a head add theirs (the maxima buffer is free: every P has been consumed)
      float* sum_s = reinterpret_cast<float*>(pair_s);
      sum_s[half * 128 + row] = l;
      named_bar_sync(3 + qd, 64);
      l += sum_s[(half ^ 1) * 128 + row];
      const float inv = l > 0.f ? 1.f / l : 0.f;
      __nv_bfloat16* orow = a.out + ((int64_t)t * a.H + hg * 128 + row) * kMlaDv + cta * kMlaDvHalf;
      const int64_t prow = (int64_t)unit * a.H + hg * 128 + row;
      if (a.n_split > 1 && cta == 0 && half == 0 && row < heads_here)
        a.part_lse[prow] = l > 0.f ? m + log2f(l) : -CUDART_INF_F;
#pragma unroll 1
      for (int c = half * (kMlaDvHalf / 2); c < (half + 1) * (kMlaDvHalf / 2); c += 32) {
        uint32_t ov[32];
        tmem_ld32(t_row + kColO + c, ov);
        tmem_wait_ld();
        if (by_tma) {
          uint8_t* prow_s = kv_s + (c >> 6) * kMlaQPanelBytes + row * 128;
          const int ch0 = (c & 63) >> 3;                 // first of this iteration's four 16-byte chunks in the 128-byte row
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 w;
            w.x = pack_bf16x2(__uint_as_float(ov[i + 0]) * inv, __uint_as_float(ov[i + 1]) * inv);
            w.y = pack_bf16x2(__uint_as_float(ov[i + 2]) * inv, __uint_as_float(ov[i + 3]) * inv);
            w.z = pack_bf16x2(__uint_as_float(ov[i + 4]) * inv, __uint_as_float(ov[i + 5]) * inv);
            w.w = pack_bf16x2(__uint_as_float(ov[i + 6]) * inv, __uint_as_float(ov[i + 7]) * inv);
            *reinterpret_cast<uint4*>(prow_s + (((ch0 + (i >> 3)) ^ (row & 7)) << 4)) = w;
          }
        } else if (row < heads_here && a.n_split > 1) {
          float4* po = reinterpret_cast<float4*>(a.part_o + prow * kMlaDv + cta * kMlaDvHalf + c);
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
    if (by_tma) {                                      // every thread of warps 0-7 comes here, whatever became of its waits
      fence_async_smem();                              // the stores below read the panels through the async proxy
      named_bar_sync(7, 256);
      if (threadIdx.x == 0 && !*abort_flag) {
#pragma unroll
        for (int pn = 0; pn < 4; ++pn)                 // x in 4-byte units: 32 per 64-column panel
          tma_store_2d(&tmap_o, kv_s + pn * kMlaQPanelBytes, (cta * 4 + pn) * 32, t * a.H + hg * 128);
        bulk_commit_and_wait_read();                   // the panels have been read: the CTA may go
      }
    }
  }

  __syncwarp();
  if (warp >= 8 && warp != kMlaCopyWarp) cluster_wait();      // MMA and gather warps: the wait that pairs with the arrive above
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // a wait gave up: let the copies that may still be in flight into this CTA land (bounded) before its shared memory goes away
    if (threadIdx.x == 0)
      for (int w = 0; w < 64; ++w) __nanosleep(1000);
    __syncthreads();
  }
  cluster_arrive_wait();          // neither CTA leaves while the other may still copy into it or arrive on its barriers
  if (warp == 8) {
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
static int launch_mla(const void* q, const void* kv, const MlaArgs& args, cudaStream_t stream) {
  if (args.T == 0 || args.H == 0) return DSA_OK;
  MlaArgs a = args;
  CUtensorMap tq, tkv, to;
  int rc = make_tmap_2d_bytes(&tq, q, (uint64_t)a.T * a.H, kMlaDqk * 2, kMlaDqk * 2, 128, 128);
  if (rc) return rc;
  // the output as [T*H rows x 1024 B], stored one [128 heads x 128 B] panel at a time -- when there is a full group of
  // 128 heads, no split, and the tensor can be mapped (16-byte aligned)
  a.tma_out = 0;
  to = tq;
  if (a.n_split == 1 && a.H >= 128 && (reinterpret_cast<uintptr_t>(a.out) & 15) == 0) {
    if ((rc = make_tmap_2d_bytes(&to, a.out, (uint64_t)a.T * a.H, kMlaDv * 2, kMlaDv * 2, 128, 128))) return rc;
    a.tma_out = 1;
  }
  // rows of the bf16 KV, one 64-dim panel (128 bytes) of one row per box: the shape tile::gather4 takes
  // (decode reads its cache with plain loads and only carries a copy of the Q map here)
  if (FP8_PAGED || a.S_kv == 0) tkv = tq;
  else if ((rc = make_tmap_2d_bytes(&tkv, kv, (uint64_t)a.S_kv, kMlaDqk * 2, kMlaDqk * 2, 128, 1))) return rc;
  auto kern = sparse_mla_kernel<FP8_PAGED>;
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmemBytes) != cudaSuccess)
    return set_error(DSA_ERR_CUDA, "sparse_mla: cannot raise dynamic shared memory to %d", kMlaSmemBytes);
  const dim3 grid(2 * a.T * a.n_split, 1, (a.H + 127) / 128);
  kern<<<grid, MlaCfg<FP8_PAGED>::kThreads, kMlaSmemBytes, stream>>>(tq, tkv, to, a);
  if (a.n_split > 1) sparse_mla_combine_kernel<<<dim3(a.T, a.H), 128, 0, stream>>>(a);
  return check_launch("sparse_mla");
}

int sparse_mla_prefill_launch(const void* q, const void* kv, const int32_t* idx, void* out, int T, int H, int S_kv,
                              int K, float scale, int32_t* status, cudaStream_t stream) {
  MlaArgs a{};
  a.idx = idx;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.T = T; a.H = H; a.K = K; a.S_kv = S_kv;
  a.scale_log2e = scale * 1.4426950408889634f;
  a.status = status;
  a.n_split = 1;
  return launch_mla<false>(q, kv, a, stream);
}

// With few queries (decode) one CTA pair per query leaves most SMs idle and walks 2048 slots serially:
// cut the slot list into parts of >= 256 slots while the grid still fits the GPU in one wave.  More
// parts than that lose: every part pays the set-up again and writes an fp32 partial output that the
// combine kernel reads back.
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
  return launch_mla<true>(q, nullptr, a, stream);
}

}  // namespace dsa
