// Per-row top-k by radix select (sm_100a).  Stands in for the torch.topk calls at
// sparse_attn/DSA.py:361, 567 and 675-676 of the reference.
//
// One CTA per row.  fp32 values are mapped to order-preserving 32-bit keys.  A
// pass histograms the next 12 key bits (shared-memory atomics) of the elements
// that still match the decided prefix, a block-wide suffix scan finds the bin
// holding the k-th largest element, and passes repeat until that bin is small
// enough to finish in shared memory (or all 32 bits are decided, which handles
// rows full of equal values).  One final pass over the row writes, in column
// order, the elements above the threshold bin straight to the output and
// stages the threshold bin's elements in shared memory, where each candidate's
// rank is counted directly.  Ties at the k-th value go to the lower column.
// Compaction uses block prefix sums, not atomics, so the output is
// bit-identical from run to run.  The row is read once from HBM; later passes
// hit L2 (a 131072-column row is 512 KB).
#include <math_constants.h>

#include "dsa_common.cuh"
#include "dsa_host.h"

namespace dsa {

constexpr int kTopkThreads = 512;
constexpr int kTopkWarps = kTopkThreads / 32;
constexpr int kDigitBits = 12;
constexpr int kBins = 1 << kDigitBits;
constexpr int kBinsPerThread = kBins / kTopkThreads;   // 8
constexpr int kCand = 2048;
constexpr int kVec = 4;
constexpr int kChunk = kTopkThreads * kVec;

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct RowReader {
  const float* x;     // row base
  int lo, hi;         // window
  int base;           // first chunk start (multiple of 4, <= lo)
  bool vec;           // 16-byte loads allowed
  __device__ __forceinline__ void load(int i, float (&v)[kVec]) const {
    // i is a multiple of 4; elements outside [lo, hi) are returned as-is and ignored by callers
    if (vec) {
      const float4 f = __ldg(reinterpret_cast<const float4*>(x + i));
      v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
    } else {
#pragma unroll
      for (int j = 0; j < kVec; ++j) v[j] = (i + j >= lo && i + j < hi) ? __ldg(x + i + j) : 0.f;
    }
  }
};

// inclusive warp scan of a packed pair of 16-bit counters
__device__ __forceinline__ uint32_t warp_inclusive_scan(uint32_t v) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t n = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += n;
  }
  return v;
}

__global__ void __launch_bounds__(kTopkThreads)
topk_select_kernel(const float* __restrict__ logits, int64_t ld, const int32_t* __restrict__ ks,
                   const int32_t* __restrict__ ke, int T, int S, int k, int32_t* __restrict__ out) {
  __shared__ uint32_t hist[kBins];
  __shared__ uint32_t cand_key[kCand];
  __shared__ int32_t cand_idx[kCand];
  __shared__ uint32_t warp_tot[2][kTopkWarps];
  __shared__ uint32_t s_bin, s_need, s_cnt;

  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;
  int lo = ks ? max(ks[row], 0) : 0;
  int hi = ke ? min(ke[row], S) : S;
  const int n = max(hi - lo, 0);
  int32_t* o = out + (int64_t)row * k;
  if (n <= k) {
    for (int j = tid; j < k; j += kTopkThreads) o[j] = j < n ? lo + j : -1;
    return;
  }
  RowReader rd;
  rd.x = logits + (int64_t)row * ld;
  rd.lo = lo;
  rd.hi = hi;
  rd.base = lo & ~(kVec - 1);
  rd.vec = ((reinterpret_cast<uintptr_t>(rd.x) & 15) == 0) && (ld % kVec == 0);
  const int n_chunks = (hi - rd.base + kChunk - 1) / kChunk;

  uint32_t prefix = 0;    // value of the decided high bits
  int pbits = 0;          // how many high bits are decided
  uint32_t need = k;      // how many elements are still wanted from the matching set
  uint32_t cnt = 0;       // size of the threshold bin

  while (true) {
    const int dbits = min(kDigitBits, 32 - pbits);
    const int shift = 32 - pbits - dbits;
    const uint32_t dmask = (1u << dbits) - 1u;
    for (int b = tid; b < kBins; b += kTopkThreads) hist[b] = 0;
    __syncthreads();
    for (int c = 0; c < n_chunks; ++c) {
      const int i = rd.base + c * kChunk + tid * kVec;
      if (i >= hi) continue;
      float v[kVec];
      rd.load(i, v);
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        if (i + j < lo || i + j >= hi) continue;
        const uint32_t key = order_key(v[j]);
        if (pbits == 0 || (key >> (32 - pbits)) == prefix) atomicAdd(&hist[(key >> shift) & dmask], 1u);
      }
    }
    __syncthreads();
    // suffix scan over bins: thread t owns bins [8t, 8t+8); scan in reversed thread order
    uint32_t mine = 0;
#pragma unroll
    for (int j = 0; j < kBinsPerThread; ++j) mine += hist[tid * kBinsPerThread + j];
    const int rt = kTopkThreads - 1 - tid;          // reversed thread id
    // butterfly: bring value of reversed order into scan order
    uint32_t v = mine;
    // scan within warp in reversed lane order
    {
      const int rl = 31 - lane;
#pragma unroll
      for (int off = 1; off < 32; off <<= 1) {
        const uint32_t nb = __shfl_down_sync(0xffffffffu, v, off);
        if (rl >= off) v += nb;
      }
    }
    if (lane == 0) warp_tot[0][warp] = v;           // total of this warp
    __syncthreads();
    uint32_t above = 0;                             // sum over warps with higher bins
    for (int w2 = warp + 1; w2 < kTopkWarps; ++w2) above += warp_tot[0][w2];
    const uint32_t incl = v + above;                // sum of bins >= 8*tid
    const uint32_t excl = incl - mine;              // sum of bins >= 8*(tid+1)
    (void)rt;
    if (excl < need && need <= incl) {
      uint32_t cum = excl;
      for (int j = kBinsPerThread - 1; j >= 0; --j) {
        const uint32_t h = hist[tid * kBinsPerThread + j];
        if (cum + h >= need) {
          s_bin = tid * kBinsPerThread + j;
          s_need = need - cum;
          s_cnt = h;
          break;
        }
        cum += h;
      }
    }
    __syncthreads();
    prefix = (pbits == 0 ? 0u : (prefix << dbits)) | s_bin;
    need = s_need;
    cnt = s_cnt;
    pbits += dbits;
    __syncthreads();
    if (cnt <= kCand || pbits == 32) break;
  }

  // ---- final pass: ordered compaction ---------------------------------------
  const uint32_t n_above = k - need;                // elements strictly above the threshold bin
  const bool all_tied = (pbits == 32);              // every candidate equals the k-th value
  const int pshift = 32 - pbits;                    // 0 when all bits are decided
  uint32_t base_sel = 0, base_cand = 0;
  for (int c = 0; c < n_chunks; ++c) {
    const int i = rd.base + c * kChunk + tid * kVec;
    uint32_t keys[kVec];
    uint32_t packed = 0;
    uint32_t fsel = 0, fcand = 0;
    if (i < hi) {
      float v[kVec];
      rd.load(i, v);
#pragma unroll
      for (int j = 0; j < kVec; ++j) {
        keys[j] = order_key(v[j]);
        if (i + j < lo || i + j >= hi) continue;
        const uint32_t top = pshift >= 32 ? 0u : (keys[j] >> pshift);
        if (top > prefix) { fsel |= 1u << j; packed += 1u; }
        else if (top == prefix) { fcand |= 1u << j; packed += 1u << 16; }
      }
    }
    const uint32_t incl = warp_inclusive_scan(packed);
    if (lane == 31) warp_tot[c & 1][warp] = incl;
    __syncthreads();
    uint32_t before = 0, total = 0;
#pragma unroll
    for (int w2 = 0; w2 < kTopkWarps; ++w2) {
      const uint32_t t2 = warp_tot[c & 1][w2];
      if (w2 < warp) before += t2;
      total += t2;
    }
    const uint32_t excl = incl - packed + before;
    uint32_t ps = base_sel + (excl & 0xffffu);
    uint32_t pc = base_cand + (excl >> 16);
#pragma unroll
    for (int j = 0; j < kVec; ++j) {
      if (fsel & (1u << j)) {
        o[ps++] = i + j;
      } else if (fcand & (1u << j)) {
        if (all_tied) {
          if (pc < need) o[n_above + pc] = i + j;
        } else if (pc < (uint32_t)kCand) {
          cand_key[pc] = keys[j];
          cand_idx[pc] = i + j;
        }
        ++pc;
      }
    }
    base_sel += total & 0xffffu;
    base_cand += total >> 16;
  }
  if (all_tied) return;
  __syncthreads();
  // ---- rank the candidates: larger key first, lower column first on ties ------
  for (uint32_t a = tid; a < cnt; a += kTopkThreads) {
    const uint32_t ka = cand_key[a];
    uint32_t rank = 0;
    for (uint32_t b = 0; b < cnt; ++b) {
      const uint32_t kb = cand_key[b];
      rank += (kb > ka) || (kb == ka && b < a);
    }
    if (rank < need) o[n_above + rank] = cand_idx[a];
  }
}

int topk_select_launch(const float* logits, int64_t ld, const int32_t* ks, const int32_t* ke, int T, int S, int k,
                       int32_t* out, cudaStream_t stream) {
  if (T == 0 || k == 0) return DSA_OK;
  topk_select_kernel<<<T, kTopkThreads, 0, stream>>>(logits, ld, ks, ke, T, S, k, out);
  return check_launch("topk_select");
}

}  // namespace dsa
