// Per-row top-k by radix select (sm_100a).  Stands in for the torch.topk calls at
// sparse_attn/DSA.py:361, 567 and 675-676 of the reference.
//
// One CTA per row.  fp32 values are mapped to order-preserving 32-bit keys and
// the k-th largest key is found digit by digit (12 + 12 + 8 bits):
//   1. histogram the top 12 key bits of the row (shared-memory atomics), suffix-
//      scan the bins to find the bin holding the k-th largest element;
//   2. if that bin holds more than 2048 elements, repeat on the next digit over
//      the row (only rows with tightly clustered values need this);
//   3. one ordered pass over the row writes every element above the threshold
//      bin straight to the output and stages the threshold bin's elements
//      ("candidates") in shared memory, in column order;
//   4. the remaining digits are resolved on the staged candidates, and a final
//      ordered compaction emits candidates above the exact k-th key plus the
//      first `need` candidates equal to it -- ties go to the lower column.
// Compaction uses block prefix sums, never atomics, so the output is
// bit-identical from run to run.  The row is read from HBM once; the second
// read hits L2 (a 131072-column row is 512 KB).
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
constexpr int kCandPerThread = kCand / kTopkThreads;   // 4
constexpr int kVec = 4;
constexpr int kEltPerThread = 16;                      // final pass: 4 x float4, contiguous
constexpr int kChunkHist = kTopkThreads * kVec;        // histogram pass: coalesced float4
constexpr int kChunkFinal = kTopkThreads * kEltPerThread;

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return u ^ (static_cast<uint32_t>(static_cast<int32_t>(u) >> 31) | 0x80000000u);
}

struct TopkSmem {
  uint32_t hist[kBins];
  uint32_t cand_key[kCand];
  int32_t cand_idx[kCand];
  uint32_t warp_tot[2][kTopkWarps];
  uint32_t bin, need, cnt;
};

// Block-wide: given hist[], find the bin b with  sum(hist[b+1..]) < need <= sum(hist[b..]).
// Leaves bin / need (remaining within the bin) / cnt (= hist[b]) in shared memory.
__device__ __forceinline__ void find_threshold_bin(TopkSmem& sm, uint32_t need) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t h[kBinsPerThread];
  uint32_t mine = 0;
#pragma unroll
  for (int j = 0; j < kBinsPerThread; ++j) {
    h[j] = sm.hist[tid * kBinsPerThread + j];
    mine += h[j];
  }
  uint32_t v = mine;                     // suffix-inclusive scan inside the warp
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const uint32_t nb = __shfl_down_sync(0xffffffffu, v, off);
    if (lane + off < 32) v += nb;
  }
  if (lane == 0) sm.warp_tot[0][warp] = v;
  __syncthreads();
  uint32_t above = 0;
  for (int w2 = warp + 1; w2 < kTopkWarps; ++w2) above += sm.warp_tot[0][w2];
  const uint32_t incl = v + above;       // elements in bins >= first bin of this thread
  uint32_t cum = incl - mine;            // elements in bins above this thread's
  if (cum < need && need <= incl) {
#pragma unroll
    for (int j = kBinsPerThread - 1; j >= 0; --j) {
      if (cum < need && cum + h[j] >= need) {
        sm.bin = tid * kBinsPerThread + j;
        sm.need = need - cum;
        sm.cnt = h[j];
      }
      cum += h[j];
    }
  }
  __syncthreads();
}

// Exclusive block prefix of a packed (lo16, hi16) counter pair; also returns the block total.
// `buf` alternates between calls so one __syncthreads per call is enough.
__device__ __forceinline__ uint32_t block_exclusive_scan(TopkSmem& sm, uint32_t packed, int buf, uint32_t& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t incl = packed;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += nb;
  }
  if (lane == 31) sm.warp_tot[buf][warp] = incl;
  __syncthreads();
  uint32_t wt = lane < kTopkWarps ? sm.warp_tot[buf][lane] : 0u;
  uint32_t winc = wt;
#pragma unroll
  for (int o = 1; o < kTopkWarps; o <<= 1) {
    const uint32_t nb = __shfl_up_sync(0xffffffffu, winc, o);
    if (lane >= o) winc += nb;
  }
  total = __shfl_sync(0xffffffffu, winc, kTopkWarps - 1);
  const uint32_t before = __shfl_sync(0xffffffffu, winc - wt, warp);
  return incl - packed + before;
}

__global__ void __launch_bounds__(kTopkThreads, 3)
topk_select_kernel(const float* __restrict__ logits, int64_t ld, const int32_t* __restrict__ ks,
                   const int32_t* __restrict__ ke, int T, int S, int k, int32_t* __restrict__ out) {
  __shared__ TopkSmem sm;
  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const int lo = ks ? max(ks[row], 0) : 0;
  const int hi = ke ? min(ke[row], S) : S;
  const int n = max(hi - lo, 0);
  int32_t* o = out + (int64_t)row * k;
  if (n <= k) {
    for (int j = tid; j < k; j += kTopkThreads) o[j] = j < n ? lo + j : -1;
    return;
  }
  const float* x = logits + (int64_t)row * ld;
  const bool vec = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && (ld % kVec == 0);
  const int base = lo & ~(kVec - 1);           // chunk origin: multiple of 4, <= lo

  uint32_t prefix = 0;    // value of the decided high key bits
  int pbits = 0;          // how many high bits are decided
  uint32_t need = k;      // elements still wanted from the set matching the prefix
  uint32_t cnt = 0;       // size of the threshold bin

  // ---- 1./2. histogram passes over the row ------------------------------------
  while (true) {
    const int dbits = min(kDigitBits, 32 - pbits);
    const int shift = 32 - pbits - dbits;
    const uint32_t dmask = (1u << dbits) - 1u;
    for (int b = tid; b < kBins; b += kTopkThreads) sm.hist[b] = 0;
    __syncthreads();
    if (vec) {
      // interior float4s need no window test; the (at most two) edge float4s do
      const int first_full = (lo + kVec - 1) & ~(kVec - 1);
      const int last_full = hi & ~(kVec - 1);
      if (pbits == 0) {
#pragma unroll 4
        for (int i = first_full + tid * kVec; i < last_full; i += kChunkHist) {
          const float4 f = __ldg(reinterpret_cast<const float4*>(x + i));
          atomicAdd(&sm.hist[order_key(f.x) >> shift], 1u);
          atomicAdd(&sm.hist[order_key(f.y) >> shift], 1u);
          atomicAdd(&sm.hist[order_key(f.z) >> shift], 1u);
          atomicAdd(&sm.hist[order_key(f.w) >> shift], 1u);
        }
      } else {
        const int pshift = 32 - pbits;
#pragma unroll 4
        for (int i = first_full + tid * kVec; i < last_full; i += kChunkHist) {
          const float4 f = __ldg(reinterpret_cast<const float4*>(x + i));
          const float v[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t key = order_key(v[j]);
            if ((key >> pshift) == prefix) atomicAdd(&sm.hist[(key >> shift) & dmask], 1u);
          }
        }
      }
      // edges: [lo, first_full) and [last_full, hi)
      const int n_head = min(first_full, hi) - lo;
      const int n_tail = last_full >= first_full ? hi - last_full : 0;
      if (tid < n_head + n_tail) {
        const int i = tid < n_head ? lo + tid : last_full + (tid - n_head);
        const uint32_t key = order_key(__ldg(x + i));
        if (pbits == 0 || (key >> (32 - pbits)) == prefix) atomicAdd(&sm.hist[(key >> shift) & dmask], 1u);
      }
    } else {
      for (int i = lo + tid; i < hi; i += kTopkThreads) {
        const uint32_t key = order_key(__ldg(x + i));
        if (pbits == 0 || (key >> (32 - pbits)) == prefix) atomicAdd(&sm.hist[(key >> shift) & dmask], 1u);
      }
    }
    __syncthreads();
    find_threshold_bin(sm, need);
    prefix = (pbits == 0 ? 0u : (prefix << dbits)) | sm.bin;
    need = sm.need;
    cnt = sm.cnt;
    pbits += dbits;
    __syncthreads();
    if (cnt <= (uint32_t)kCand || pbits == 32) break;
  }

  // ---- 3. ordered pass: emit what is above the threshold bin, stage the bin ----
  const uint32_t n_above = k - need;
  const bool all_tied = (pbits == 32);           // every candidate equals the k-th value
  const int pshift = 32 - pbits;
  uint32_t base_sel = 0, base_cand = 0;
  const int n_chunks = (hi - base + kChunkFinal - 1) / kChunkFinal;
  for (int c = 0; c < n_chunks; ++c) {
    const int i0 = base + c * kChunkFinal + tid * kEltPerThread;
    float v[kEltPerThread];
    uint32_t fsel = 0, fcand = 0;
    if (i0 < hi) {
      if (vec) {
#pragma unroll
        for (int q = 0; q < kEltPerThread / kVec; ++q) {
          // a float4 that starts below hi lies inside the row's allocation (ld % 4 == 0)
          const float4 f = (i0 + q * kVec < hi) ? __ldg(reinterpret_cast<const float4*>(x + i0 + q * kVec))
                                                : make_float4(0.f, 0.f, 0.f, 0.f);
          v[q * 4 + 0] = f.x; v[q * 4 + 1] = f.y; v[q * 4 + 2] = f.z; v[q * 4 + 3] = f.w;
        }
      } else {
#pragma unroll
        for (int j = 0; j < kEltPerThread; ++j) v[j] = (i0 + j >= lo && i0 + j < hi) ? __ldg(x + i0 + j) : 0.f;
      }
      const bool interior = (i0 >= lo) && (i0 + kEltPerThread <= hi);
#pragma unroll
      for (int j = 0; j < kEltPerThread; ++j) {
        const uint32_t top = pshift >= 32 ? 0u : (order_key(v[j]) >> pshift);
        const bool in = interior || (i0 + j >= lo && i0 + j < hi);
        fsel |= (uint32_t)(in && top > prefix) << j;
        fcand |= (uint32_t)(in && top == prefix) << j;
      }
    }
    const uint32_t packed = __popc(fsel) | (__popc(fcand) << 16);
    uint32_t total;
    const uint32_t excl = block_exclusive_scan(sm, packed, c & 1, total);
    if (fsel | fcand) {
      uint32_t ps = base_sel + (excl & 0xffffu);
      uint32_t pc = base_cand + (excl >> 16);
#pragma unroll
      for (int j = 0; j < kEltPerThread; ++j) {
        if (fsel & (1u << j)) {
          o[ps++] = i0 + j;
        } else if (fcand & (1u << j)) {
          if (all_tied) {
            if (pc < need) o[n_above + pc] = i0 + j;
          } else {
            sm.cand_key[pc] = order_key(v[j]);
            sm.cand_idx[pc] = i0 + j;
          }
          ++pc;
        }
      }
    }
    base_sel += total & 0xffffu;
    base_cand += total >> 16;
  }
  if (all_tied) return;
  __syncthreads();

  // ---- 4. resolve the remaining digits on the staged candidates -----------------
  uint32_t ck[kCandPerThread];
#pragma unroll
  for (int j = 0; j < kCandPerThread; ++j) {
    const uint32_t a = tid * kCandPerThread + j;        // contiguous per thread: keeps column order
    ck[j] = a < cnt ? sm.cand_key[a] : 0u;
  }
  while (pbits < 32) {
    const int dbits = min(kDigitBits, 32 - pbits);
    const int shift = 32 - pbits - dbits;
    const uint32_t dmask = (1u << dbits) - 1u;
    for (int b = tid; b < kBins; b += kTopkThreads) sm.hist[b] = 0;
    __syncthreads();
#pragma unroll
    for (int j = 0; j < kCandPerThread; ++j) {
      const uint32_t a = tid * kCandPerThread + j;
      if (a < cnt && (ck[j] >> (32 - pbits)) == prefix) atomicAdd(&sm.hist[(ck[j] >> shift) & dmask], 1u);
    }
    __syncthreads();
    find_threshold_bin(sm, need);
    prefix = (prefix << dbits) | sm.bin;
    need = sm.need;
    pbits += dbits;
    __syncthreads();
  }
  // prefix is now the exact k-th largest key; `need` of the candidates equal to it are wanted
  const uint32_t n_gt_base = k - need;                   // slots before the tied ones... filled below
  uint32_t fgt = 0, feq = 0;
#pragma unroll
  for (int j = 0; j < kCandPerThread; ++j) {
    const uint32_t a = tid * kCandPerThread + j;
    if (a < cnt) {
      fgt |= (uint32_t)(ck[j] > prefix) << j;
      feq |= (uint32_t)(ck[j] == prefix) << j;
    }
  }
  uint32_t total;
  const uint32_t excl = block_exclusive_scan(sm, __popc(fgt) | (__popc(feq) << 16), 0, total);
  // output layout: [0, n_above) above the bin, then candidates > key, then the `need` tied ones
  uint32_t pg = n_above + (excl & 0xffffu);
  uint32_t pe = excl >> 16;
  (void)n_gt_base;
#pragma unroll
  for (int j = 0; j < kCandPerThread; ++j) {
    const uint32_t a = tid * kCandPerThread + j;
    if (fgt & (1u << j)) {
      o[pg++] = sm.cand_idx[a];
    } else if (feq & (1u << j)) {
      if (pe < need) o[k - need + pe] = sm.cand_idx[a];
      ++pe;
    }
  }
}

int topk_select_launch(const float* logits, int64_t ld, const int32_t* ks, const int32_t* ke, int T, int S, int k,
                       int32_t* out, cudaStream_t stream) {
  if (T == 0 || k == 0) return DSA_OK;
  topk_select_kernel<<<T, kTopkThreads, 0, stream>>>(logits, ld, ks, ke, T, S, k, out);
  return check_launch("topk_select");
}

}  // namespace dsa
