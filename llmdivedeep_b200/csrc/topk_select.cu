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
//
// Long rows first try a single pass: a sample of the row (one 128-float block in
// every 16 or more) is ranked in shared memory, a threshold a few standard
// deviations below the sample's estimate of the k-th value is taken from it, and one
// ordered pass stages every element at or above that threshold (at most 4096) as a
// candidate; step 4 then runs on the candidates alone.  If the staged count turns
// out below k or above 4096 the row falls back to steps 1-4, so the result never
// depends on the sample.
#include <math_constants.h>

#include <cstdlib>

#include "dsa_common.cuh"
#include "dsa_host.h"

namespace dsa {

constexpr int kTopkThreads = 512;
constexpr int kTopkWarps = kTopkThreads / 32;
constexpr int kDigitBits = 12;
constexpr int kBins = 1 << kDigitBits;
constexpr int kBinsPerThread = kBins / kTopkThreads;   // 8
constexpr int kCand = 2048;                            // two-pass path: largest threshold bin staged
constexpr int kCandPerThread = kCand / kTopkThreads;   // 4
constexpr int kCandS = 4096;                           // sampled path: candidate capacity
constexpr int kCandSPerThread = kCandS / kTopkThreads; // 8
constexpr int kSampleBlock = 128;                      // floats per sampled block (one float4 per lane)
constexpr int kSampleMaxBlocks = 64;                   // at most 8192 sampled values
constexpr int kSamplePerThread = kSampleMaxBlocks / kTopkWarps * 4;   // 16
constexpr int kSampleMinRow = 16384;
constexpr int kRun = 32;                               // sampled path: contiguous columns per thread per chunk
constexpr int kChunkRun = kTopkThreads * kRun;                   // shorter rows take the two-pass path
constexpr int kVec = 4;
constexpr int kEltPerThread = 16;                      // final pass: 4 x float4, contiguous
constexpr int kChunkHist = kTopkThreads * kVec;        // histogram pass: coalesced float4
constexpr int kChunkFinal = kTopkThreads * kEltPerThread;

__device__ __forceinline__ uint32_t order_key(float x) {
  const uint32_t u = __float_as_uint(x);
  return u ^ (static_cast<uint32_t>(static_cast<int32_t>(u) >> 31) | 0x80000000u);
}

// hist and cand_key share storage: candidate keys are copied to registers (followed by a block
// barrier) before the histogram is next cleared, and the histogram is dead while candidates are staged.
struct alignas(16) TopkSmem {
  union {
    uint32_t hist[kBins];
    uint32_t cand_key[kCandS];
  };
  int32_t cand_idx[kCandS];
  uint32_t warp_tot[2][kTopkWarps];
  uint32_t bin, need, cnt;
};
static_assert(kBins == kCandS, "hist and cand_key are one array");

__device__ __forceinline__ void zero_hist(TopkSmem& sm) {
  uint4* h4 = reinterpret_cast<uint4*>(sm.hist);
#pragma unroll
  for (int b = threadIdx.x; b < kBins / 4; b += kTopkThreads) h4[b] = make_uint4(0u, 0u, 0u, 0u);
}

// Block-wide: given hist[], find the bin b with  sum(hist[b+1..]) < need <= sum(hist[b..]).
// Leaves bin / need (remaining within the bin) / cnt (= hist[b]) in shared memory.
__device__ __forceinline__ void find_threshold_bin(TopkSmem& sm, uint32_t need) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t h[kBinsPerThread];
  uint32_t mine = 0;
#pragma unroll
  for (int j = 0; j < kBinsPerThread; j += 4) {
    const uint4 q = *reinterpret_cast<const uint4*>(&sm.hist[tid * kBinsPerThread + j]);
    h[j] = q.x; h[j + 1] = q.y; h[j + 2] = q.z; h[j + 3] = q.w;
    mine += q.x + q.y + q.z + q.w;
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

// Digit passes over keys held in registers (bit j of `valid` says whether ck[j] counts): refines
// (prefix, pbits, need) 12 bits at a time until `stop_bits` key bits are decided.  Ends on a block barrier.
template <int NPT>
__device__ __forceinline__ void digit_passes(TopkSmem& sm, const uint32_t (&ck)[NPT], uint32_t valid, uint32_t& prefix,
                                             int& pbits, uint32_t& need, int stop_bits) {
  while (pbits < stop_bits) {
    const int dbits = min(kDigitBits, 32 - pbits);
    const int shift = 32 - pbits - dbits;
    const uint32_t dmask = (1u << dbits) - 1u;
    zero_hist(sm);
    __syncthreads();
#pragma unroll
    for (int j = 0; j < NPT; ++j) {
      const bool match = pbits == 0 || (ck[j] >> (32 - pbits)) == prefix;
      if (((valid >> j) & 1u) && match) atomicAdd(&sm.hist[(ck[j] >> shift) & dmask], 1u);
    }
    __syncthreads();
    find_threshold_bin(sm, need);
    prefix = (pbits == 0 ? 0u : (prefix << dbits)) | sm.bin;
    need = sm.need;
    pbits += dbits;
    __syncthreads();
  }
}

// Ordered emission of staged candidates (thread t holds candidates [t*NPT, t*NPT+NPT) in column order):
// those above the exact k-th key `kth` go to o[n_above...], the first `need` equal to it fill the tail.
template <int NPT>
__device__ __forceinline__ void emit_candidates(TopkSmem& sm, const uint32_t (&ck)[NPT], uint32_t valid, uint32_t kth,
                                                uint32_t need, uint32_t n_above, int k, int32_t* __restrict__ o) {
  const int tid = threadIdx.x;
  uint32_t fgt = 0, feq = 0;
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    if ((valid >> j) & 1u) {
      fgt |= (uint32_t)(ck[j] > kth) << j;
      feq |= (uint32_t)(ck[j] == kth) << j;
    }
  }
  uint32_t total;
  const uint32_t excl = block_exclusive_scan(sm, __popc(fgt) | (__popc(feq) << 16), 0, total);
  uint32_t pg = n_above + (excl & 0xffffu);
  uint32_t pe = excl >> 16;
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    const uint32_t a = tid * NPT + j;
    if (fgt & (1u << j)) {
      o[pg++] = sm.cand_idx[a];
    } else if (feq & (1u << j)) {
      if (pe < need) o[k - need + pe] = sm.cand_idx[a];
      ++pe;
    }
  }
}

// Staging test of the sampled pass on the raw float bits u, exact for every bit pattern:
// key(u) >= thr.  tfb holds the float bits whose key is thr.  For a threshold that is a non-negative
// float a signed compare does it (negative floats are negative integers, a positive NaN is the largest);
// for a negative threshold an unsigned one does (every non-negative float lies below the sign bit).
template <bool NEG>
__device__ __forceinline__ bool at_or_above(float v, uint32_t tfb) {
  const uint32_t u = __float_as_uint(v);
  return NEG ? (u <= tfb) : (static_cast<int32_t>(u) >= static_cast<int32_t>(tfb));
}

// One 16384-column chunk of the sampled pass: warp w owns columns [w*1024, w*1024+1024) of the chunk and
// reads them as 8 coalesced float4 rows.  Returns the hit flags of this lane, bit q*4+e for column
// wbase + q*128 + lane*4 + e.
template <bool NEG>
__device__ __forceinline__ uint32_t chunk_flags(const float* __restrict__ x, int wbase, int lane, int lo, int hi,
                                                uint32_t tfb) {
  uint32_t fc = 0;
  if (wbase >= lo && wbase + kRun * 32 <= hi) {
#pragma unroll
    for (int q = 0; q < kRun / kVec; ++q) {
      const float4 f = __ldg(reinterpret_cast<const float4*>(x + wbase + q * 128 + lane * kVec));
      if (at_or_above<NEG>(f.x, tfb)) fc |= 1u << (q * 4 + 0);
      if (at_or_above<NEG>(f.y, tfb)) fc |= 1u << (q * 4 + 1);
      if (at_or_above<NEG>(f.z, tfb)) fc |= 1u << (q * 4 + 2);
      if (at_or_above<NEG>(f.w, tfb)) fc |= 1u << (q * 4 + 3);
    }
  } else if (wbase < hi && wbase + kRun * 32 > lo) {
    for (int q = 0; q < kRun / kVec; ++q) {
      const int i = wbase + q * 128 + lane * kVec;
      if (i < hi && i + kVec > lo) {         // a float4 that starts below hi lies inside the row's allocation
        const float4 f = __ldg(reinterpret_cast<const float4*>(x + i));
        const float v[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
        for (int e2 = 0; e2 < kVec; ++e2)
          if (i + e2 >= lo && i + e2 < hi && at_or_above<NEG>(v[e2], tfb)) fc |= 1u << (q * 4 + e2);
      }
    }
  }
  return fc;
}

__device__ __forceinline__ uint32_t stage_hits(TopkSmem& sm, const float* __restrict__ x, int wbase, int lane,
                                               uint32_t fc, uint32_t pc) {
  while (fc) {                               // few bits set: reload the hits (L1) rather than keep 32 values
    const int j = __ffs(fc) - 1;
    fc &= fc - 1;
    const int col = wbase + (j >> 2) * 128 + lane * kVec + (j & 3);
    sm.cand_key[pc] = order_key(__ldg(x + col));
    sm.cand_idx[pc] = col;
    ++pc;
  }
  return pc;
}

// The ordered pass of the sampled path: stages every element with key >= thr, two chunks per block scan.
// Candidates end up in a fixed order (chunk, thread, column) that does not depend on timing.
// Returns the staged count, or 0xffffffff once it would exceed the capacity (uniform over the block).
template <bool NEG>
__device__ __forceinline__ uint32_t stage_row(TopkSmem& sm, const float* __restrict__ x, int lo, int hi, uint32_t tfb) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int base = lo & ~(kVec - 1);
  const int n_pairs = (hi - base + 2 * kChunkRun - 1) / (2 * kChunkRun);
  uint32_t staged = 0;
  for (int c = 0; c < n_pairs; ++c) {
    const int wb0 = base + (2 * c) * kChunkRun + warp * (kRun * 32);
    const int wb1 = wb0 + kChunkRun;
    const uint32_t f0 = chunk_flags<NEG>(x, wb0, lane, lo, hi, tfb);
    const uint32_t f1 = chunk_flags<NEG>(x, wb1, lane, lo, hi, tfb);
    uint32_t total;
    const uint32_t excl = block_exclusive_scan(sm, __popc(f0) | (__popc(f1) << 16), c & 1, total);
    const uint32_t t0 = total & 0xffffu, t1 = total >> 16;
    if (staged + t0 + t1 > (uint32_t)kCandS) return 0xffffffffu;   // every thread sees the same totals
    stage_hits(sm, x, wb0, lane, f0, staged + (excl & 0xffffu));
    stage_hits(sm, x, wb1, lane, f1, staged + t0 + (excl >> 16));
    staged += t0 + t1;
  }
  __syncthreads();
  return staged;
}

// Emission for the sampled path, whose candidates are not in column order: candidates above the exact k-th
// key `kth` first, then `need` of those equal to it -- the ones in the lowest columns, found by a second
// radix select on the column numbers when there are more ties than wanted.
template <int NPT>
__device__ __forceinline__ void emit_unordered(TopkSmem& sm, const uint32_t (&ck)[NPT], uint32_t valid, uint32_t kth,
                                               uint32_t need, int k, int32_t* __restrict__ o) {
  const int tid = threadIdx.x;
  uint32_t fgt = 0, feq = 0;
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    if ((valid >> j) & 1u) {
      fgt |= (uint32_t)(ck[j] > kth) << j;
      feq |= (uint32_t)(ck[j] == kth) << j;
    }
  }
  uint32_t total;
  uint32_t excl = block_exclusive_scan(sm, __popc(fgt) | (__popc(feq) << 16), 0, total);
  uint32_t tkey[NPT];                         // complement of the column: lowest column = largest key
#pragma unroll
  for (int j = 0; j < NPT; ++j) tkey[j] = ~static_cast<uint32_t>(sm.cand_idx[tid * NPT + j]);
  uint32_t pg = excl & 0xffffu;
#pragma unroll
  for (int j = 0; j < NPT; ++j)
    if (fgt & (1u << j)) o[pg++] = static_cast<int32_t>(~tkey[j]);
  if ((total >> 16) > need) {                 // uniform: more ties than wanted, keep the lowest columns
    uint32_t prefix = 0, need2 = need;
    int pbits = 0;
    __syncthreads();                          // the scan above is done with warp_tot before hist work starts
    digit_passes<NPT>(sm, tkey, feq, prefix, pbits, need2, 32);
#pragma unroll
    for (int j = 0; j < NPT; ++j)
      if (tkey[j] < prefix) feq &= ~(1u << j);
    excl = block_exclusive_scan(sm, __popc(feq) << 16, 1, total);
  }
  uint32_t pe = k - need + (excl >> 16);
#pragma unroll
  for (int j = 0; j < NPT; ++j)
    if (feq & (1u << j)) o[pe++] = static_cast<int32_t>(~tkey[j]);
}

// The threshold of the sampled pass: the key a few standard deviations below the sample's estimate of the k-th value.
// Returns false (for every thread of the block alike) when the geometry of the row rules the sampled pass out.  The
// result depends on the row alone, so every CTA that evaluates it for one row gets the same key.
__device__ __forceinline__ bool sample_threshold(TopkSmem& sm, const float* __restrict__ x, int lo, int hi, int k,
                                                 uint32_t& thr_out) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n = hi - lo;
  const int first = (lo + kVec - 1) & ~(kVec - 1);
  const int nblk = (hi - first) / kSampleBlock;
  const int sb = max(16, (nblk + kSampleMaxBlocks - 1) / kSampleMaxBlocks);   // one block sampled in every sb
  const int mblk = nblk / sb;
  const int m = mblk * kSampleBlock;
  const float frac = (float)m / (float)n;
  const float mu = (float)k * frac;                       // top-k elements expected inside the sample
  const float rf = ceilf(mu + 4.f * sqrtf(mu) + 2.f);     // rank taken: about 4 sigma below the k-th value
  if (m < 1024 || rf > (float)m || rf > 0.8f * (float)kCandS * frac) return false;

  // ---- sample: up to 4 blocks per warp, one float4 per lane -----------------------
  uint32_t skey[kSamplePerThread];
  uint32_t svalid = 0;
#pragma unroll
  for (int i = 0; i < kSamplePerThread / 4; ++i) {
    const int j = warp + kTopkWarps * i;
    float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
    if (j < mblk) {
      f = __ldg(reinterpret_cast<const float4*>(x + first + (j * sb + sb / 2) * kSampleBlock + lane * kVec));
      svalid |= 0xFu << (4 * i);
    }
    skey[4 * i + 0] = order_key(f.x); skey[4 * i + 1] = order_key(f.y);
    skey[4 * i + 2] = order_key(f.z); skey[4 * i + 3] = order_key(f.w);
  }
  // The rf-th largest sample key, to 4096 key steps, in one histogram pass: bins count down from a
  // base near the top of the sample (the smallest of the warps' maxima, which one outlier cannot move),
  // so the digits are mantissa bits and spread over the bins.  Keys more than 2^24 steps below the base
  // are left out; if fewer than rf keys remain the generic digit passes take over.
  uint32_t wmax = 0;
#pragma unroll
  for (int j = 0; j < kSamplePerThread; ++j)
    if ((svalid >> j) & 1u) wmax = max(wmax, skey[j]);
  wmax = __reduce_max_sync(0xffffffffu, wmax);
  if (lane == 0) sm.warp_tot[0][warp] = (svalid != 0u) ? wmax : 0xffffffffu;
  if (tid == 0) sm.bin = 0xffffffffu;
  zero_hist(sm);
  __syncthreads();
  const uint32_t key_base = __reduce_min_sync(0xffffffffu, lane < kTopkWarps ? sm.warp_tot[0][lane] : 0xffffffffu);
#pragma unroll
  for (int j = 0; j < kSamplePerThread; ++j) {
    if ((svalid >> j) & 1u) {
      if (skey[j] >= key_base) {
        atomicAdd(&sm.hist[kBins - 1], 1u);
      } else {
        const uint32_t q = (key_base - skey[j] - 1u) >> 12;
        if (q < (uint32_t)(kBins - 1)) atomicAdd(&sm.hist[kBins - 2 - q], 1u);
      }
    }
  }
  __syncthreads();
  uint32_t prefix = 0, need = (uint32_t)rf;
  int pbits = 0;
  find_threshold_bin(sm, need);
  uint32_t thr;
  if (sm.bin != 0xffffffffu) {
    const uint32_t below = (uint32_t)(kBins - 1 - sm.bin) << 12;       // lower edge of the bin, in key steps below the base
    thr = key_base > below ? key_base - below : 0u;
    __syncthreads();
  } else {
    __syncthreads();
    digit_passes<kSamplePerThread>(sm, skey, svalid, prefix, pbits, need, 24);
    thr = prefix << 8;                                    // lower edge of the 24-bit bin of the sample's rf-th key
  }
  thr_out = thr;
  return true;
}

// One ordered pass over columns [lo, hi) of the row: stages everything whose key is at or above thr.
// Returns the staged count, or 0xffffffff once it would exceed the capacity (uniform over the block).
__device__ __forceinline__ uint32_t stage_above(TopkSmem& sm, const float* __restrict__ x, int lo, int hi, uint32_t thr) {
  const bool neg = (thr & 0x80000000u) == 0u;             // the threshold is a negative float
  const uint32_t tfb = neg ? ~thr : (thr ^ 0x80000000u);  // its bits as a float
  return neg ? stage_row<true>(sm, x, lo, hi, tfb) : stage_row<false>(sm, x, lo, hi, tfb);
}

// The exact k-th key among `staged` candidates (all with key >= thr, in any order) and the output.
// Offsets d = key - thr are >= 0; when all are below 2^24 (floats within a few binades of the
// threshold) two 12-bit passes over d << 8 settle it, and their digits are mantissa bits, which
// spread over the histogram instead of piling onto a few exponent bins.
__device__ __forceinline__ void select_among_staged(TopkSmem& sm, uint32_t staged, uint32_t thr, int k,
                                                    int32_t* __restrict__ o) {
  const int tid = threadIdx.x;
  uint32_t prefix, need;
  int pbits;
  uint32_t ck[kCandSPerThread];
  uint32_t valid = 0;
  int wide = 0;
#pragma unroll
  for (int j = 0; j < kCandSPerThread; ++j) {
    const uint32_t a = tid * kCandSPerThread + j;
    const bool ok = a < staged;
    ck[j] = ok ? sm.cand_key[a] - thr : 0u;
    valid |= (uint32_t)ok << j;
    wide |= (ck[j] >> 24) != 0u;
  }
  wide = __syncthreads_or(wide);                           // also: keys are in registers, hist may reuse the storage
  prefix = 0; pbits = 0; need = (uint32_t)k;
  uint32_t kth_off;
  if (!wide) {
#pragma unroll
    for (int j = 0; j < kCandSPerThread; ++j) ck[j] <<= 8;
    digit_passes<kCandSPerThread>(sm, ck, valid, prefix, pbits, need, 24);
    kth_off = prefix << 8;
  } else {
    digit_passes<kCandSPerThread>(sm, ck, valid, prefix, pbits, need, 32);
    kth_off = prefix;
  }
  emit_unordered<kCandSPerThread>(sm, ck, valid, kth_off, need, k, o);
}

// Single pass over a long row, steered by a sample.  Returns false (for every thread of the block alike)
// when the row has to take the two-pass path: geometry out of range, or the staged count missed [k, 4096].
// Needs 16-byte aligned rows.
__device__ __forceinline__ bool sampled_single_pass(TopkSmem& sm, const float* __restrict__ x, int lo, int hi, int k,
                                                    int32_t* __restrict__ o) {
  uint32_t thr;
  if (!sample_threshold(sm, x, lo, hi, k, thr)) return false;
  const uint32_t staged = stage_above(sm, x, lo, hi, thr);
  if (staged == 0xffffffffu || staged < (uint32_t)k) return false;   // missed [k, capacity]: two-pass path
  select_among_staged(sm, staged, thr, k, o);
  return true;
}

// One row, one CTA: the whole selection.
__device__ __forceinline__ void topk_row(TopkSmem& sm, const float* __restrict__ logits, int64_t ld,
                                         const int32_t* __restrict__ ks, const int32_t* __restrict__ ke, int S, int k,
                                         int32_t* __restrict__ out, int sample, int row) {
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

  if (vec && n >= kSampleMinRow && sample) {
    if (sampled_single_pass(sm, x, lo, hi, k, o)) return;
    __syncthreads();
  }

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
  uint32_t valid = 0;
#pragma unroll
  for (int j = 0; j < kCandPerThread; ++j) {
    const uint32_t a = tid * kCandPerThread + j;        // contiguous per thread: keeps column order
    ck[j] = a < cnt ? sm.cand_key[a] : 0u;
    valid |= (uint32_t)(a < cnt) << j;
  }
  __syncthreads();                                      // keys are in registers: hist may reuse the storage
  digit_passes<kCandPerThread>(sm, ck, valid, prefix, pbits, need, 32);
  // prefix is now the exact k-th largest key; `need` of the candidates equal to it are wanted.
  // Output layout: [0, n_above) above the bin, then candidates > key, then the `need` tied ones.
  emit_candidates<kCandPerThread>(sm, ck, valid, prefix, need, n_above, k, o);
}

__global__ void __launch_bounds__(kTopkThreads, 3)
topk_select_kernel(const float* __restrict__ logits, int64_t ld, const int32_t* __restrict__ ks,
                   const int32_t* __restrict__ ke, int T, int S, int k, int32_t* __restrict__ out, int sample) {
  __shared__ TopkSmem sm;
  topk_row(sm, logits, ld, ks, ke, S, k, out, sample, blockIdx.x);
}

// sample = 0 forces the two-pass path on every row (the test hook that pits the two paths against each other)
int topk_select_launch(const float* logits, int64_t ld, const int32_t* ks, const int32_t* ke, int T, int S, int k,
                       int32_t* out, int sample, cudaStream_t stream) {
  if (T == 0 || k == 0) return DSA_OK;
  // (Tried for few long rows, i.e. decode: a cluster of four CTAs per row, each staging a quarter of the columns and
  // CTA 0 collecting the candidates through distributed shared memory.  Same output, order included, and 22.2 us
  // against 23.0 for 64 rows of 131072.  In cycles per row: one CTA spends 5600 on the sample and threshold, 22200 on
  // the staging pass, 9900 on the exact select and the output; the cluster 6100 + 7100 + 10800, but also 3500 in its
  // two cluster barriers and 4100 pulling ~2100 candidates across.)
  topk_select_kernel<<<T, kTopkThreads, 0, stream>>>(logits, ld, ks, ke, T, S, k, out, sample);
  return check_launch("topk_select");
}

}  // namespace dsa
