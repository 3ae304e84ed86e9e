// Per-block FP8 e4m3 quantiser: one kernel for what the reference does with about eight eager
// torch kernels (sparse_attn/DSA.py:102-132): fp32 absmax over each block of 64 or 128 values,
// scale = max(absmax, 1e-6) / 448, q = x / scale rounded to e4m3.  Both divisions are IEEE
// round-to-nearest, so the bytes and scales equal the reference's CPU result exactly.
// HBM-bound: 2 (bf16) or 4 (fp32) bytes read and 1 byte + 4/block written per value.
#include <cuda_bf16.h>
#include <cuda_fp8.h>

#include "dsa_common.cuh"
#include "dsa_host.h"

namespace dsa {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// One warp per block of BLOCK values: lane l owns BLOCK/32 consecutive values.
template <typename T, int BLOCK>
__global__ void __launch_bounds__(256) fp8_quant_kernel(const T* __restrict__ x, int64_t n_blocks,
                                                        uint8_t* __restrict__ q, float* __restrict__ scale) {
  constexpr int PER = BLOCK / 32;
  const int lane = threadIdx.x & 31;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < n_blocks; b += warps) {
    const T* src = x + b * BLOCK + lane * PER;
    float v[PER];
    if constexpr (sizeof(T) == 2 && PER == 4) {
      const uint2 raw = __ldg(reinterpret_cast<const uint2*>(src));
      const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
      const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      v[0] = __low2float(p0); v[1] = __high2float(p0); v[2] = __low2float(p1); v[3] = __high2float(p1);
    } else if constexpr (sizeof(T) == 4 && PER == 4) {
      const float4 raw = __ldg(reinterpret_cast<const float4*>(src));
      v[0] = raw.x; v[1] = raw.y; v[2] = raw.z; v[3] = raw.w;
    } else {
#pragma unroll
      for (int i = 0; i < PER; ++i) v[i] = to_f32<T>(src[i]);
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = __fdiv_rn(fmaxf(amax, 1e-6f), 448.f);
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      packed |= (uint32_t)__nv_cvt_float_to_fp8(__fdiv_rn(v[i], sc), __NV_SATFINITE, __NV_E4M3) << (8 * i);
    if constexpr (PER == 4) {
      reinterpret_cast<uint32_t*>(q + b * BLOCK)[lane] = packed;
    } else {
      reinterpret_cast<uint16_t*>(q + b * BLOCK)[lane] = (uint16_t)packed;
    }
    if (lane == 0) scale[b] = sc;
  }
}

// RoPE on the first `rope_dim` values of every head row, then the quantiser above, in one pass over a bf16
// tensor whose rows are one FP8 block each (head_dim = BLOCK): what DsaIndexer.forward does between its
// projections and the scorer (sparse_attn/DSA.py:513-524, 530-531) with a dozen eager kernels and an fp32
// intermediate four times the size of the input.  The arithmetic keeps the reference's order and roundings,
// so the bytes and scales equal those of the eager chain:
//   NeoX form (halves):   y[i] = x[i] c - x[i+h] s,  y[i+h] = x[i] s + x[i+h] c   in fp32, each product and the
//                         sum rounded separately (separate torch ops: no fused multiply-add), NOT rounded to bf16;
//   interleaved (GPT-J):  the same on (even, odd) pairs, result rounded to bf16 (the reference writes it into a
//                         tensor of x's dtype).
// Row r belongs to position r / rows_per_pos (query rows: heads per token; key rows: 1).  One warp per row.
template <int BLOCK, bool INTERLEAVE>
__global__ void __launch_bounds__(256) rope_fp8_quant_kernel(const __nv_bfloat16* __restrict__ x, int64_t n_rows, int rope_dim,
                                                             int rows_per_pos, const float* __restrict__ cos_t,
                                                             const float* __restrict__ sin_t, uint8_t* __restrict__ q,
                                                             float* __restrict__ scale) {
  constexpr int PER = BLOCK / 32;
  const int lane = threadIdx.x & 31;
  const int half = rope_dim >> 1;
  const int64_t warps = (int64_t)gridDim.x * (blockDim.x >> 5);
  for (int64_t b = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); b < n_rows; b += warps) {
    const __nv_bfloat16* src = x + b * BLOCK + lane * PER;
    float v[PER];
    if constexpr (PER == 4) {
      const uint2 raw = __ldg(reinterpret_cast<const uint2*>(src));
      const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
      const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
      v[0] = __low2float(p0); v[1] = __high2float(p0); v[2] = __low2float(p1); v[3] = __high2float(p1);
    } else {
      const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(src);
      v[0] = __low2float(p0); v[1] = __high2float(p0);
    }
    const int64_t pos = b / rows_per_pos;
    const float* cr = cos_t + pos * half;
    const float* sr = sin_t + pos * half;
    const int d0 = lane * PER;                          // first dim of this lane
    if constexpr (INTERLEAVE) {
      if (d0 < rope_dim) {
#pragma unroll
        for (int i = 0; i < PER; i += 2) {
          const float c = __ldg(cr + ((d0 + i) >> 1)), s = __ldg(sr + ((d0 + i) >> 1));
          const float e = __fsub_rn(__fmul_rn(v[i], c), __fmul_rn(v[i + 1], s));
          const float o = __fadd_rn(__fmul_rn(v[i], s), __fmul_rn(v[i + 1], c));
          v[i] = __bfloat162float(__float2bfloat16_rn(e));
          v[i + 1] = __bfloat162float(__float2bfloat16_rn(o));
        }
      }
    } else {
      // partner lane holds the other half of the pair (half / PER lanes away); every lane takes part in the shuffle
      const int shift = half / PER;
      float other[PER];
#pragma unroll
      for (int i = 0; i < PER; ++i) other[i] = __shfl_xor_sync(0xffffffffu, v[i], shift);
      if (d0 < rope_dim) {
        const bool first = d0 < half;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
          const int t = first ? d0 + i : d0 + i - half;
          const float c = __ldg(cr + t), s = __ldg(sr + t);
          v[i] = first ? __fsub_rn(__fmul_rn(v[i], c), __fmul_rn(other[i], s))      // x1 c - x2 s
                       : __fadd_rn(__fmul_rn(other[i], s), __fmul_rn(v[i], c));     // x1 s + x2 c
        }
      }
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) amax = fmaxf(amax, fabsf(v[i]));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float sc = __fdiv_rn(fmaxf(amax, 1e-6f), 448.f);
    uint32_t packed = 0;
#pragma unroll
    for (int i = 0; i < PER; ++i)
      packed |= (uint32_t)__nv_cvt_float_to_fp8(__fdiv_rn(v[i], sc), __NV_SATFINITE, __NV_E4M3) << (8 * i);
    if constexpr (PER == 4) {
      reinterpret_cast<uint32_t*>(q + b * BLOCK)[lane] = packed;
    } else {
      reinterpret_cast<uint16_t*>(q + b * BLOCK)[lane] = (uint16_t)packed;
    }
    if (lane == 0) scale[b] = sc;
  }
}

int rope_fp8_quant_launch(const void* x, int64_t n_rows, int head_dim, int rope_dim, int interleave, int rows_per_pos,
                          const float* cos_t, const float* sin_t, void* q, float* scale, cudaStream_t stream) {
  if (n_rows == 0) return DSA_OK;
  const int64_t want = (n_rows + 7) / 8;
  const int grid = (int)(want < (int64_t)sm_count() * 16 ? want : (int64_t)sm_count() * 16);
  const __nv_bfloat16* xi = static_cast<const __nv_bfloat16*>(x);
  uint8_t* qo = static_cast<uint8_t*>(q);
#define DSA_ROPE_CASE(B, I) rope_fp8_quant_kernel<B, I><<<grid, 256, 0, stream>>>(xi, n_rows, rope_dim, rows_per_pos, cos_t, sin_t, qo, scale)
  if (head_dim == 128 && interleave) DSA_ROPE_CASE(128, true);
  else if (head_dim == 128) DSA_ROPE_CASE(128, false);
  else if (head_dim == 64 && interleave) DSA_ROPE_CASE(64, true);
  else if (head_dim == 64) DSA_ROPE_CASE(64, false);
  else return set_error(DSA_ERR_SHAPE, "rope_fp8_quant: head dim %d not supported (64 or 128)", head_dim);
#undef DSA_ROPE_CASE
  return check_launch("rope_fp8_quant");
}

int fp8_quant_launch(const void* x, int x_is_bf16, int64_t n_blocks, int block, void* q, float* scale,
                     cudaStream_t stream) {
  if (n_blocks == 0) return DSA_OK;
  const int64_t want = (n_blocks + 7) / 8;
  const int grid = (int)(want < (int64_t)sm_count() * 16 ? want : (int64_t)sm_count() * 16);
  uint8_t* qo = static_cast<uint8_t*>(q);
  if (block == 128 && x_is_bf16)
    fp8_quant_kernel<__nv_bfloat16, 128><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), n_blocks, qo, scale);
  else if (block == 128)
    fp8_quant_kernel<float, 128><<<grid, 256, 0, stream>>>(static_cast<const float*>(x), n_blocks, qo, scale);
  else if (block == 64 && x_is_bf16)
    fp8_quant_kernel<__nv_bfloat16, 64><<<grid, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(x), n_blocks, qo, scale);
  else if (block == 64)
    fp8_quant_kernel<float, 64><<<grid, 256, 0, stream>>>(static_cast<const float*>(x), n_blocks, qo, scale);
  else
    return set_error(DSA_ERR_SHAPE, "fp8_quant: block size %d not supported (64 or 128)", block);
  return check_launch("fp8_quant");
}

}  // namespace dsa
