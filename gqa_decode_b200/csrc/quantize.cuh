// Per-KV-head E4M3 quantisation of a K or V cache on the GPU: the producer of the FP8
// decode kernels' input format.  Same arithmetic as the reference's quantize_kv_fp8
// (gqa_decode/fp8_utils.py:23-41), which runs it as half a dozen full passes of tensor
// ops: amax over each head clamped to >= 1e-12, scale = amax / 448,
// code = e4m3(clamp(float(x) / amax * 448, +-448)) with round-to-nearest-even.
// Two HBM-bound kernels: an absolute-maximum pass (2 B/element read) and a convert pass
// (2 B read + 1 B written per element).
#pragma once
#include <cuda_fp8.h>

#include "ptx.cuh"
#include "schedule.cuh"

namespace gqa {

constexpr int kQuantThreads = 256;

// amax[g] = max |x| over group g; `amax` must be zero on entry.  |x| >= 0, so the float
// bit patterns order like unsigned integers and atomicMax on them is exact.
template <typename T16>
__global__ void __launch_bounds__(kQuantThreads)
amax_kernel(const T16* __restrict__ x, long long elems_per_group, float* __restrict__ amax) {
  const long long g = blockIdx.y;
  const uint4* p = reinterpret_cast<const uint4*>(x + g * elems_per_group);
  const long long n8 = elems_per_group / 8;
  float m = 0.f;
#pragma unroll 4
  for (long long i = (long long)blockIdx.x * kQuantThreads + threadIdx.x; i < n8;
       i += (long long)gridDim.x * kQuantThreads) {
    const uint4 v = __ldg(p + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const T16 lo = *reinterpret_cast<const T16*>(&w[j]);
      const T16 hi = *(reinterpret_cast<const T16*>(&w[j]) + 1);
      m = fmaxf(m, fmaxf(fabsf(Mma16<T16>::to_float(lo)), fabsf(Mma16<T16>::to_float(hi))));
    }
  }
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  __shared__ float part[kQuantThreads / 32];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < kQuantThreads / 32; ++i) m = fmaxf(m, part[i]);
    atomicMax(reinterpret_cast<unsigned*>(amax + g), __float_as_uint(m));
  }
}

// x / a, correctly rounded, for many x and one divisor a whose correctly rounded reciprocal is
// r: the quotient estimate x * r corrected once with the exact remainder (two fused
// multiply-adds instead of the dozen instructions of a general division).  Exact whenever
// the significand of a is not all ones and r is a normal number - a is a 16-bit float's
// value here (8 or 11 significant bits; checked against the division for every pair of
// significands), and divisors beyond 2^100, whose reciprocals are subnormal, take the general
// division.
__device__ __forceinline__ float divide_by(float x, float a, float r) {
  if (a > 0x1p100f) return __fdiv_rn(x, a);
  const float q = __fmul_rn(x, r);
  return __fmaf_rn(__fmaf_rn(-a, q, x), r, q);
}

// Eight 16-bit values -> eight E4M3 codes: float(x) / amax * 448 rounded to nearest even.  The
// reference's clamp to +-448 never acts here (|x| <= amax, so the quotient is at most 1 and the
// product at most 448); the conversion saturates finite values on its own.
template <typename T16>
__device__ __forceinline__ uint2 quantize8(const uint4 v, float a, float r) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t out[2] = {0u, 0u};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const T16 lo = *reinterpret_cast<const T16*>(&w[j]);
    const T16 hi = *(reinterpret_cast<const T16*>(&w[j]) + 1);
    const float f0 = __fmul_rn(divide_by(Mma16<T16>::to_float(lo), a, r), 448.f);
    const float f1 = __fmul_rn(divide_by(Mma16<T16>::to_float(hi), a, r), 448.f);
    const unsigned short pr = __nv_cvt_float2_to_fp8x2(make_float2(f0, f1), __NV_SATFINITE, __NV_E4M3);
    out[j >> 1] |= (uint32_t)pr << (16 * (j & 1));
  }
  return make_uint2(out[0], out[1]);
}

template <typename T16>
__global__ void __launch_bounds__(kQuantThreads)
quantize_kernel(const T16* __restrict__ x, long long elems_per_group, const float* __restrict__ amax,
                uint8_t* __restrict__ codes, float* __restrict__ scale) {
  const long long g = blockIdx.y;
  const float a = fmaxf(amax[g], 1e-12f);
  const float r = __frcp_rn(a);
  if (blockIdx.x == 0 && threadIdx.x == 0) scale[g] = __fdiv_rn(a, 448.f);
  const uint4* p = reinterpret_cast<const uint4*>(x + g * elems_per_group);
  uint2* q = reinterpret_cast<uint2*>(codes + g * elems_per_group);
  const long long n8 = elems_per_group / 8;
  const long long stride = (long long)gridDim.x * kQuantThreads;
  long long i = (long long)blockIdx.x * kQuantThreads + threadIdx.x;
  // four 16-byte loads in flight per thread before the first conversion
  constexpr int kAhead = 4;
  for (; i + (kAhead - 1) * stride < n8; i += kAhead * stride) {
    uint4 v[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) v[u] = __ldg(p + i + u * stride);
#pragma unroll
    for (int u = 0; u < kAhead; ++u) q[i + u * stride] = quantize8<T16>(v[u], a, r);
  }
  for (; i < n8; i += stride) q[i] = quantize8<T16>(__ldg(p + i), a, r);
}

// Append one token per sequence to E4M3 caches whose per-(sequence, head) scales are
// already fixed: code = e4m3(clamp(float(x) / amax * 448, +-448)) with amax = scale * 448,
// i.e. the arithmetic above with the stored scale (values beyond the head's range saturate
// and are counted).  One block per (sequence, KV head), four elements per thread.
struct AppendParams {
  const void* k_new;       // [batch, Hkv, D] 16-bit
  const void* v_new;
  uint8_t* k_cache;        // E4M3 codes, padded or paged layout
  uint8_t* v_cache;
  const float* k_scale;    // [batch * Hkv]
  const float* v_scale;
  const int* positions;    // [batch] row the token goes to
  const int* block_table;  // paged layouts
  int* saturated;          // optional counter of clamped elements
  int num_kv_heads, head_dim, max_seq, layout, page_size, table_stride;
};

template <typename T16>
__global__ void append_quantize_kernel(const AppendParams p) {
  const int g = blockIdx.x, b = g / p.num_kv_heads, h = g % p.num_kv_heads;
  const int pos = __ldg(p.positions + b);
  if (pos < 0 || pos >= p.max_seq) return;  // nothing to write: the caller sized the cache
  long long row;  // row of D codes inside the cache
  if (p.layout == kLayoutPadded) {
    row = (long long)g * p.max_seq + pos;
  } else {
    const int page = __ldg(p.block_table + (long long)b * p.table_stride + pos / p.page_size);
    const int off = pos % p.page_size;
    row = p.layout == kLayoutPagedHnd
              ? ((long long)page * p.num_kv_heads + h) * p.page_size + off
              : ((long long)page * p.page_size + off) * p.num_kv_heads + h;
  }
  const int d = 4 * threadIdx.x;
  int clamped = 0;
#pragma unroll
  for (int which = 0; which < 2; ++which) {
    const T16* src = static_cast<const T16*>(which ? p.v_new : p.k_new) + (long long)g * p.head_dim + d;
    uint8_t* dst = (which ? p.v_cache : p.k_cache) + row * p.head_dim + d;
    const float a = fmaxf(__fmul_rn(__ldg((which ? p.v_scale : p.k_scale) + g), 448.f), 1e-12f);
    const uint2 v = *reinterpret_cast<const uint2*>(src);
    const uint32_t w[2] = {v.x, v.y};
    uint32_t out = 0u;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const T16 lo = *reinterpret_cast<const T16*>(&w[j]);
      const T16 hi = *(reinterpret_cast<const T16*>(&w[j]) + 1);
      float f0 = __fmul_rn(__fdiv_rn(Mma16<T16>::to_float(lo), a), 448.f);
      float f1 = __fmul_rn(__fdiv_rn(Mma16<T16>::to_float(hi), a), 448.f);
      clamped += (fabsf(f0) > 448.f) + (fabsf(f1) > 448.f);
      f0 = fminf(fmaxf(f0, -448.f), 448.f);
      f1 = fminf(fmaxf(f1, -448.f), 448.f);
      const unsigned short pr = __nv_cvt_float2_to_fp8x2(make_float2(f0, f1), __NV_SATFINITE, __NV_E4M3);
      out |= (uint32_t)pr << (16 * j);
    }
    *reinterpret_cast<uint32_t*>(dst) = out;
  }
  if (p.saturated && clamped) atomicAdd(p.saturated, clamped);
}

}  // namespace gqa
