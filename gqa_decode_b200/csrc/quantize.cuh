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

template <typename T16>
__global__ void __launch_bounds__(kQuantThreads)
quantize_kernel(const T16* __restrict__ x, long long elems_per_group, const float* __restrict__ amax,
                uint8_t* __restrict__ codes, float* __restrict__ scale) {
  const long long g = blockIdx.y;
  const float a = fmaxf(amax[g], 1e-12f);
  if (blockIdx.x == 0 && threadIdx.x == 0) scale[g] = __fdiv_rn(a, 448.f);
  const uint4* p = reinterpret_cast<const uint4*>(x + g * elems_per_group);
  uint2* q = reinterpret_cast<uint2*>(codes + g * elems_per_group);
  const long long n8 = elems_per_group / 8;
  for (long long i = (long long)blockIdx.x * kQuantThreads + threadIdx.x; i < n8;
       i += (long long)gridDim.x * kQuantThreads) {
    const uint4 v = __ldg(p + i);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t out[2] = {0u, 0u};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const T16 lo = *reinterpret_cast<const T16*>(&w[j]);
      const T16 hi = *(reinterpret_cast<const T16*>(&w[j]) + 1);
      // float(x) / amax * 448, clamped to the E4M3 range, rounded to nearest even
      float f0 = __fmul_rn(__fdiv_rn(Mma16<T16>::to_float(lo), a), 448.f);
      float f1 = __fmul_rn(__fdiv_rn(Mma16<T16>::to_float(hi), a), 448.f);
      f0 = fminf(fmaxf(f0, -448.f), 448.f);
      f1 = fminf(fmaxf(f1, -448.f), 448.f);
      const unsigned short pr = __nv_cvt_float2_to_fp8x2(make_float2(f0, f1), __NV_SATFINITE, __NV_E4M3);
      out[j >> 1] |= (uint32_t)pr << (16 * (j & 1));
    }
    q[i] = make_uint2(out[0], out[1]);
  }
}

}  // namespace gqa
