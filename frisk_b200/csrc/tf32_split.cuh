// fp32 GEMMs on the tensor cores: the 3xTF32 split.
//
// tcgen05.mma kind::tf32 multiplies numbers with 10 explicit mantissa bits.  An fp32 value x is
// written as hi + lo with hi = x with its low 13 mantissa bits cleared and lo = (x - hi) with ITS
// low 13 bits cleared: both are exactly representable in tf32, x - hi is exact in fp32, and
// |x - hi - lo| <= 2^-21 |x|.  Then
//     A B  =  A_lo B_hi + A_hi B_lo + A_hi B_hi   (+ A_lo B_lo, dropped: <= 2^-20 |a||b| per product)
// with every product exact in the tensor core's fp32 accumulator.  The three products run as one
// GEMM whose K loop walks three segments (small terms first); the split itself is one pass over
// A and B into a workspace of twice their size.  Because hi and lo are exact tf32 numbers the
// result does not depend on whether the hardware truncates or rounds fp32 operands to tf32.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace frisk {

__device__ __forceinline__ float tf32_trunc(float x) {
  return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
}

// hi[i] = trunc(src[i]), lo[i] = trunc(src[i] - hi[i]) for i in [0, n); n4 = n / 4 float4 pieces
// plus a scalar tail.  src, hi and lo are 16-byte aligned (the plan requires it).
__global__ void __launch_bounds__(256) tf32_split_kernel(const float* __restrict__ src,
                                                         float* __restrict__ hi,
                                                         float* __restrict__ lo, int64_t n) {
  const int64_t n4 = n >> 2;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 x = __ldcs(reinterpret_cast<const float4*>(src) + i);
    float4 h, l;
    h.x = tf32_trunc(x.x); h.y = tf32_trunc(x.y); h.z = tf32_trunc(x.z); h.w = tf32_trunc(x.w);
    l.x = tf32_trunc(x.x - h.x); l.y = tf32_trunc(x.y - h.y);
    l.z = tf32_trunc(x.z - h.z); l.w = tf32_trunc(x.w - h.w);
    reinterpret_cast<float4*>(hi)[i] = h;
    reinterpret_cast<float4*>(lo)[i] = l;
  }
  for (int64_t i = (n4 << 2) + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float x = src[i];
    const float h = tf32_trunc(x);
    hi[i] = h;
    lo[i] = tf32_trunc(x - h);
  }
}

}  // namespace frisk
