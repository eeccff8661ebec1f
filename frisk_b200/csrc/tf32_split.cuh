// fp32 GEMMs on the tensor cores: the 3xTF32 split.
//
// tcgen05.mma kind::tf32 multiplies numbers with 10 explicit mantissa bits.  An fp32 value x is
// written as hi + lo with hi = x with its low 13 mantissa bits cleared and lo = (x - hi) with ITS
// low 13 bits cleared: both are exactly representable in tf32, x - hi is exact in fp32, and
// |x - hi - lo| <= 2^-21 |x|.  Then
//     A B  =  A_lo B_hi + A_hi B_lo + A_hi B_hi   (+ A_lo B_lo, dropped: <= 2^-20 |a||b| per product)
// with every product exact in the tensor core's fp32 accumulator.  The three products run as ONE
// GEMM over a K three times as long.  A pass over A and B writes, K innermost whatever the order
// A and B are stored in and every segment padded with zeros to a whole k-block of 32,
//     A' = [A_lo | A_hi]  (along K)      B' = [B_hi | B_lo]  (along K)
// into a workspace, and the kernels' producers read the k-blocks of the first third of that K from
// (A_lo, B_hi), of the second from (A_hi, B_lo), of the last from (A_hi, B_hi): small terms first.
// Because hi and lo are exact tf32 numbers the result does not depend on whether the hardware
// truncates or rounds fp32 operands to tf32.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace frisk {

__device__ __forceinline__ float tf32_trunc(float x) {
  return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
}

// src: rows x cols fp32 (cols = K), pitch ld_src.  dst: the two K segments of the operand side by
// side in every row, each `seg_cols` wide (K rounded up to a k-block, the tail zero): segment s
// holds the lo parts when bit s of `lo_mask` is set, else the hi parts.  Pitch ld_dst, a multiple
// of four like seg_cols.  One thread handles four consecutive columns (a 16-byte load when the
// source row allows it, 16-byte stores always).
__global__ void __launch_bounds__(256) tf32_split_kernel(const float* __restrict__ src,
                                                         float* __restrict__ dst, int64_t rows,
                                                         int64_t cols, int64_t seg_cols,
                                                         int64_t ld_src, int64_t ld_dst,
                                                         uint32_t lo_mask) {
  const int64_t quads = seg_cols >> 2;
  const int64_t total = rows * quads;
  const bool vec = (ld_src & 3) == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / quads, c = (i - r * quads) << 2;
    const float* s = src + r * ld_src + c;
    float* d = dst + r * ld_dst + c;
    float x[4], h[4], l[4];
    const int64_t left = cols - c;
    const int n = (int)(left < 0 ? 0 : left < 4 ? left : 4);
    if (vec && n == 4) {
      const float4 t = __ldcs(reinterpret_cast<const float4*>(s));
      x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w;
    } else {
      for (int j = 0; j < 4; ++j) x[j] = j < n ? s[j] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      h[j] = tf32_trunc(x[j]);
      l[j] = tf32_trunc(x[j] - h[j]);
    }
#pragma unroll
    for (int seg = 0; seg < 2; ++seg) {
      const float* v = (lo_mask >> seg) & 1u ? l : h;
      *reinterpret_cast<float4*>(d + seg * seg_cols) = make_float4(v[0], v[1], v[2], v[3]);
    }
  }
}

// The same split for an operand stored with K along its ROWS (A stored [K, M], B stored [K, N]):
// kind::tf32 takes its operands K-inner only (an M/N-inner tile of 32-bit elements reads as
// zeros), so the two segments are written transposed, dst[mn, s * seg_cols + k] with
// seg_cols = K rounded up to 32 and zeros behind K, through a 32 x 32 tile in shared memory (reads
// coalesced along M/N, writes along K).  grid = (ceil(mn / 32), ceil(K / 32)), block = (32, 8).
__global__ void __launch_bounds__(256) tf32_split_transpose_kernel(const float* __restrict__ src,
                                                                   float* __restrict__ dst,
                                                                   int64_t k_rows, int64_t mn_cols,
                                                                   int64_t seg_cols, int64_t ld_src,
                                                                   int64_t ld_dst, uint32_t lo_mask) {
  __shared__ float tile[32][33];
  const int64_t mn0 = (int64_t)blockIdx.x * 32, k0 = (int64_t)blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += 8) {
    const int64_t k = k0 + r, mn = mn0 + threadIdx.x;
    tile[r][threadIdx.x] = (k < k_rows && mn < mn_cols) ? __ldcs(src + k * ld_src + mn) : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += 8) {
    const int64_t mn = mn0 + r, k = k0 + threadIdx.x;
    if (mn < mn_cols) {   // k < seg_cols always; the tile holds zeros behind K
      const float x = tile[threadIdx.x][r];
      const float h = tf32_trunc(x), l = tf32_trunc(x - h);
      float* o = dst + mn * ld_dst + k;
#pragma unroll
      for (int seg = 0; seg < 2; ++seg) o[seg * seg_cols] = (lo_mask >> seg) & 1u ? l : h;
    }
  }
}

}  // namespace frisk
