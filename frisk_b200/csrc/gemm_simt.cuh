// CUDA-core GEMM: fp32 FMA on exactly decoded inputs.  Serves the fp32 configuration (single-pass
// TF32 tensor-core math cannot hold a 1e-4 relative Frobenius error at K = 512) and every shape or
// layout the TMA path cannot take (leading dimensions that are not 16-byte multiples, ...).
// 64 x 64 (or 32 x 64) output tile per CTA, 4 x 4 outputs per thread, 16-deep K slices staged in
// shared memory as fp32, the next slice fetched into registers during the FMAs.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>

#include "gemm_tcgen05.cuh"  // cast_in / cast_out

namespace frisk {

struct SimtParams {
  const void* A;
  const void* B;
  void* C;
  const float* scale_a;  // [M] or nullptr
  const float* scale_b;  // [N] or nullptr
  int64_t M, N, K;
  int64_t lda, ldb, ldc;
  int32_t transA, transB, clear_accum;
};

struct e4m3_t {
  uint8_t bits;
};
template <>
__device__ __forceinline__ float cast_in<e4m3_t>(e4m3_t v) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(v.bits, __NV_E4M3)));
}

struct e5m2_t {
  uint8_t bits;
};
template <>
__device__ __forceinline__ float cast_in<e5m2_t>(e5m2_t v) {
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(v.bits, __NV_E5M2)));
}

constexpr int kSimtTile = 64;
constexpr int kSimtBK = 16;

// TM = rows of the CTA tile (64, or 32 for problems that would not fill the SMs with 64-row
// tiles); the tile is always 64 columns wide and every thread owns 4 x 4 outputs, so a CTA has
// TM * 4 threads.
template <typename TIn, typename TOut, int TM>
__global__ void __launch_bounds__(TM * 4)
gemm_simt_kernel(const SimtParams p) {
  constexpr int kThreads = TM * 4;
  // rows are 16-byte multiples apart and every thread reads its four values at a 16-byte offset,
  // so the inner loop reads each operand with one 128-bit load
  __shared__ __align__(16) float As[kSimtBK][TM + 4];         // [k][m]
  __shared__ __align__(16) float Bs[kSimtBK][kSimtTile + 4];  // [k][n]
  const TIn* A = reinterpret_cast<const TIn*>(p.A);
  const TIn* B = reinterpret_cast<const TIn*>(p.B);
  TOut* C = reinterpret_cast<TOut*>(p.C);
  const int64_t m0 = (int64_t)blockIdx.y * TM;
  const int64_t n0 = (int64_t)blockIdx.x * kSimtTile;
  const int tx = threadIdx.x & 15;  // column group
  const int ty = threadIdx.x >> 4;  // row group

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  // The K slice after the one being multiplied is fetched into registers while the FMAs run, so
  // the global-memory latency of a slice is paid once, not once per slice.
  constexpr int kAPer = TM * kSimtBK / kThreads;         // 4 elements of the A slice per thread
  constexpr int kBPer = kSimtTile * kSimtBK / kThreads;  // 4 or 8 of the B slice
  float av[kAPer], bv[kBPer];
  // walk the contiguous global dimension with consecutive threads
  auto a_pos = [&](int idx, int& am, int& ak) {
    if (p.transA) { am = idx & (TM - 1); ak = idx / TM; } else { ak = idx & 15; am = idx >> 4; }
  };
  auto b_pos = [&](int idx, int& bn, int& bk) {
    if (p.transB) { bk = idx & 15; bn = idx >> 4; } else { bn = idx & 63; bk = idx >> 6; }
  };
  auto fetch = [&](int64_t k0) {
#pragma unroll
    for (int e = 0; e < kAPer; ++e) {
      int am, ak;
      a_pos(threadIdx.x + e * kThreads, am, ak);
      av[e] = 0.f;
      if (m0 + am < p.M && k0 + ak < p.K) {
        const int64_t off = p.transA ? (k0 + ak) * p.lda + (m0 + am) : (m0 + am) * p.lda + (k0 + ak);
        av[e] = cast_in<TIn>(A[off]);
      }
    }
#pragma unroll
    for (int e = 0; e < kBPer; ++e) {
      int bn, bk;
      b_pos(threadIdx.x + e * kThreads, bn, bk);
      bv[e] = 0.f;
      if (n0 + bn < p.N && k0 + bk < p.K) {
        const int64_t off = p.transB ? (n0 + bn) * p.ldb + (k0 + bk) : (k0 + bk) * p.ldb + (n0 + bn);
        bv[e] = cast_in<TIn>(B[off]);
      }
    }
  };
  fetch(0);
  for (int64_t k0 = 0; k0 < p.K; k0 += kSimtBK) {
#pragma unroll
    for (int e = 0; e < kAPer; ++e) {
      int am, ak;
      a_pos(threadIdx.x + e * kThreads, am, ak);
      As[ak][am] = av[e];
    }
#pragma unroll
    for (int e = 0; e < kBPer; ++e) {
      int bn, bk;
      b_pos(threadIdx.x + e * kThreads, bn, bk);
      Bs[bk][bn] = bv[e];
    }
    __syncthreads();
    if (k0 + kSimtBK < p.K) fetch(k0 + kSimtBK);
#pragma unroll
    for (int kk = 0; kk < kSimtBK; ++kk) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    if (m >= p.M) continue;
    const float sa = p.scale_a ? p.scale_a[m] : 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      float v = acc[i][j] * sa;
      if (p.scale_b) v *= p.scale_b[n];
      TOut* dst = C + m * p.ldc + n;
      if (!p.clear_accum) v += cast_in<TOut>(*dst);
      *dst = cast_out<TOut>(v);
    }
  }
}

}  // namespace frisk
