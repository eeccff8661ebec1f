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

// fp32 A [M, K] and B [K, N], both row-major at 16-byte aligned rows, M a multiple of 32, N of 64,
// K of 32 (the fp32 512^3 configuration): the same 32 x 64 tile and the same sum per output, in
// the same order, as gemm_simt_kernel<float, TOut, 32> -- so the same bits -- with the K slices
// brought in by 16-byte cp.async into a ring of three shared-memory stages, two slices ahead of
// the FMAs, and one __syncthreads per slice.  The generic kernel pays the latency of a slice's
// scalar loads in every slice (512^3: 32 slices, 0.8 us each); this one is bound by the FMA issue
// of the 128 SMs it has tiles for (measured: six stages, or four groups of warps sharing each
// slice's k, are no faster).
constexpr int kSimtPipeBK = 32;
constexpr int kSimtPipeStages = 3;

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gsrc) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <typename TOut>
__global__ void __launch_bounds__(128)
gemm_simt_f32_pipelined_kernel(const SimtParams p) {
  constexpr int TM = 32, TN = kSimtTile, BK = kSimtPipeBK, S = kSimtPipeStages;
  // A as stored (k contiguous, rows padded by 4 floats: the four rows a thread reads at one k lie
  // in different banks), B as stored (n contiguous)
  __shared__ __align__(16) float As[S][TM][BK + 4];
  __shared__ __align__(16) float Bs[S][BK][TN + 4];
  const float* A = reinterpret_cast<const float*>(p.A);
  const float* B = reinterpret_cast<const float*>(p.B);
  TOut* C = reinterpret_cast<TOut*>(p.C);
  const int64_t m0 = (int64_t)blockIdx.y * TM;
  const int64_t n0 = (int64_t)blockIdx.x * TN;
  const int t = threadIdx.x;
  const int tx = t & 15;  // column group
  const int ty = t >> 4;  // row group

  auto load_stage = [&](int s, int64_t k0) {
    // A: 32 rows x 8 chunks of 16 bytes; B: 32 k-rows x 16 chunks
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int idx = t + e * 128, r = idx >> 3, c = (idx & 7) * 4;
      cp_async_16(&As[s][r][c], A + (m0 + r) * p.lda + k0 + c);
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int idx = t + e * 128, r = idx >> 4, c = (idx & 15) * 4;
      cp_async_16(&Bs[s][r][c], B + (k0 + r) * p.ldb + n0 + c);
    }
  };

  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int nk = (int)(p.K / BK);
#pragma unroll
  for (int s = 0; s < S - 1; ++s) {
    if (s < nk) load_stage(s, (int64_t)s * BK);
    cp_async_commit();
  }
  for (int it = 0; it < nk; ++it) {
    cp_async_wait<S - 2>();   // slice `it` has landed (this thread's part; the barrier covers the rest)
    __syncthreads();          // ... and everybody is done with the stage refilled below
    const int nx = it + S - 1;
    if (nx < nk) load_stage(nx % S, (int64_t)nx * BK);
    cp_async_commit();
    const int s = it % S;
#pragma unroll
    for (int k4 = 0; k4 < BK; k4 += 4) {
      float a[4][4], b[4][4];   // [row][k], [k][column]
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float4 v = *reinterpret_cast<const float4*>(&As[s][ty * 4 + i][k4]);
        a[i][0] = v.x; a[i][1] = v.y; a[i][2] = v.z; a[i][3] = v.w;
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk) {
        const float4 v = *reinterpret_cast<const float4*>(&Bs[s][k4 + kk][tx * 4]);
        b[kk][0] = v.x; b[kk][1] = v.y; b[kk][2] = v.z; b[kk][3] = v.w;
      }
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i][kk], b[kk][j], acc[i][j]);
    }
  }
  cp_async_wait<0>();

#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t m = m0 + ty * 4 + i;
    const float sa = p.scale_a ? p.scale_a[m] : 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int64_t n = n0 + tx * 4 + j;
      float v = acc[i][j] * sa;
      if (p.scale_b) v *= p.scale_b[n];
      TOut* dst = C + m * p.ldc + n;
      if (!p.clear_accum) v += cast_in<TOut>(*dst);
      *dst = cast_out<TOut>(v);
    }
  }
}

}  // namespace frisk
