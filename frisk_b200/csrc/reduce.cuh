// frisk.reduce on buffers in global memory: two kernels, both bound by HBM bandwidth (every source
// element is read once, 16 bytes per load where alignment allows, streaming past L1).
//
//   reduce_lines_kernel    the reduced dimension is the innermost one: a group of lanes (a warp
//                          for long lines) per (line, piece of the line), four independent
//                          accumulators and four or eight loads in flight per lane, a shuffle tree.
//   reduce_columns_kernel  the reduced dimension has contiguous elements after it: a CTA is a
//                          TY x TX sheet of threads, TX along the contiguous dimension (coalesced),
//                          TY over the reduced one, folded through shared memory at the end.
//
// When the problem has too few lines or columns to fill the SMs the reduced dimension is cut into
// pieces, the first launch writes fp32 partial results to a workspace and a second launch of the
// same kernels folds the pieces.  The order of operations is fixed by the shape alone.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace frisk_reduce {

constexpr int kThreads = 256;
constexpr int kWarpsPerCta = kThreads / 32;

struct Params {
  int64_t outer, extent, inner;
  int64_t chunk_len;  // elements of the reduced dimension per piece
  int32_t chunks;
  int32_t clear;      // final launches only: 0 folds the old destination value in
  int32_t lanes_log2; // lines kernel: lanes per (line, piece)
  int32_t tx_log2;    // columns kernel: TX = 1 << tx_log2 threads along the contiguous dimension
  int64_t xblocks;    // columns kernel: CTAs along the contiguous dimension
};

// The second launch of a two-launch reduce is a programmatic dependent launch: its CTAs may be
// scheduled while the first kernel drains, and wait here until that kernel's writes are visible.
// In a kernel launched the ordinary way both instructions do nothing.
__device__ __forceinline__ void dependent_launch_prologue() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <int KIND> struct Op;
template <> struct Op<0> {
  static __device__ __forceinline__ float identity() { return 0.f; }
  static __device__ __forceinline__ float apply(float a, float b) { return a + b; }
};
template <> struct Op<1> {
  static __device__ __forceinline__ float identity() { return 1.f; }
  static __device__ __forceinline__ float apply(float a, float b) { return a * b; }
};
template <> struct Op<2> {
  static __device__ __forceinline__ float identity() { return __int_as_float(0x7f800000); }
  static __device__ __forceinline__ float apply(float a, float b) { return fminf(a, b); }
};
template <> struct Op<3> {
  static __device__ __forceinline__ float identity() { return __int_as_float(0xff800000); }
  static __device__ __forceinline__ float apply(float a, float b) { return fmaxf(a, b); }
};

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// The 16 / sizeof(T) elements of one 16-byte load as fp32.
template <typename T> struct Vec;
template <> struct Vec<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  }
};
template <> struct Vec<__half> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = p.x;
      f[2 * i + 1] = p.y;
    }
  }
};
template <> struct Vec<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
};

// How a line is folded.  In general: fp32 accumulators, every element converted.
template <typename T, int KIND> struct Fold {
  using Acc = float;
  static __device__ __forceinline__ Acc init() { return Op<KIND>::identity(); }
  static __device__ __forceinline__ Acc vec(const uint4& v, Acc acc) {
    float f[Vec<T>::N];
    Vec<T>::unpack(v, f);
#pragma unroll
    for (int i = 0; i < Vec<T>::N; ++i) acc = Op<KIND>::apply(acc, f[i]);
    return acc;
  }
  static __device__ __forceinline__ Acc one(T x, Acc acc) { return Op<KIND>::apply(acc, to_f32(x)); }
  static __device__ __forceinline__ Acc join(Acc a, Acc b) { return Op<KIND>::apply(a, b); }
  static __device__ __forceinline__ float finish(Acc a) { return a; }
};
// min and max of 16-bit floats are exact in their own format: two elements per instruction,
// no conversion (the packed min / max return the other operand when one is NaN, like fminf).
template <typename T2, bool IS_MAX> struct PackedMinMax {
  using Acc = T2;
  static __device__ __forceinline__ Acc op(Acc a, Acc b) { return IS_MAX ? __hmax2(a, b) : __hmin2(a, b); }
  static __device__ __forceinline__ Acc vec(const uint4& v, Acc acc) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    Acc t0 = op(*reinterpret_cast<const Acc*>(&w[0]), *reinterpret_cast<const Acc*>(&w[1]));
    Acc t1 = op(*reinterpret_cast<const Acc*>(&w[2]), *reinterpret_cast<const Acc*>(&w[3]));
    return op(acc, op(t0, t1));
  }
  static __device__ __forceinline__ Acc join(Acc a, Acc b) { return op(a, b); }
};
template <bool IS_MAX> struct FoldHalf : PackedMinMax<__half2, IS_MAX> {
  using Acc = __half2;
  static __device__ __forceinline__ Acc init() {
    const unsigned short bits = IS_MAX ? 0xfc00 : 0x7c00;  // -inf / +inf
    return __half2half2(__ushort_as_half(bits));
  }
  static __device__ __forceinline__ Acc one(__half x, Acc acc) {
    return PackedMinMax<__half2, IS_MAX>::op(acc, __half2half2(x));
  }
  static __device__ __forceinline__ float finish(Acc a) {
    const float2 f = __half22float2(a);
    return IS_MAX ? fmaxf(f.x, f.y) : fminf(f.x, f.y);
  }
};
template <bool IS_MAX> struct FoldBf16 : PackedMinMax<__nv_bfloat162, IS_MAX> {
  using Acc = __nv_bfloat162;
  static __device__ __forceinline__ Acc init() {
    const unsigned short bits = IS_MAX ? 0xff80 : 0x7f80;
    return __bfloat162bfloat162(__ushort_as_bfloat16(bits));
  }
  static __device__ __forceinline__ Acc one(__nv_bfloat16 x, Acc acc) {
    return PackedMinMax<__nv_bfloat162, IS_MAX>::op(acc, __bfloat162bfloat162(x));
  }
  static __device__ __forceinline__ float finish(Acc a) {
    const float2 f = __bfloat1622float2(a);
    return IS_MAX ? fmaxf(f.x, f.y) : fminf(f.x, f.y);
  }
};
template <> struct Fold<__half, 2> : FoldHalf<false> {};
template <> struct Fold<__half, 3> : FoldHalf<true> {};
template <> struct Fold<__nv_bfloat16, 2> : FoldBf16<false> {};
template <> struct Fold<__nv_bfloat16, 3> : FoldBf16<true> {};

// dst[line] (FINAL) or partial[line * chunks + chunk] = fold of src[line, begin .. end).
// A group of L = 1 << lanes_log2 lanes per (line, piece): fewer than a warp for short lines, so
// that a warp covers several consecutive lines; a warp for long ones; several warps, up to the
// CTA, when the lines are few (the second launch of a two-launch reduce).
// DEPTH: 16-byte loads in flight per lane, 4 or 8.  Eight pay when folding is cheap next to the
// load (fp32 elements, packed min / max); with a conversion per element (sums of 16-bit floats)
// the extra registers cost more residency than the deeper queue returns.
template <typename TIn, typename TOut, int KIND, bool FINAL, int DEPTH>
__global__ void __launch_bounds__(kThreads) reduce_lines_kernel(const TIn* __restrict__ src,
                                                                TOut* __restrict__ dst, Params p) {
  using O = Op<KIND>;
  using F = Fold<TIn, KIND>;
  constexpr int N = Vec<TIn>::N;
  dependent_launch_prologue();
  const int L = 1 << p.lanes_log2;
  const int64_t unit = ((int64_t)blockIdx.x * kThreads + threadIdx.x) >> p.lanes_log2;
  const int sub = threadIdx.x & (L - 1);
  const bool live = unit < p.outer * p.chunks;
  const int64_t line = live ? unit / p.chunks : 0;
  float r = O::identity();
  if (live) {
    const int64_t begin = (unit - line * p.chunks) * p.chunk_len;
    const int64_t end = begin + p.chunk_len < p.extent ? begin + p.chunk_len : p.extent;
    const TIn* s = src + line * p.extent;
    typename F::Acc acc0 = F::init(), acc1 = F::init(), acc2 = F::init(), acc3 = F::init();
    // a piece has fewer than 2^31 elements (the host cuts longer lines): 32-bit counters from here
    const TIn* piece = s + begin;
    const int len = (int)(end - begin);
    int head = (int)(((16 - (reinterpret_cast<uintptr_t>(piece) & 15)) & 15) / sizeof(TIn));
    if (head > len) head = len;  // up to the first 16-byte boundary: fewer than N elements
    for (int h = sub; h < head; h += L) acc1 = F::one(piece[h], acc1);
    const int nvec = (len - head) / N;
    const uint4* v = reinterpret_cast<const uint4*>(piece + head) + sub;
    int k = sub;
    if (DEPTH == 8)
    for (; k + 7 * L < nvec; k += 8 * L, v += 8 * L) {
      const uint4 a = __ldcs(v), b = __ldcs(v + L), c = __ldcs(v + 2 * L), d = __ldcs(v + 3 * L);
      const uint4 e = __ldcs(v + 4 * L), f = __ldcs(v + 5 * L), g = __ldcs(v + 6 * L), h = __ldcs(v + 7 * L);
      acc0 = F::vec(e, F::vec(a, acc0));
      acc1 = F::vec(f, F::vec(b, acc1));
      acc2 = F::vec(g, F::vec(c, acc2));
      acc3 = F::vec(h, F::vec(d, acc3));
    }
    for (; k + 3 * L < nvec; k += 4 * L, v += 4 * L) {  // four loads in flight per lane
      const uint4 a = __ldcs(v), b = __ldcs(v + L), c = __ldcs(v + 2 * L), d = __ldcs(v + 3 * L);
      acc0 = F::vec(a, acc0);
      acc1 = F::vec(b, acc1);
      acc2 = F::vec(c, acc2);
      acc3 = F::vec(d, acc3);
    }
    for (; k < nvec; k += L, v += L) acc0 = F::vec(__ldcs(v), acc0);
    for (int t = head + nvec * N + sub; t < len; t += L) acc2 = F::one(piece[t], acc2);  // fewer than N left
    r = F::finish(F::join(F::join(acc0, acc1), F::join(acc2, acc3)));
  }
  for (int off = (L < 32 ? L : 32) >> 1; off > 0; off >>= 1) r = O::apply(r, __shfl_xor_sync(0xffffffffu, r, off));
  if (L > 32) {  // a group of several warps: their results meet in shared memory
    __shared__ float across[kWarpsPerCta];
    if ((threadIdx.x & 31) == 0) across[threadIdx.x >> 5] = r;
    __syncthreads();
    if (sub == 0)
      for (int w = 1; w < (L >> 5); ++w) r = O::apply(r, across[(threadIdx.x >> 5) + w]);
  }
  if (live && sub == 0) {
    if (FINAL) {
      if (!p.clear) r = O::apply(to_f32(dst[line]), r);
      dst[line] = from_f32<TOut>(r);
    } else {
      dst[unit] = from_f32<TOut>(r);
    }
  }
}

// dst[o, c] (FINAL) or partial[(o * chunks + chunk) * inner + c] = fold over e of src[o, e, c].
// VEC consecutive columns per thread (one 16-byte load when VEC > 1, which needs inner % VEC == 0
// and an aligned base).  grid.x = outer * chunks * xblocks.
template <typename TIn, typename TOut, int KIND, bool FINAL, int VEC>
__global__ void __launch_bounds__(kThreads) reduce_columns_kernel(const TIn* __restrict__ src,
                                                                  TOut* __restrict__ dst, Params p) {
  using O = Op<KIND>;
  __shared__ float fold[kThreads * VEC];
  dependent_launch_prologue();
  const int tx = threadIdx.x & ((1 << p.tx_log2) - 1), ty = threadIdx.x >> p.tx_log2;
  const int ny = kThreads >> p.tx_log2;
  int64_t b = blockIdx.x;
  const int64_t xb = b % p.xblocks;
  b /= p.xblocks;
  const int64_t chunk = b % p.chunks, o = b / p.chunks;
  const int64_t col = ((xb << p.tx_log2) + tx) * VEC;
  const bool live = col < p.inner;
  const int64_t begin = chunk * p.chunk_len;
  const int64_t end = begin + p.chunk_len < p.extent ? begin + p.chunk_len : p.extent;

  float acc[VEC], acc2[VEC];
#pragma unroll
  for (int v = 0; v < VEC; ++v) acc[v] = acc2[v] = O::identity();
  if (live) {
    const TIn* s = src + o * p.extent * p.inner + col;
    int64_t e = begin + ty;
    const int64_t step = (int64_t)ny * p.inner;
    const TIn* q = s + e * p.inner;
    if (VEC > 1) {
      for (; e + 3 * ny < end; e += 4 * ny, q += 4 * step) {  // four rows in flight per thread
        const uint4 a = __ldcs(reinterpret_cast<const uint4*>(q));
        const uint4 b = __ldcs(reinterpret_cast<const uint4*>(q + step));
        const uint4 c = __ldcs(reinterpret_cast<const uint4*>(q + 2 * step));
        const uint4 d = __ldcs(reinterpret_cast<const uint4*>(q + 3 * step));
        float fa[Vec<TIn>::N], fb[Vec<TIn>::N];
        Vec<TIn>::unpack(a, fa);
        Vec<TIn>::unpack(b, fb);
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          acc[v] = O::apply(acc[v], fa[v]);
          acc2[v] = O::apply(acc2[v], fb[v]);
        }
        Vec<TIn>::unpack(c, fa);
        Vec<TIn>::unpack(d, fb);
#pragma unroll
        for (int v = 0; v < VEC; ++v) {
          acc[v] = O::apply(acc[v], fa[v]);
          acc2[v] = O::apply(acc2[v], fb[v]);
        }
      }
      for (; e < end; e += ny, q += step) {
        float fa[Vec<TIn>::N];
        Vec<TIn>::unpack(__ldcs(reinterpret_cast<const uint4*>(q)), fa);
#pragma unroll
        for (int v = 0; v < VEC; ++v) acc[v] = O::apply(acc[v], fa[v]);
      }
    } else {
      for (; e + 3 * ny < end; e += 4 * ny, q += 4 * step) {
        const float a = to_f32(q[0]), b = to_f32(q[step]), c = to_f32(q[2 * step]), d = to_f32(q[3 * step]);
        acc[0] = O::apply(O::apply(acc[0], a), c);
        acc2[0] = O::apply(O::apply(acc2[0], b), d);
      }
      for (; e < end; e += ny, q += step) acc[0] = O::apply(acc[0], to_f32(q[0]));
    }
  }
#pragma unroll
  for (int v = 0; v < VEC; ++v) fold[threadIdx.x * VEC + v] = O::apply(acc[v], acc2[v]);
  __syncthreads();
  for (int half = ny >> 1; half > 0; half >>= 1) {
    if (ty < half) {
#pragma unroll
      for (int v = 0; v < VEC; ++v)
        fold[threadIdx.x * VEC + v] =
            O::apply(fold[threadIdx.x * VEC + v], fold[(threadIdx.x + (half << p.tx_log2)) * VEC + v]);
    }
    __syncthreads();
  }
  if (ty == 0 && live) {
#pragma unroll
    for (int v = 0; v < VEC; ++v) {
      float r = fold[tx * VEC + v];
      if (FINAL) {
        TOut* d = dst + o * p.inner + col + v;
        if (!p.clear) r = O::apply(to_f32(*d), r);
        *d = from_f32<TOut>(r);
      } else {
        dst[(o * p.chunks + chunk) * p.inner + col + v] = from_f32<TOut>(r);
      }
    }
  }
}

}  // namespace frisk_reduce
