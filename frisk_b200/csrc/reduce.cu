// Host side of frisk.reduce on whole buffers: how a shape is cut into launches, and the C ABI
// entry points declared in include/frisk_b200.h.
#include "reduce.cuh"

#include <algorithm>
#include <cstdio>
#include <string>

#include "../../include/frisk_b200.h"
#include "abi_internal.h"

namespace {

using frisk_reduce::kThreads;
using frisk_reduce::kWarpsPerCta;
using frisk_reduce::Params;

int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

int elem_bytes(int dt) { return dt == FRISK_DT_F32 ? 4 : (dt == FRISK_DT_F16 || dt == FRISK_DT_BF16) ? 2 : 0; }

struct Plan {
  bool lines = false;
  int vec = 1;          // first launch
  int vec2 = 1;         // second launch (fp32 partials)
  int tx_log2 = 0, tx_log2_2 = 0;
  int lanes_log2 = 5, lanes_log2_2 = 5;  // lines kernel
  bool deep = false;                     // lines kernel, first launch: eight loads in flight per lane
  int64_t xblocks = 1, xblocks2 = 1;
  int64_t chunk_len = 0;
  int64_t chunks = 1;
  int64_t ctas = 0, ctas2 = 0;
  size_t ws_bytes = 0;
};

int log2_ceil(int64_t v) {
  int l = 0;
  while ((int64_t(1) << l) < v) ++l;
  return l;
}

// The CTA as a TY x TX sheet: TX threads along the contiguous dimension, the other TY = 256 / TX
// over the reduced dimension.  The first launch reads from HBM and keeps TX at 64 when the rows
// are that wide (1 KiB contiguous per row and CTA) so that four row groups share a CTA; the second
// launch reads partial results that are still in L2 and prefers many small CTAs (TX <= 32).
// A short reduced dimension gets fewer TY rows and the threads go to the contiguous side.
void columns_shape(int64_t inner, int64_t extent, int vec, bool first, bool plenty, int* tx_log2,
                   int64_t* xblocks) {
  const int64_t ivecs = inner / vec;
  // `plenty`: even CTAs that span 256 vectors of a row fill the device; then a CTA reads 4 KiB
  // contiguous per row and keeps its four loads per thread in flight over four rows.
  const int ty_log2 = plenty ? 0 : std::min(first ? 2 : 3, log2_ceil(std::max<int64_t>(extent, 1)));
  *tx_log2 = std::min(log2_ceil(ivecs), log2_ceil(kThreads) - ty_log2);
  *xblocks = ceil_div(ivecs, int64_t(1) << *tx_log2);
}

// Lanes per line piece: about four 16-byte loads per lane, at most `cap` (log2; 8 = the CTA).
int lanes_for(int64_t piece, int vec, int cap) {
  return std::min(cap, log2_ceil(std::max<int64_t>(1, ceil_div(ceil_div(piece, vec), 4))));
}

// `slots`: CTAs the device holds at once for the first-launch kernel (SMs x CTAs per SM).
int make_plan(const frisk_reduce_desc& d, bool src_align16, int64_t slots, Plan* out) {
  const int es = elem_bytes(d.dtype);
  if (d.outer < 0 || d.extent < 0 || d.inner < 0 || d.kind < 0 || d.kind > 3) {
    frisk_internal_set_error("reduce: negative size or unknown kind");
    return FRISK_ERR_INVALID_ARGUMENT;
  }
  if (!es) {
    frisk_internal_set_error("reduce: element type must be f32, f16 or bf16");
    return FRISK_ERR_UNSUPPORTED;
  }
  Plan p;
  p.lines = d.inner == 1;
  p.chunk_len = std::max<int64_t>(d.extent, 1);
  if (d.outer == 0 || d.inner == 0) {  // nothing to write
    *out = p;
    return FRISK_OK;
  }
  if (p.lines) {
    // Up to a warp per line.  With fewer lines than about half the warps the device holds, cut the
    // lines so that every SM has work; pieces stay at least 4096 elements long.
    const int64_t want = slots * kWarpsPerCta;
    p.vec = 16 / es;
    if (d.outer * 2 < want && d.extent >= 2 * 4096) {
      int64_t chunks = std::min(ceil_div(want, d.outer), d.extent / 4096);
      p.chunk_len = ceil_div(ceil_div(d.extent, chunks), 1024) * 1024;
      p.chunks = ceil_div(d.extent, p.chunk_len);
    }
    if (p.chunk_len > (int64_t(1) << 30)) {  // the kernel counts inside a piece in 32 bits
      p.chunk_len = int64_t(1) << 30;
      p.chunks = ceil_div(d.extent, p.chunk_len);
    }
    // First launch: at most a warp per piece (measured on 8192 x 8192: groups of 2, 4 and 8 warps
    // per line were 2 - 25 % slower; the work per CTA gets too short).  Second launch: one line of
    // partial results per CTA if need be, it is the only work there is.
    p.lanes_log2 = lanes_for(std::min(p.chunk_len, std::max<int64_t>(d.extent, 1)), p.vec, 5);
    p.lanes_log2_2 = lanes_for(p.chunks, 4, 8);
    // Eight loads in flight where a lane has them to issue and folding is cheap (measured on
    // 8192 x 8192, same box: fp32 sums 51 -> 44 us, fp16 maxima 27.5 -> 24.5 us, but bf16 / fp16
    // sums 27.8 -> 29 us and 1 KiB lines 27 -> 30.5 us).
    p.deep = p.lanes_log2 == 5 && (es == 4 || d.kind >= FRISK_REDUCE_MIN) &&
             std::min(p.chunk_len, d.extent) / p.vec >= 8 * 32;
    p.ctas = ceil_div((d.outer * p.chunks) << p.lanes_log2, kThreads);
    p.ctas2 = p.chunks > 1 ? ceil_div(d.outer << p.lanes_log2_2, kThreads) : 0;
  } else {
    p.vec = (src_align16 && (d.inner * es) % 16 == 0) ? 16 / es : 1;
    const bool plenty = d.outer * ceil_div(d.inner / p.vec, kThreads) * 2 >= slots;
    columns_shape(d.inner, d.extent, p.vec, true, plenty, &p.tx_log2, &p.xblocks);
    const int64_t ny = kThreads >> p.tx_log2;
    const int64_t base = d.outer * p.xblocks, want = slots;
    if (base * 2 < want && d.extent >= 2 * 8 * ny) {
      int64_t chunks = std::min(std::max<int64_t>(1, want / base), d.extent / (8 * ny));  // one wave of CTAs
      p.chunk_len = ceil_div(ceil_div(d.extent, chunks), ny) * ny;
      p.chunks = ceil_div(d.extent, p.chunk_len);
    }
    p.ctas = base * p.chunks;
    if (p.chunks > 1) {
      p.vec2 = d.inner % 4 == 0 ? 4 : 1;  // the workspace is 256-byte aligned
      columns_shape(d.inner, p.chunks, p.vec2, false, false, &p.tx_log2_2, &p.xblocks2);
      p.ctas2 = d.outer * p.xblocks2;
    }
  }
  if (p.chunks > 1) p.ws_bytes = (size_t)(d.outer * p.chunks * d.inner) * sizeof(float);
  if (p.ctas > 0x7fffffffll || p.ctas2 > 0x7fffffffll || p.chunks > 0x7fffffffll) {
    frisk_internal_set_error("reduce: the shape needs more than 2^31 - 1 CTAs");
    return FRISK_ERR_TOO_LARGE;
  }
  *out = p;
  return FRISK_OK;
}

template <typename TIn, typename TOut, int KIND, bool FINAL>
const void* kernel_of(bool lines, int vec, bool deep = false) {
  using namespace frisk_reduce;
  if (lines && deep) return reinterpret_cast<const void*>(&reduce_lines_kernel<TIn, TOut, KIND, FINAL, 8>);
  if (lines) return reinterpret_cast<const void*>(&reduce_lines_kernel<TIn, TOut, KIND, FINAL, 4>);
  if (vec > 1) return reinterpret_cast<const void*>(&reduce_columns_kernel<TIn, TOut, KIND, FINAL, Vec<TIn>::N>);
  return reinterpret_cast<const void*>(&reduce_columns_kernel<TIn, TOut, KIND, FINAL, 1>);
}

// `dependent`: a programmatic dependent launch (it follows the first launch of the same reduce).
cudaError_t launch(const void* kernel, const void* src, void* dst, const Params& p, int64_t ctas, bool dependent,
                   cudaStream_t st) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)ctas);
  cfg.blockDim = dim3(kThreads);
  cfg.stream = st;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = dependent ? 1 : 0;
  Params pp = p;
  void* args[] = {&src, &dst, &pp};
  return cudaLaunchKernelExC(&cfg, kernel, args);
}

template <typename T, int KIND>
cudaError_t run_typed(const frisk_reduce_desc& d, const Plan& pl, const void* src, void* dst, void* ws,
                      cudaStream_t st) {
  Params p{};
  p.outer = d.outer;
  p.extent = d.extent;
  p.inner = d.inner;
  p.chunk_len = pl.chunk_len;
  p.chunks = (int32_t)pl.chunks;
  p.clear = d.clear;
  p.lanes_log2 = pl.lanes_log2;
  p.tx_log2 = pl.tx_log2;
  p.xblocks = pl.xblocks;
  if (pl.chunks == 1)
    return launch(kernel_of<T, T, KIND, true>(pl.lines, pl.vec, pl.deep), src, dst, p, pl.ctas, false, st);
  cudaError_t e = launch(kernel_of<T, float, KIND, false>(pl.lines, pl.vec, pl.deep), src, ws, p, pl.ctas, false, st);
  if (e != cudaSuccess) return e;
  Params q = p;  // the pieces are the reduced dimension of the second launch
  q.extent = pl.chunks;
  q.chunk_len = pl.chunks;
  q.chunks = 1;
  q.lanes_log2 = pl.lanes_log2_2;
  q.tx_log2 = pl.tx_log2_2;
  q.xblocks = pl.xblocks2;
  return launch(kernel_of<float, T, KIND, true>(pl.lines, pl.vec2), ws, dst, q, pl.ctas2, true, st);
}

// The first-launch kernel of a shape that goes through the workspace, for the occupancy query.
template <typename T>
const void* partial_kernel(int kind, bool lines, int vec) {
  switch (kind) {
    case FRISK_REDUCE_ADD: return kernel_of<T, float, 0, false>(lines, vec);
    case FRISK_REDUCE_MUL: return kernel_of<T, float, 1, false>(lines, vec);
    case FRISK_REDUCE_MIN: return kernel_of<T, float, 2, false>(lines, vec);
    default: return kernel_of<T, float, 3, false>(lines, vec);
  }
}

template <typename T>
cudaError_t run_kind(const frisk_reduce_desc& d, const Plan& pl, const void* src, void* dst, void* ws,
                     cudaStream_t st) {
  switch (d.kind) {
    case FRISK_REDUCE_ADD: return run_typed<T, 0>(d, pl, src, dst, ws, st);
    case FRISK_REDUCE_MUL: return run_typed<T, 1>(d, pl, src, dst, ws, st);
    case FRISK_REDUCE_MIN: return run_typed<T, 2>(d, pl, src, dst, ws, st);
    default: return run_typed<T, 3>(d, pl, src, dst, ws, st);
  }
}

int fail_cuda(cudaError_t e, const char* what) {
  frisk_internal_set_error((std::string(what) + ": " + cudaGetErrorString(e)).c_str());
  return FRISK_ERR_CUDA;
}

int sm_count_of(int device, int* sms) {
  int dev = device;
  if (dev < 0) {
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  }
  cudaError_t e = cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceGetAttribute");
  return FRISK_OK;
}

// CTAs of the first-launch kernel that fit the device at once.  The column cut depends on the
// vector width, which depends on the alignment; the two variants use about the same registers, so
// the query is made for the one the alignment selects.
int slots_for(const frisk_reduce_desc& d, bool aligned, int64_t* slots) {
  int sms = 0;
  if (int rc = sm_count_of(d.device, &sms)) return rc;
  const int es = elem_bytes(d.dtype);
  const bool lines = d.inner == 1;
  const int vec = es && (lines || (aligned && (d.inner * es) % 16 == 0)) ? 16 / es : 1;
  const void* k = d.dtype == FRISK_DT_F32   ? partial_kernel<float>(d.kind, lines, vec)
                  : d.dtype == FRISK_DT_F16 ? partial_kernel<__half>(d.kind, lines, vec)
                                            : partial_kernel<__nv_bfloat16>(d.kind, lines, vec);
  int per_sm = 0;
  cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k, kThreads, 0);
  if (e != cudaSuccess) return fail_cuda(e, "cudaOccupancyMaxActiveBlocksPerMultiprocessor");
  *slots = (int64_t)sms * std::max(per_sm, 1);
  return FRISK_OK;
}

}  // namespace

extern "C" {

int frisk_b200_reduce_info(const frisk_reduce_desc* desc, int src_align16, frisk_reduce_info* out) {
  if (!desc || !out) return FRISK_ERR_INVALID_ARGUMENT;
  // The cut depends on how many CTAs the device holds; without a device a B200's 148 SMs with six
  // CTAs each are assumed so that the arithmetic can be inspected anywhere.
  int64_t slots = 148 * 6;
  int count = 0;
  if (cudaGetDeviceCount(&count) == cudaSuccess && count > 0) {
    if (elem_bytes(desc->dtype) && desc->kind >= 0 && desc->kind <= 3)
      if (int rc = slots_for(*desc, src_align16 != 0, &slots)) return rc;
  } else {
    (void)cudaGetLastError();
  }
  Plan p;
  if (int rc = make_plan(*desc, src_align16 != 0, slots, &p)) return rc;
  out->lines = p.lines;
  out->vector = p.vec;
  out->chunks = (int32_t)p.chunks;
  out->launches = (desc->outer == 0 || desc->inner == 0) ? 0 : p.chunks > 1 ? 2 : 1;
  out->chunk_len = p.chunk_len;
  out->ctas = p.ctas;
  out->workspace_bytes = p.ws_bytes;
  return FRISK_OK;
}

int frisk_b200_reduce_workspace_bytes(const frisk_reduce_desc* desc, size_t* out) {
  if (!desc || !out) return FRISK_ERR_INVALID_ARGUMENT;
  frisk_reduce_info info;
  // For columns the cut depends on whether the source allows 16-byte loads, which is known only
  // when the pointer is: report the larger of the two needs.
  size_t need = 0;
  for (int aligned = 0; aligned < 2; ++aligned) {
    if (int rc = frisk_b200_reduce_info(desc, aligned, &info)) return rc;
    need = std::max(need, info.workspace_bytes);
  }
  *out = need;
  return FRISK_OK;
}

int frisk_b200_reduce_run(const frisk_reduce_desc* desc, const void* src, void* dst, void* workspace,
                          size_t ws_bytes, void* stream) {
  if (!desc) return FRISK_ERR_INVALID_ARGUMENT;
  const int es = elem_bytes(desc->dtype);
  const bool aligned = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  int64_t slots = 1;
  if (es && desc->kind >= 0 && desc->kind <= 3)
    if (int rc = slots_for(*desc, aligned, &slots)) return rc;
  Plan p;
  if (int rc = make_plan(*desc, aligned, slots, &p)) return rc;
  if (desc->outer == 0 || desc->inner == 0) return FRISK_OK;
  if (!dst || (!src && desc->extent > 0)) {
    frisk_internal_set_error("reduce: null src or dst");
    return FRISK_ERR_INVALID_ARGUMENT;
  }
  if ((reinterpret_cast<uintptr_t>(src) % es) || (reinterpret_cast<uintptr_t>(dst) % es)) {
    frisk_internal_set_error("reduce: src and dst must be aligned to the element size");
    return FRISK_ERR_MISALIGNED;
  }
  if (p.ws_bytes && (!workspace || ws_bytes < p.ws_bytes)) {
    frisk_internal_set_error("reduce: workspace missing or too small");
    return FRISK_ERR_WORKSPACE;
  }
  if (p.ws_bytes && (reinterpret_cast<uintptr_t>(workspace) & 15)) {
    frisk_internal_set_error("reduce: workspace must be 16-byte aligned");
    return FRISK_ERR_MISALIGNED;
  }
  int prev = -1;
  if (desc->device >= 0) {
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
    if (prev != desc->device && (e = cudaSetDevice(desc->device)) != cudaSuccess) return fail_cuda(e, "cudaSetDevice");
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
  switch (desc->dtype) {
    case FRISK_DT_F32: e = run_kind<float>(*desc, p, src, dst, workspace, st); break;
    case FRISK_DT_F16: e = run_kind<__half>(*desc, p, src, dst, workspace, st); break;
    default: e = run_kind<__nv_bfloat16>(*desc, p, src, dst, workspace, st); break;
  }
  if (prev >= 0 && prev != desc->device) cudaSetDevice(prev);
  if (e != cudaSuccess) return fail_cuda(e, "reduce kernel launch");
  return FRISK_OK;
}

int frisk_b200_reduce_run_host(const frisk_reduce_desc* desc, const void* src, void* dst) {
  if (!desc) return FRISK_ERR_INVALID_ARGUMENT;
  const int es = elem_bytes(desc->dtype);
  if (!es) {
    frisk_internal_set_error("reduce: element type must be f32, f16 or bf16");
    return FRISK_ERR_UNSUPPORTED;
  }
  if (desc->outer < 0 || desc->extent < 0 || desc->inner < 0) return FRISK_ERR_INVALID_ARGUMENT;
  const size_t src_bytes = (size_t)(desc->outer * desc->extent * desc->inner) * es;
  const size_t dst_bytes = (size_t)(desc->outer * desc->inner) * es;
  if (dst_bytes == 0) return FRISK_OK;
  if (!dst || (src_bytes && !src)) return FRISK_ERR_INVALID_ARGUMENT;
  size_t ws_bytes = 0;
  if (int rc = frisk_b200_reduce_workspace_bytes(desc, &ws_bytes)) return rc;
  int prev = -1;
  if (desc->device >= 0) {
    cudaError_t e = cudaGetDevice(&prev);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
    if ((e = cudaSetDevice(desc->device)) != cudaSuccess) return fail_cuda(e, "cudaSetDevice");
  }
  void *dsrc = nullptr, *ddst = nullptr, *dws = nullptr;
  cudaStream_t st = nullptr;
  int rc = FRISK_OK;
  cudaError_t e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
  if (e == cudaSuccess) e = cudaMalloc(&dsrc, std::max<size_t>(src_bytes, 16));
  if (e == cudaSuccess) e = cudaMalloc(&ddst, dst_bytes);
  if (e == cudaSuccess && ws_bytes) e = cudaMalloc(&dws, ws_bytes);
  if (e == cudaSuccess && src_bytes) e = cudaMemcpyAsync(dsrc, src, src_bytes, cudaMemcpyHostToDevice, st);
  if (e == cudaSuccess && !desc->clear) e = cudaMemcpyAsync(ddst, dst, dst_bytes, cudaMemcpyHostToDevice, st);
  if (e == cudaSuccess) {
    frisk_reduce_desc d = *desc;
    d.device = -1;
    rc = frisk_b200_reduce_run(&d, dsrc, ddst, dws, ws_bytes, st);
    if (rc == FRISK_OK) e = cudaMemcpyAsync(dst, ddst, dst_bytes, cudaMemcpyDeviceToHost, st);
  }
  if (e == cudaSuccess && rc == FRISK_OK) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) rc = fail_cuda(e, "frisk_b200_reduce_run_host");
  if (st) cudaStreamSynchronize(st);
  cudaFree(dsrc);
  cudaFree(ddst);
  cudaFree(dws);
  if (st) cudaStreamDestroy(st);
  if (prev >= 0 && prev != desc->device) cudaSetDevice(prev);
  return rc;
}

}  // extern "C"
