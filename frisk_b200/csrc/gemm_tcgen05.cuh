// Persistent, warp-specialised GEMM for sm_100a:
//   warp 0   : TMA producer  (global -> 128B-swizzled shared memory, mbarrier completion)
//   warp 1   : MMA issuer    (tcgen05.mma, fp32 accumulators in tensor memory)
//   warps 2-5: epilogue      (tcgen05.ld -> registers -> scale / cast -> global)
// One kernel serves two plans:
//   * whole-tile mode: every CTA walks output tiles (128*mi x tile_n) round-robin and writes C;
//   * split mode     : the (tile, k-block) units are dealt in contiguous ranges to all CTAs
//                      ("stream-K"); partial sums are added into an fp32 workspace and a
//                      small finalize kernel casts them to C.  With the operands swapped on the
//                      host (weights feed the 128-row operand) this is the skinny / decode path:
//                      the weight matrix is streamed once from HBM by all SMs.
// The kernel computes D[r, c] = sum_k Arole[r, k] * Brole[c, k]; the host decides whether D is C
// or C transposed (`transposed_out`).
//
// Every wait on an mbarrier is bounded: when it runs out the CTA raises a flag in shared memory,
// ORs a code into the status word, lets all roles fall through to the common tear-down (which
// frees tensor memory) and returns.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"

namespace frisk {

constexpr int kMaxStages = 12;
constexpr int kGemmThreads = 192;
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s per wait, far above any legitimate wait

enum : int32_t {
  kStatusProducerTimeout = 1,
  kStatusMmaTimeout = 2,
  kStatusEpilogueTimeout = 4,
  kStatusTestTimeout = 8
};

struct OperandParams {
  uint64_t desc_base;         // UMMA shared-memory descriptor without the start address
  uint32_t stage_bytes;       // bytes of one pipeline stage taken by this operand
  uint32_t num_boxes;         // TMA boxes per stage
  uint32_t box_bytes;
  uint32_t box_mn;            // extent of one box along the operand's M/N dimension
  uint32_t mn_major;          // 1: M/N is the contiguous global dimension
  uint32_t k_step_bytes;      // start-address advance per UMMA K step
  uint32_t sub_stride_bytes;  // distance between 128-row sub-tiles inside a stage
};

struct GemmParams {
  OperandParams a, b;  // a: 128-row (UMMA M) operand, b: UMMA N operand
  uint32_t idesc;      // tcgen05 instruction descriptor
  uint32_t kind_f8;    // 0: kind::f16, 1: kind::f8f6f4
  uint32_t mi;         // 128-row sub-tiles per CTA tile (1 or 2)
  uint32_t tile_n;     // UMMA N
  uint32_t bk_elems;   // K elements per stage
  uint32_t k_steps;    // MMAs per stage and sub-tile
  uint32_t stages;
  uint32_t stage_bytes;
  uint32_t acc_bufs;   // accumulator buffers in tensor memory (1 or 2)
  uint32_t tmem_cols;  // power of two >= 32
  uint32_t rows, cols; // extent of D
  uint32_t tiles_r, tiles_c, num_kb;
  uint32_t group_r;    // tile rasterisation: rows of tiles walked together
  uint32_t split_mode;
  // epilogue
  void* C;
  float* ws;               // fp32 partial sums, C orientation, leading dimension ws_ld
  const float* row_scale;  // per D row, or nullptr
  const float* col_scale;  // per D column, or nullptr
  int64_t ldc;
  int64_t ws_ld;
  int32_t c_type;          // frisk_dtype of C
  uint32_t transposed_out; // 1: D[r, c] is C[c, r]
  uint32_t clear_accum;
  uint32_t c_vec_ok;       // C rows allow 16-byte stores
  int32_t* status;
};

__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity,
                                             volatile uint32_t* abort_flag, int32_t* status,
                                             int32_t code) {
  if (ptx::mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (ptx::mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0xFF) == 0) {
      if (*abort_flag) return false;
      if (ptx::globaltimer_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        if (status) atomicOr(status, code);
        return false;
      }
    }
  }
}

// Sequence of (tile, k-block range) work items of one CTA; identical in all three roles.
struct WorkIter {
  uint32_t tile, kb0, kb1;
  // whole-tile mode
  uint32_t next_tile, tile_step, num_tiles;
  // split mode
  uint64_t u, u_end;
  uint32_t num_kb, split;

  __device__ void init(const GemmParams& p) {
    num_kb = p.num_kb;
    split = p.split_mode;
    num_tiles = p.tiles_r * p.tiles_c;
    if (split) {
      const uint64_t total = (uint64_t)num_tiles * num_kb;
      u = total * blockIdx.x / gridDim.x;
      u_end = total * (blockIdx.x + 1) / gridDim.x;
    } else {
      next_tile = blockIdx.x;
      tile_step = gridDim.x;
    }
  }
  __device__ bool next() {
    if (split) {
      if (u >= u_end) return false;
      tile = (uint32_t)(u / num_kb);
      kb0 = (uint32_t)(u - (uint64_t)tile * num_kb);
      const uint64_t left = u_end - u;
      kb1 = (left < (uint64_t)(num_kb - kb0)) ? kb0 + (uint32_t)left : num_kb;
      u += kb1 - kb0;
      return true;
    }
    if (next_tile >= num_tiles) return false;
    tile = next_tile;
    next_tile += tile_step;
    kb0 = 0;
    kb1 = num_kb;
    return true;
  }
};

// Tile index -> (tile row, tile column).  Tiles are walked in bands of `group_r` tile rows,
// down the band first, so that CTAs running at the same time share A rows and B columns in L2.
__device__ __forceinline__ void tile_coords(const GemmParams& p, uint32_t tile, uint32_t& tr,
                                            uint32_t& tc) {
  const uint32_t band_tiles = p.group_r * p.tiles_c;
  const uint32_t band = tile / band_tiles;
  const uint32_t first_r = band * p.group_r;
  const uint32_t rows_in_band = min(p.group_r, p.tiles_r - first_r);
  const uint32_t in_band = tile - band * band_tiles;
  tr = first_r + in_band % rows_in_band;
  tc = in_band / rows_in_band;
}

template <typename T>
__device__ __forceinline__ T cast_out(float v);
template <>
__device__ __forceinline__ float cast_out<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half cast_out<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 cast_out<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}
template <typename T>
__device__ __forceinline__ float cast_in(T v);
template <>
__device__ __forceinline__ float cast_in<float>(float v) { return v; }
template <>
__device__ __forceinline__ float cast_in<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float cast_in<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

// Writes NC accumulator values of one D row (columns col0 .. col0+NC-1) held by this thread.
template <typename TC, int NC>
__device__ __forceinline__ void epilogue_store(const GemmParams& p, uint32_t row, uint32_t col0,
                                               const uint32_t (&acc)[NC]) {
  if (row >= p.rows) return;
  const float rs = p.row_scale ? __ldg(p.row_scale + row) : 1.0f;
  if (p.split_mode) {
    // raw partial sums; scales and the cast happen in the finalize kernel
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const uint32_t col = col0 + j;
      if (col < p.cols) {
        float* dst = p.transposed_out ? p.ws + (int64_t)col * p.ws_ld + row
                                      : p.ws + (int64_t)row * p.ws_ld + col;
        atomicAdd(dst, __uint_as_float(acc[j]));
      }
    }
    return;
  }
  TC* C = reinterpret_cast<TC*>(p.C);
  if (p.transposed_out) {
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const uint32_t col = col0 + j;
      if (col < p.cols) {
        float v = __uint_as_float(acc[j]) * rs;
        if (p.col_scale) v *= __ldg(p.col_scale + col);
        TC* dst = C + (int64_t)col * p.ldc + row;
        if (!p.clear_accum) v += cast_in<TC>(*dst);
        *dst = cast_out<TC>(v);
      }
    }
    return;
  }
  TC* dst = C + (int64_t)row * p.ldc + col0;
  constexpr int kPerVec = 16 / (int)sizeof(TC);
  if (p.c_vec_ok && col0 + NC <= p.cols) {
#pragma unroll
    for (int v0 = 0; v0 < NC; v0 += kPerVec) {
      union {
        uint4 u;
        TC e[kPerVec];
      } pack;
      if (!p.clear_accum) pack.u = *reinterpret_cast<const uint4*>(dst + v0);
#pragma unroll
      for (int j = 0; j < kPerVec; ++j) {
        float v = __uint_as_float(acc[v0 + j]) * rs;
        if (p.col_scale) v *= __ldg(p.col_scale + col0 + v0 + j);
        if (!p.clear_accum) v += cast_in<TC>(pack.e[j]);
        pack.e[j] = cast_out<TC>(v);
      }
      *reinterpret_cast<uint4*>(dst + v0) = pack.u;
    }
  } else {
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const uint32_t col = col0 + j;
      if (col < p.cols) {
        float v = __uint_as_float(acc[j]) * rs;
        if (p.col_scale) v *= __ldg(p.col_scale + col);
        if (!p.clear_accum) v += cast_in<TC>(dst[j]);
        dst[j] = cast_out<TC>(v);
      }
    }
  }
}

template <typename TC>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kMaxStages];
  __shared__ __align__(8) uint64_t bar_empty[kMaxStages];
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ uint32_t abort_word;

  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t lane = threadIdx.x & 31;
  volatile uint32_t* abort_flag = &abort_word;

  // tiles live in dynamic shared memory, 1024-byte aligned (one swizzle atom)
  const uint32_t tiles_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;

  if (threadIdx.x == 0) {
    abort_word = 0;
    for (uint32_t s = 0; s < p.stages; ++s) {
      ptx::mbar_init(ptx::smem_u32(&bar_full[s]), 1);
      ptx::mbar_init(ptx::smem_u32(&bar_empty[s]), 1);
    }
    for (uint32_t i = 0; i < 2; ++i) {
      ptx::mbar_init(ptx::smem_u32(&bar_acc_full[i]), 1);
      ptx::mbar_init(ptx::smem_u32(&bar_acc_empty[i]), 4);  // one arrival per epilogue warp
    }
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), p.tmem_cols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  WorkIter work;
  work.init(p);

  if (warp == 0) {
    // ------------------------------------------------------------- TMA producer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, issued = 0;
      bool ok = true;
      while (ok && work.next()) {
        uint32_t tr, tc;
        tile_coords(p, work.tile, tr, tc);
        const int32_t r0 = (int32_t)(tr * 128u * p.mi);
        const int32_t c0 = (int32_t)(tc * p.tile_n);
        for (uint32_t kb = work.kb0; kb < work.kb1; ++kb) {
          if (!bounded_wait(ptx::smem_u32(&bar_empty[stage]), phase ^ 1, abort_flag, p.status,
                            kStatusProducerTimeout)) {
            ok = false;
            break;
          }
          const uint32_t full = ptx::smem_u32(&bar_full[stage]);
          ptx::mbar_arrive_expect_tx(full, p.stage_bytes);
          const uint32_t a_dst = tiles_base + stage * p.stage_bytes;
          const uint32_t b_dst = a_dst + p.a.stage_bytes;
          const int32_t k0 = (int32_t)(kb * p.bk_elems);
          for (uint32_t bx = 0; bx < p.a.num_boxes; ++bx) {
            const int32_t mn = r0 + (int32_t)(bx * p.a.box_mn);
            if (p.a.mn_major)
              ptx::tma_load_2d(a_dst + bx * p.a.box_bytes, &tmap_a, full, mn, k0);
            else
              ptx::tma_load_2d(a_dst + bx * p.a.box_bytes, &tmap_a, full, k0, mn);
          }
          for (uint32_t bx = 0; bx < p.b.num_boxes; ++bx) {
            const int32_t mn = c0 + (int32_t)(bx * p.b.box_mn);
            if (p.b.mn_major)
              ptx::tma_load_2d(b_dst + bx * p.b.box_bytes, &tmap_b, full, mn, k0);
            else
              ptx::tma_load_2d(b_dst + bx * p.b.box_bytes, &tmap_b, full, k0, mn);
          }
          ++issued;
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // Give copies that are still in flight a bounded chance to land before the CTA exits.
        // Stages below `stage` were last armed in the current round (parity `phase`), the others
        // in the previous one; a stage that was never armed is skipped.
        for (uint32_t s = 0; s < p.stages; ++s) {
          if (issued <= s) continue;
          const uint32_t armed_parity = (s < stage) ? phase : (phase ^ 1u);
          const uint64_t t0 = ptx::globaltimer_ns();
          while (!ptx::mbar_try_wait(ptx::smem_u32(&bar_full[s]), armed_parity) &&
                 ptx::globaltimer_ns() - t0 < 1000000ull) {
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, item = 0;
      bool ok = true;
      while (ok && work.next()) {
        const uint32_t acc = item % p.acc_bufs;
        const uint32_t acc_phase = (item / p.acc_bufs) & 1u;
        if (!bounded_wait(ptx::smem_u32(&bar_acc_empty[acc]), acc_phase ^ 1, abort_flag, p.status,
                          kStatusMmaTimeout)) {
          ok = false;
          break;
        }
        ptx::tc_fence_after();
        const uint32_t d_base = tmem_base + acc * (p.mi * p.tile_n);
        for (uint32_t kb = work.kb0; kb < work.kb1; ++kb) {
          if (!bounded_wait(ptx::smem_u32(&bar_full[stage]), phase, abort_flag, p.status,
                            kStatusMmaTimeout)) {
            ok = false;
            break;
          }
          ptx::tc_fence_after();
          const uint32_t a_addr = tiles_base + stage * p.stage_bytes;
          const uint32_t b_addr = a_addr + p.a.stage_bytes;
          for (uint32_t ks = 0; ks < p.k_steps; ++ks) {
            const uint64_t bdesc =
                p.b.desc_base | (uint64_t)(((b_addr + ks * p.b.k_step_bytes) & 0x3FFFFu) >> 4);
            for (uint32_t sub = 0; sub < p.mi; ++sub) {
              const uint64_t adesc =
                  p.a.desc_base |
                  (uint64_t)(((a_addr + sub * p.a.sub_stride_bytes + ks * p.a.k_step_bytes) &
                              0x3FFFFu) >> 4);
              const uint32_t accumulate = (kb > work.kb0 || ks > 0) ? 1u : 0u;
              if (p.kind_f8)
                ptx::mma_f8(d_base + sub * p.tile_n, adesc, bdesc, p.idesc, accumulate);
              else
                ptx::mma_f16(d_base + sub * p.tile_n, adesc, bdesc, p.idesc, accumulate);
            }
          }
          ptx::tc_commit(ptx::smem_u32(&bar_empty[stage]));  // frees the stage when the MMAs retire
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        ptx::tc_commit(ptx::smem_u32(&bar_acc_full[acc]));
        ++item;
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------- epilogue
    const uint32_t quarter = warp & 3u;  // TMEM lanes 32*quarter .. +31 belong to this warp
    uint32_t item = 0;
    bool ok = true;
    while (ok && work.next()) {
      const uint32_t acc = item % p.acc_bufs;
      const uint32_t acc_phase = (item / p.acc_bufs) & 1u;
      uint32_t tr, tc;
      tile_coords(p, work.tile, tr, tc);
      // the tcgen05.ld below is warp-collective: leave the loop only as a whole warp
      ok = __all_sync(0xffffffffu,
                      bounded_wait(ptx::smem_u32(&bar_acc_full[acc]), acc_phase, abort_flag,
                                   p.status, kStatusEpilogueTimeout));
      if (!ok) break;
      ptx::tc_fence_after();
      for (uint32_t sub = 0; sub < p.mi; ++sub) {
        const uint32_t row = (tr * p.mi + sub) * 128u + quarter * 32u + lane;
        const uint32_t t_row = tmem_base + ((quarter * 32u) << 16) + acc * (p.mi * p.tile_n) +
                               sub * p.tile_n;
        if ((p.tile_n & 31u) == 0) {
          for (uint32_t cc = 0; cc < p.tile_n; cc += 32) {
            uint32_t v[32];
            ptx::tmem_ld_32x32b_x32(t_row + cc, v);
            ptx::tmem_ld_wait();
            epilogue_store<TC, 32>(p, row, tc * p.tile_n + cc, v);
          }
        } else {
          for (uint32_t cc = 0; cc < p.tile_n; cc += 16) {
            uint32_t v[16];
            ptx::tmem_ld_32x32b_x16(t_row + cc, v);
            ptx::tmem_ld_wait();
            epilogue_store<TC, 16>(p, row, tc * p.tile_n + cc, v);
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&bar_acc_empty[acc]));
      ++item;
    }
    __syncwarp();
  }

  // ---------------------------------------------------------------- tear-down
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, p.tmem_cols);
  }
}

// Casts the fp32 partial sums of a split plan into C and clears them for the next run.
template <typename TC>
__global__ void splitk_finalize_kernel(float* __restrict__ ws, int64_t ws_ld, TC* __restrict__ C,
                                       int64_t ldc, int64_t M, int64_t N,
                                       const float* __restrict__ scale_m,
                                       const float* __restrict__ scale_n, int clear_accum) {
  const int64_t n4 = (N + 3) / 4;
  const int64_t total = M * n4;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / n4;
    const int64_t n0 = (i - m * n4) * 4;
    float* src = ws + m * ws_ld + n0;
    float v[4];
    const bool full = (n0 + 4 <= N) && ((ws_ld & 3) == 0);
    if (full) {
      const float4 t = __ldcg(reinterpret_cast<const float4*>(src));
      v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
      *reinterpret_cast<float4*>(src) = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
      for (int j = 0; j < 4; ++j) {
        if (n0 + j < N) {
          v[j] = __ldcg(src + j);
          src[j] = 0.f;
        }
      }
    }
    const float sm = scale_m ? scale_m[m] : 1.0f;
    for (int j = 0; j < 4; ++j) {
      if (n0 + j < N) {
        float x = v[j] * sm;
        if (scale_n) x *= scale_n[n0 + j];
        TC* dst = C + m * ldc + n0 + j;
        if (!clear_accum) x += cast_in<TC>(*dst);
        *dst = cast_out<TC>(x);
      }
    }
  }
}

}  // namespace frisk
