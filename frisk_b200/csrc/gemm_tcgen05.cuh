// Persistent, warp-specialised GEMM for sm_100a:
//   warps 0,6: TMA producers (global -> 128B-swizzled shared memory, mbarrier completion);
//              they take alternate k-blocks, because one warp cannot issue a stage's loads as
//              fast as the tensor pipe consumes a stage
//   warp 1   : MMA issuer    (tcgen05.mma, fp32 accumulators in tensor memory)
//   warps 2-5: epilogue      (tcgen05.ld -> registers -> scale / cast -> global)
// Two instantiations of one template:
//   * whole tiles (kSplit = false): every CTA walks output tiles (128 x tile_n) round-robin and
//     writes C;
//   * K-split (kSplit = true), the few-row ("skinny" / decode) plans: the operands are swapped
//     on the host (the weights feed the 128-row operand) and several CTAs share a tile's K range,
//     so the weight matrix is streamed once from HBM by many SMs.  Split mode 3: one cluster per
//     tile, a K slice per CTA, partial tiles pushed through distributed shared memory and summed
//     by their owners.  Split mode 2: (tile, k-block) units dealt in contiguous ranges to the
//     CTAs ("stream-K"), partials in private workspace slots, summed by the last CTA to arrive.
//     Split mode 1: partials added to an fp32 workspace with atomics, cast by a second kernel.
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
constexpr int kMaxPeers = 7;   // a node has eight GPUs: seven others
// Staging area of the whole-tile epilogue: each of the four epilogue warps owns 32 rows x 128 bytes.
constexpr uint32_t kEpiStageBytesPerWarp = 32u * 128u;
constexpr uint32_t kEpiStageBytes = 4u * kEpiStageBytesPerWarp;
// Measurement builds (-DFRISK_B200_MEASURE) keep the debug modes and the clock stamps of CTA 0;
// the normal build compiles them out of the kernels.
#ifdef FRISK_B200_MEASURE
constexpr bool kMeasureBuild = true;
// FRISK_STAMP(cond, slot): CTA 0 records its clock, relative to kernel entry, in trace[slot].
#define FRISK_STAMP(cond, slot)                                  \
  do {                                                           \
    if (trace && (cond)) trace[(slot)] = clock64() - t_entry;    \
  } while (0)
#define FRISK_MEASURE_ONLY(...) __VA_ARGS__
#else
constexpr bool kMeasureBuild = false;
#define FRISK_STAMP(cond, slot) \
  do {                          \
  } while (0)
#define FRISK_MEASURE_ONLY(...)
#endif
// Warps that wait for a long time sleep between polls: a tight polling loop takes issue slots
// from the MMA warp on the same SM sub-partition and nearly halves its issue rate.
constexpr uint32_t kEpilogueBackoffNs = 128;
constexpr uint32_t kProducerBackoffNs = 32;
constexpr int kProducerWarps = 2;  // warps 0 and 6 issue the TMA loads of alternate k-blocks
constexpr int kGemmThreads = 224;
// ~0.3 s of SM clock per wait: far above any legitimate wait (a whole GEMM takes milliseconds),
// short enough that a stuck kernel is gone well before a shared GPU's context-switch timeout
constexpr long long kWaitLimitCycles = 1ll << 29;

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

// Tensor maps of the destinations of a TMA-store epilogue: C, then every peer's copy.
struct CStoreMaps {
  CUtensorMap m[1 + kMaxPeers];
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
  uint32_t seg_kb;     // 3xTF32 plans: k-blocks per K segment (num_kb = 3 * seg_kb)
  uint32_t group_r;    // tile rasterisation: rows of tiles walked together (bands) ...
  uint32_t group_c;    // ... or, when not 0, columns of tiles walked together (panels)
  uint32_t l2_hints;   // bit 0: a-role loads evict-first in L2, bit 1: b-role loads evict-last
  uint32_t split_mode;  // 0: whole tiles; 1: stream-K, atomics into ws + finalize kernel;
                        // 2: stream-K, private partial slots, the last CTA of a tile reduces
                        // 3: one cluster per tile, each CTA a K slice, partials summed
                        //    through distributed shared memory (no workspace)
  uint32_t max_items;   // split mode 2: most tiles one CTA's unit range can touch
  uint32_t cluster_k;   // split mode 3: CTAs per cluster = K slices per tile
  uint32_t red_overlay; // split mode 3: the region the partials are pushed into lies ON the stage
                        // buffers instead of behind them (one more cluster barrier, before the
                        // pushes: every CTA's main loop must be over), which leaves the whole of
                        // shared memory to the pipeline
  // CTA-pair kernel: work items (whole tiles, then half-width items of the last wave's tiles)
  uint32_t n_items, narrow_from, idesc_narrow;
  // CTA-pair kernel, K planes: K is cut into k_parts parts of kb_per k-blocks; an item is one part
  // of one tile, and part z leaves as fp32 into plane z (C + z * plane_elems elements, which the
  // host points at the workspace); kplanes_sum_kernel then folds the planes into the caller's C.
  // k_parts <= 1: whole K per item.
  uint32_t k_parts, kb_per;
  uint64_t plane_elems;
  uint32_t* counters;   // split mode 2: k-blocks arrived per tile (zero between launches)
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
  uint32_t epilogue_backoff_ns;  // sleep between polls of the accumulator-ready barrier
  // whole-tile epilogue (the one-CTA whole-tile kernel and the CTA-pair kernel)
  uint32_t epi_staged;     // 1: rows go through shared memory and leave as 128-byte row pieces
                           // (2: the same with linear instead of swizzled staging rows)
                           // 3: rows go through shared memory and leave as TMA tensor stores
                           //    (CTA-pair kernel; two staging buffers per warp)
  uint32_t n_peers;        // other GPUs that receive a copy of every C tile (row-sharded all-gather)
  void* peer_c[kMaxPeers]; // where this GPU's rows of C start in each peer's buffer (same ldc)
  // frisk.reduce of C over its columns, folded into the epilogue
  uint32_t rr_kind;        // 0: none; 1 + frisk_reduce_kind
  float* rr_partials;      // [2 * tiles_c][rows] fp32: one fold per row and half tile
  uint32_t debug_mode;     // measurement only: bit 0 = issue no loads, bit 1 = issue no MMAs
  long long* trace;        // measurement only: clock64 samples of CTA 0 (may be nullptr)
  int32_t* status;
};

// Slow path of bounded_wait: polls until the phase completes, the CTA aborts or the limit runs
// out.  Called by whole warps (every lane polls the same barrier, so the outcome is warp-uniform).
__device__ __noinline__ bool bounded_wait_slow(uint32_t bar, uint32_t parity,
                                               volatile uint32_t* abort_flag, int32_t* status,
                                               int32_t code, uint32_t backoff_ns) {
  const long long t0 = clock64();
  bool done = false;
  while (!done) {
#pragma unroll 1
    for (int i = 0; i < 256 && !done; ++i) {
      done = ptx::mbar_try_wait(bar, parity) != 0;
      if (!done && backoff_ns) __nanosleep(backoff_ns);
    }
    if (done) break;
    if (*abort_flag) break;
    if (clock64() - t0 > kWaitLimitCycles) {
      *abort_flag = 1;
      if (status) atomicOr(status, code);
      break;
    }
  }
  // one answer for the whole warp: the callers go on to warp-collective instructions
  return __all_sync(0xffffffffu, done);
}

// Waits for a phase of an mbarrier with a limit.  Returns false when the limit ran out here or in
// another role of the CTA; the caller then falls through to the kernel's tear-down.
__device__ __forceinline__ bool bounded_wait(uint32_t bar, uint32_t parity,
                                             volatile uint32_t* abort_flag, int32_t* status,
                                             int32_t code, uint32_t backoff_ns = 0) {
  // the vote makes the outcome provably warp-uniform for the compiler (see the role branches)
  if (__all_sync(0xffffffffu, ptx::mbar_try_wait(bar, parity))) return true;
  return bounded_wait_slow(bar, parity, abort_flag, status, code, backoff_ns);
}

// Sequence of (tile, k-block range) work items of one CTA; identical in all three roles.
struct WorkIter {
  uint32_t tile, kb0, kb1;
  // whole-tile mode
  uint32_t next_tile, tile_step, num_tiles;
  // split mode
  uint32_t u, u_end;   // total units x grid size stays below 2^32 (checked when planning)
  uint32_t num_kb, split;

  __device__ void init(uint32_t num_kb_, uint32_t split_, uint32_t num_tiles_,
                       uint32_t cluster_k = 1) {
    num_kb = num_kb_;
    split = split_;
    num_tiles = num_tiles_;
    if (split == 3) {
      // cluster c owns tile c; the CTA of rank r in it owns k-blocks [num_kb r / S, num_kb (r+1) / S).
      // S is a power of two: shifts, because a division costs this short kernel ~100 cycles a time
      const uint32_t sh = 31u - __clz(cluster_k);
      const uint32_t t = blockIdx.x >> sh, r = blockIdx.x & (cluster_k - 1u);
      tile = t;
      kb0 = (num_kb * r) >> sh;
      kb1 = (num_kb * (r + 1)) >> sh;
      u = 0;
      u_end = 1;   // one work item
    } else if (split) {
      const uint32_t total = num_tiles * num_kb;
      u = total * blockIdx.x / gridDim.x;
      u_end = total * (blockIdx.x + 1) / gridDim.x;
    } else {
      next_tile = blockIdx.x;
      tile_step = gridDim.x;
    }
  }
  __device__ bool next() {
    if (split == 3) {
      if (u >= u_end) return false;
      u = u_end;
      return true;
    }
    if (split) {
      if (u >= u_end) return false;
      tile = u / num_kb;
      kb0 = u - tile * num_kb;
      const uint32_t left = u_end - u;
      kb1 = (left < num_kb - kb0) ? kb0 + left : num_kb;
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

// Tile index -> (tile row, tile column).  Two walks:
//   bands  (group_c == 0): `group_r` tile rows at a time, down the band first, so that CTAs running
//          at the same time share A rows and B columns in L2; every band streams all of B;
//   panels (group_c != 0): `group_c` tile columns at a time, along the panel's columns first, then
//          down all the rows: the panel of B (group_c x tile_n columns, all of K) stays in L2 while
//          A streams past it once per panel -- the walk for a tall A against a B that does not
//          fit in L2 as a whole.
__device__ __forceinline__ void tile_coords(uint32_t group_r, uint32_t tiles_r, uint32_t tiles_c,
                                            uint32_t tile, uint32_t& tr, uint32_t& tc,
                                            uint32_t group_c = 0) {
  if (tiles_c == 1) {  // one column of tiles (every split plan): nothing to divide
    tr = tile;
    tc = 0;
    return;
  }
  if (group_c) {
    const uint32_t panel_tiles = group_c * tiles_r;
    const uint32_t panel = tile / panel_tiles;
    const uint32_t first_c = panel * group_c;
    const uint32_t cols_in_panel = min(group_c, tiles_c - first_c);
    const uint32_t in_panel = tile - panel * panel_tiles;
    tr = in_panel / cols_in_panel;
    tc = first_c + in_panel % cols_in_panel;
    return;
  }
  const uint32_t band_tiles = group_r * tiles_c;
  const uint32_t band = tile / band_tiles;
  const uint32_t first_r = band * group_r;
  const uint32_t rows_in_band = min(group_r, tiles_r - first_r);
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

// The epilogue's view of the kernel parameters.  Every role copies what its loop needs out of the
// __grid_constant__ parameter block into plain locals first: the block is read through its address,
// and the inline-PTX statements clobber memory, so a field left in the block would be re-fetched
// with a generic load after every one of them (measured: ~350 cycles per tcgen05.mma issued).
struct EpiArgs {
  void* C;
  float* ws;
  const float* row_scale;
  const float* col_scale;
  int64_t ldc, ws_ld;
  uint32_t rows, cols;
  uint32_t split_mode, transposed_out, clear_accum, c_vec_ok;
};

// Writes NC accumulator values of one D row (columns col0 .. col0+NC-1) held by this thread.
template <typename TC, int NC>
__device__ __forceinline__ void epilogue_store(const EpiArgs& p, uint32_t row, uint32_t col0,
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

// ---- whole-tile epilogue: values -> (row fold) -> C, directly or through shared memory ---------
// What the whole-tile kernels need beyond EpiArgs.  `peers` points into the kernel's parameter
// block (GemmParams::peer_c), which is indexed at run time: the loops over the peers are kept
// rolled, because this code shares the SM's instruction cache with the MMA issue loop and every
// kilobyte of unrolled stores showed up in the main loop's rate.
struct EpiExt {
  uint32_t staged, n_peers, rr_kind;
  void* const* peers;
  // staged == 3: the rows leave through TMA stores.  c_maps[0] describes C, c_maps[1 + q] peer q's
  // copy; tma_seq counts the warp's chunks (the staging buffer alternates with it).
  const CUtensorMap* c_maps = nullptr;
  uint32_t tma_seq = 0;
};

__device__ __forceinline__ float fold_identity(uint32_t rr_kind) {
  // 1 add, 2 mul, 3 min, 4 max
  return rr_kind == 1u ? 0.f : rr_kind == 2u ? 1.f : rr_kind == 3u ? __int_as_float(0x7f800000)
                                                                   : __int_as_float(0xff800000);
}
__device__ __forceinline__ float fold_step(uint32_t rr_kind, float a, float b) {
  // min / max skip NaN operands like fminf / fmaxf
  return rr_kind == 1u ? a + b : rr_kind == 2u ? a * b : rr_kind == 3u ? fminf(a, b) : fmaxf(a, b);
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}

// A warp's staging area holds 32 rows x 128 bytes in the 128-byte swizzle: the 16-byte chunk j of
// row r sits at chunk position j ^ (r & 7).  A warp's 32 writes of one chunk column (lane = row)
// and its reads of four whole rows (8 lanes per row) both touch every bank exactly four times,
// the minimum for 512 bytes.
// `xor_mask` is 7 for that layout; 0 leaves the rows linear (desc.epilogue = 3, kept to measure
// what the swizzle buys: every chunk-column write then hits one bank group eight times).
__device__ __forceinline__ uint32_t staged_chunk(uint32_t stage, uint32_t r, uint32_t j,
                                                 uint32_t xor_mask) {
  return stage + r * 128u + ((j ^ (r & xor_mask)) << 4);
}
template <typename TC>
__device__ __forceinline__ TC* staged_elem(uint32_t stage, uint32_t r, uint32_t c, uint32_t xor_mask) {
  constexpr uint32_t kPerVec = 16u / (uint32_t)sizeof(TC);
  const uint32_t a = staged_chunk(stage, r, c / kPerVec, xor_mask) + (c % kPerVec) * (uint32_t)sizeof(TC);
  return reinterpret_cast<TC*>(__cvta_shared_to_generic(a));
}

// Element-wise traffic between the staging area and C, with bounds: the path of a C that cannot
// take 16-byte accesses and of the chunk that crosses the last column.  Rolled loops, out of line.
template <typename TC, int NC>
__device__ __noinline__ void stage_old_c(const TC* C, int64_t ldc, uint32_t rows, uint32_t cols,
                                         uint32_t stage, uint32_t lane, uint32_t warp_row0,
                                         uint32_t col0, uint32_t xor_mask) {
#pragma unroll 1
  for (uint32_t e = lane; e < 32u * NC; e += 32u) {
    const uint32_t r = e / NC, c = e % NC;
    TC v = cast_out<TC>(0.f);
    if (warp_row0 + r < rows && col0 + c < cols) v = C[(int64_t)(warp_row0 + r) * ldc + col0 + c];
    *staged_elem<TC>(stage, r, c, xor_mask) = v;
  }
}
template <typename TC, int NC>
__device__ __noinline__ void staged_rows_out(TC* C, void* const* peers, uint32_t n_peers,
                                             int64_t ldc, uint32_t rows, uint32_t cols,
                                             uint32_t stage, uint32_t lane, uint32_t warp_row0,
                                             uint32_t col0, uint32_t xor_mask) {
#pragma unroll 1
  for (uint32_t e = lane; e < 32u * NC; e += 32u) {
    const uint32_t r = e / NC, c = e % NC;
    if (warp_row0 + r >= rows || col0 + c >= cols) continue;
    const TC v = *staged_elem<TC>(stage, r, c, xor_mask);
    const int64_t off = (int64_t)(warp_row0 + r) * ldc + col0 + c;
    C[off] = v;
#pragma unroll 1
    for (uint32_t q = 0; q < n_peers; ++q) reinterpret_cast<TC*>(peers[q])[off] = v;
  }
}

// One warp's 32 rows x NC columns of D = C (lane = row; NC * sizeof(TC) = 128 bytes): scale, add
// the old C if asked, round once, fold the rounded values into `red` (the row fold sees what a
// reduce of the stored C would see), and store:
//   staged: the rows go through the warp's staging area and leave as whole 128-byte row pieces,
//           four rows per store instruction, to C and to every peer's copy;
//   TMA:    the rows go into one of the warp's two staging buffers and one lane issues a tensor
//           store (cp.async.bulk.tensor, clipped at C's extents by the hardware) per destination;
//           the buffer is written again only after those stores have read it;
//   direct: every thread writes its own row piece (16-byte stores at row stride);
//   a C without 16-byte alignment, or the chunk that crosses the last column, goes element-wise.
// `stage` is the warp's staging area (shared-memory address), `warp_row0` the D row of lane 0.
template <typename TC, int NC>
__device__ __forceinline__ void epilogue_chunk(const EpiArgs& p, EpiExt& x, uint32_t stage,
                                               uint32_t lane, uint32_t warp_row0, uint32_t col0,
                                               const uint32_t (&acc)[NC], float& red) {
  constexpr int kPerVec = 16 / (int)sizeof(TC);
  constexpr int kVecs = NC / kPerVec;
  static_assert(kVecs == 8, "a chunk is 128 bytes of a C row");
  const uint32_t row = warp_row0 + lane;
  const bool row_ok = row < p.rows;
  const bool full = col0 + NC <= p.cols;          // warp-uniform
  const bool vec = p.c_vec_ok && full;            // warp-uniform
  const uint32_t xm = x.staged == 2u ? 0u : 7u;
  TC* const C = reinterpret_cast<TC*>(p.C);
  TC* const crow = C + (int64_t)row * p.ldc + col0;
  union Pack {
    uint4 u;
    TC e[kPerVec];
  };
  Pack out[kVecs];
  const bool tma = x.staged == 3u;  // warp-uniform; the plan guarantees a 16-byte aligned C
  if (tma) {
    // The stores of the chunk before last read the buffer this chunk goes into; the element-wise
    // read of an old C below uses the first buffer whatever the turn, so it waits for all of them.
    if (lane == 0) {
      if (!p.clear_accum && !vec) ptx::bulk_wait_group_read<0>();
      else ptx::bulk_wait_group_read<1>();
    }
    __syncwarp();
  }
  if (!p.clear_accum) {
    if (vec) {
      if (row_ok) {
#pragma unroll
        for (int v0 = 0; v0 < kVecs; ++v0) out[v0].u = *reinterpret_cast<const uint4*>(crow + v0 * kPerVec);
      }
    } else {
      stage_old_c<TC, NC>(C, p.ldc, p.rows, p.cols, stage, lane, warp_row0, col0, xm);
      __syncwarp();
#pragma unroll
      for (int v0 = 0; v0 < kVecs; ++v0) out[v0].u = ld_shared_v4(staged_chunk(stage, lane, (uint32_t)v0, xm));
      __syncwarp();
    }
  }
  const float rs = (p.row_scale && row_ok) ? __ldg(p.row_scale + row) : 1.0f;
  // The common cases get loops without per-element tests: on a shape whose main loop is short the
  // epilogue's instruction count is the kernel's time (measured: 2.2 x the instructions, and 6 us
  // more per tile, with the tests inside one generic loop).
  if (full && p.clear_accum && !p.col_scale && (x.rr_kind == 1u || x.rr_kind >= 3u)) {
    // the fold of the rounded values with the kind fixed outside the loop (add, min, max)
    if (x.rr_kind == 1u) {
#pragma unroll
      for (int j = 0; j < NC; ++j) {
        const TC o = cast_out<TC>(__uint_as_float(acc[j]) * rs);
        out[j / kPerVec].e[j % kPerVec] = o;
        red += cast_in<TC>(o);
      }
    } else if (x.rr_kind == 3u) {
#pragma unroll
      for (int j = 0; j < NC; ++j) {
        const TC o = cast_out<TC>(__uint_as_float(acc[j]) * rs);
        out[j / kPerVec].e[j % kPerVec] = o;
        red = fminf(red, cast_in<TC>(o));
      }
    } else {
#pragma unroll
      for (int j = 0; j < NC; ++j) {
        const TC o = cast_out<TC>(__uint_as_float(acc[j]) * rs);
        out[j / kPerVec].e[j % kPerVec] = o;
        red = fmaxf(red, cast_in<TC>(o));
      }
    }
  } else if (full && p.clear_accum && !x.rr_kind) {
    if (!p.col_scale) {
#pragma unroll
      for (int j = 0; j < NC; ++j)
        out[j / kPerVec].e[j % kPerVec] = cast_out<TC>(__uint_as_float(acc[j]) * rs);
    } else {
      const float* cs = p.col_scale + col0;
#pragma unroll
      for (int j = 0; j < NC; ++j)
        out[j / kPerVec].e[j % kPerVec] = cast_out<TC>(__uint_as_float(acc[j]) * rs * __ldg(cs + j));
    }
  } else {
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const bool col_ok = full || col0 + j < p.cols;
      float v = __uint_as_float(acc[j]) * rs;
      if (p.col_scale && col_ok) v *= __ldg(p.col_scale + col0 + j);
      if (!p.clear_accum) v += cast_in<TC>(out[j / kPerVec].e[j % kPerVec]);
      const TC o = cast_out<TC>(v);
      out[j / kPerVec].e[j % kPerVec] = o;
      if (x.rr_kind && col_ok) red = fold_step(x.rr_kind, red, cast_in<TC>(o));
    }
  }
  if (vec && !x.staged) {
    if (row_ok) {
#pragma unroll
      for (int v0 = 0; v0 < kVecs; ++v0) *reinterpret_cast<uint4*>(crow + v0 * kPerVec) = out[v0].u;
#pragma unroll 1
      for (uint32_t q = 0; q < x.n_peers; ++q) {
        TC* prow = reinterpret_cast<TC*>(x.peers[q]) + (int64_t)row * p.ldc + col0;
#pragma unroll
        for (int v0 = 0; v0 < kVecs; ++v0) *reinterpret_cast<uint4*>(prow + v0 * kPerVec) = out[v0].u;
      }
    }
    return;
  }
  if (tma) {
    const uint32_t buf = stage + (x.tma_seq & 1u) * kEpiStageBytesPerWarp;
    ++x.tma_seq;
#pragma unroll
    for (int v0 = 0; v0 < kVecs; ++v0) st_shared_v4(staged_chunk(buf, lane, (uint32_t)v0, 7u), out[v0].u);
    ptx::fence_proxy_async_smem();   // the writes above, made visible to the TMA unit
    __syncwarp();
    if (lane == 0) {
      if (warp_row0 < p.rows && col0 < p.cols) {
#pragma unroll 1
        for (uint32_t q = 0; q <= x.n_peers; ++q)
          ptx::tma_store_2d(x.c_maps + q, buf, (int32_t)col0, (int32_t)warp_row0);
      }
      ptx::bulk_commit_group();   // one group per chunk, empty or not: the waits count groups
    }
    return;
  }
#pragma unroll
  for (int v0 = 0; v0 < kVecs; ++v0) st_shared_v4(staged_chunk(stage, lane, (uint32_t)v0, xm), out[v0].u);
  __syncwarp();
  if (vec) {
    const uint32_t sub = lane >> 3, ch = lane & 7u;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const uint32_t rr = (uint32_t)it * 4u + sub;
      const uint4 piece = ld_shared_v4(staged_chunk(stage, rr, ch, xm));
      if (warp_row0 + rr < p.rows) {
        const int64_t off = (int64_t)(warp_row0 + rr) * p.ldc + col0 + ch * kPerVec;
        *reinterpret_cast<uint4*>(C + off) = piece;
#pragma unroll 1
        for (uint32_t q = 0; q < x.n_peers; ++q)
          *reinterpret_cast<uint4*>(reinterpret_cast<TC*>(x.peers[q]) + off) = piece;
      }
    }
  } else {
    staged_rows_out<TC, NC>(C, x.peers, x.n_peers, p.ldc, p.rows, p.cols, stage, lane, warp_row0, col0, xm);
  }
  __syncwarp();   // the staging area is rewritten by the next chunk
}

// The warp's 32 rows of one work item: `cols_item` columns from D column `col0`, accumulator
// rows at tensor-memory address `t_row`.  Columns are taken 128 bytes of C at a time; the
// tensor-memory loads of a piece are issued together and waited for once.
template <typename TC>
__device__ __forceinline__ void epilogue_item(const EpiArgs& ep, EpiExt& ex, uint32_t stage,
                                              uint32_t lane, uint32_t warp_row0, uint32_t col0,
                                              uint32_t cols_item, uint32_t t_row, float& red) {
  constexpr int CH = 128 / (int)sizeof(TC);
  for (uint32_t cc = 0; cc < cols_item; cc += CH) {
    uint32_t v[CH];
#pragma unroll
    for (int h = 0; h < CH / 32; ++h)
      ptx::tmem_ld_32x32b_x32(t_row + cc + 32u * h, reinterpret_cast<uint32_t(&)[32]>(v[32 * h]));
    ptx::tmem_ld_wait();
    epilogue_chunk<TC, CH>(ep, ex, stage, lane, warp_row0, col0 + cc, v, red);
  }
}

// ---- frisk.reduce over the columns of C, folded into the whole-tile epilogue -------------------
// Every thread folds the rounded values of its row as they pass (epilogue_chunk) and writes one
// fp32 per (row, half tile) to partials[slot][row]; row_fold_finalize_kernel, launched behind the
// GEMM, folds a row's slots in slot order into the destination.  (A last-arriving CTA folding the
// slots inside the GEMM kernel -- an arrival counter, a fence, three rendezvous of the epilogue
// threads -- was measured first: with that code merely present, a GEMM that never ran it executed
// 34 % more instructions and kept the tensor pipe busy 70 % instead of 95 % of the cycles.)
struct RowFold {
  uint32_t kind, nslots;
  float* partials;
};

// `weight` is 2 for a whole tile (which also marks the tile's second slot as empty), 1 for a half.
__device__ __forceinline__ void row_fold_store(const RowFold& f, uint32_t row, uint32_t rows,
                                               uint32_t slot, uint32_t weight, float red) {
  if (row < rows) {
    f.partials[(size_t)slot * rows + row] = red;
    if (weight == 2u) f.partials[(size_t)(slot + 1u) * rows + row] = fold_identity(f.kind);
  }
}

// Rendezvous of the 128 epilogue threads on an mbarrier (count 128), bounded like every other
// wait of the kernel: a named hardware barrier could not give up if one warp had left the loop.
__device__ __forceinline__ bool epilogue_rendezvous(uint32_t bar, uint32_t& phase,
                                                    volatile uint32_t* abort_flag, int32_t* status) {
  ptx::mbar_arrive(bar);
  const bool ok = bounded_wait(bar, phase, abort_flag, status, kStatusEpilogueTimeout);
  phase ^= 1u;
  return ok;
}

// ---- split mode 2: partial tiles in private slots, reduced by the last CTA to arrive -----------
// A slot holds one partial tile as [column][row] fp32 (rows fastest, so a warp's 32 rows of one
// column are one 128-byte store).  Slot of CTA c for tile t: c * max_items + (t - first tile of c).
__device__ __forceinline__ uint32_t unit_begin(uint32_t total_units, uint32_t cta, uint32_t grid) {
  return total_units * cta / grid;
}

template <int NC>
__device__ __forceinline__ void slot_store(float* slot, uint32_t tile_rows, uint32_t r_local,
                                           uint32_t c0, const uint32_t (&acc)[NC]) {
#pragma unroll
  for (int j = 0; j < NC; ++j)
    slot[(size_t)(c0 + j) * tile_rows + r_local] = __uint_as_float(acc[j]);
}

// Sums, in CTA order (so the result does not depend on who arrives last), every partial of
// `tile` for 16 columns of one row.
__device__ __forceinline__ void reduce_slots_x16(const float* ws, uint32_t tile, uint32_t num_kb,
                                                 uint32_t total_units, uint32_t grid,
                                                 uint32_t max_items, uint32_t tile_rows,
                                                 uint32_t tile_elems, uint32_t r_local, uint32_t c0,
                                                 uint32_t (&acc)[16]) {
  float sum[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) sum[j] = 0.f;
  const uint32_t u_lo = tile * num_kb, u_hi = u_lo + num_kb;
  uint32_t c = u_lo * grid / total_units;
  while (c + 1 < grid && unit_begin(total_units, c + 1, grid) <= u_lo) ++c;
  while (c > 0 && unit_begin(total_units, c, grid) > u_lo) --c;
  for (; c < grid; ++c) {
    const uint32_t b = unit_begin(total_units, c, grid);
    if (b >= u_hi) break;
    const uint32_t e = unit_begin(total_units, c + 1, grid);
    if (e <= u_lo) continue;
    const uint32_t first_tile = b / num_kb;
    const float* slot = ws + (size_t)(c * max_items + (tile - first_tile)) * tile_elems;
#pragma unroll
    for (int j = 0; j < 16; ++j) sum[j] += __ldcg(slot + (size_t)(c0 + j) * tile_rows + r_local);
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = __float_as_uint(sum[j]);
}

// Most partials of one tile the vector reduction handles; a tile with more (a grid much larger
// than the tile count) takes the row-wise reduce_slots_x16 instead.
constexpr uint32_t kMaxContrib = 16;
constexpr int kReduceBatch = 8;  // slots summed per round of loads by reduce_tile

// Lists, in CTA order, the slots that hold a partial of `tile`; returns how many there are (only
// the first `cap` are stored).  One thread calls this while the tile's MMAs are still running.
__device__ __noinline__ uint32_t list_contributors(uint32_t tile, uint32_t num_kb,
                                                   uint32_t total_units, uint32_t grid,
                                                   uint32_t max_items, uint32_t* out,
                                                   uint32_t cap) {
  const uint32_t u_lo = tile * num_kb, u_hi = u_lo + num_kb;
  uint32_t c = u_lo * grid / total_units;
  while (c + 1 < grid && unit_begin(total_units, c + 1, grid) <= u_lo) ++c;
  while (c > 0 && unit_begin(total_units, c, grid) > u_lo) --c;
  uint32_t n = 0;
  uint32_t b = unit_begin(total_units, c, grid);
  for (; c < grid && b < u_hi; ++c) {
    const uint32_t e = unit_begin(total_units, c + 1, grid);
    if (e > u_lo) {
      if (n < cap) out[n] = c * max_items + (tile - b / num_kb);
      ++n;
    }
    b = e;
  }
  return n;
}

// Four consecutive D rows of one column: scale, accumulate into C if asked, cast and store.
template <typename TC>
__device__ __forceinline__ void store_rows4(const EpiArgs& p, uint32_t row, uint32_t col,
                                            float4 s) {
  if (col >= p.cols || row >= p.rows) return;
  const float v[4] = {s.x, s.y, s.z, s.w};
  TC* C = reinterpret_cast<TC*>(p.C);
  struct alignas(4 * sizeof(TC)) Pack {
    TC e[4];
  };
  if (p.transposed_out && p.clear_accum && p.c_vec_ok && row + 3 < p.rows) {
    // C[col, row .. row+3] is contiguous and, with row a multiple of 4, aligned for one store
    Pack pack;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float o = v[j] * (p.row_scale ? __ldg(p.row_scale + row + j) : 1.0f);
      if (p.col_scale) o *= __ldg(p.col_scale + col);
      pack.e[j] = cast_out<TC>(o);
    }
    *reinterpret_cast<Pack*>(C + (int64_t)col * p.ldc + row) = pack;
    return;
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const uint32_t r = row + j;
    if (r < p.rows) {
      float o = v[j] * (p.row_scale ? __ldg(p.row_scale + r) : 1.0f);
      if (p.col_scale) o *= __ldg(p.col_scale + col);
      TC* dst = p.transposed_out ? C + (int64_t)col * p.ldc + r : C + (int64_t)r * p.ldc + col;
      if (!p.clear_accum) o += cast_in<TC>(*dst);
      *dst = cast_out<TC>(o);
    }
  }
}

// Sums the listed slots, in list order (so the result does not depend on who arrives last), and
// writes the tile to C.  Called by the 128 epilogue threads (tid 0 .. 127); each handles float4
// pieces tid, tid + 128, ... of the [column][row] slot image, 4 pieces x 8 slots in flight.
template <typename TC>
__device__ __forceinline__ void reduce_tile(const EpiArgs& p, const uint32_t* slots, uint32_t n,
                                            uint32_t tile_rows, uint32_t tile_elems,
                                            uint32_t row0, uint32_t col0, uint32_t tid) {
  const uint32_t n_vec = tile_elems >> 2;            // a multiple of 512
  const uint32_t row_shift = (tile_rows == 256u) ? 8u : 7u;
  for (uint32_t v0 = tid; v0 < n_vec; v0 += 512u) {
    float4 sum[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (uint32_t k0 = 0; k0 < n; k0 += kReduceBatch) {
      float4 x[kReduceBatch][4];
#pragma unroll
      for (int kk = 0; kk < kReduceBatch; ++kk) {
        if (k0 + kk < n) {
          const float4* s =
              reinterpret_cast<const float4*>(p.ws + (size_t)slots[k0 + kk] * tile_elems) + v0;
#pragma unroll
          for (int i = 0; i < 4; ++i) x[kk][i] = __ldcg(s + i * 128);
        }
      }
#pragma unroll
      for (int kk = 0; kk < kReduceBatch; ++kk) {
        if (k0 + kk < n) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            sum[i].x += x[kk][i].x;
            sum[i].y += x[kk][i].y;
            sum[i].z += x[kk][i].z;
            sum[i].w += x[kk][i].w;
          }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t e = (v0 + i * 128u) << 2;
      store_rows4<TC>(p, row0 + (e & (tile_rows - 1u)), col0 + (e >> row_shift), sum[i]);
    }
  }
}

// Split mode 3.  Rank r of a cluster owns rows [r R, (r + 1) R) of the tile, R = tile_rows /
// cluster size.  Every CTA pushes each part of its partial tile into the owner's shared memory
// (remote stores, no waiting), at [source rank][column][row in share] fp32; after one cluster
// barrier each owner sums what arrived, reading only its own shared memory, so a CTA may leave as
// soon as it has passed the barrier.  The sum runs over source ranks 0, 1, ... in that order.
template <int NC>
__device__ __forceinline__ void cluster_push(uint32_t dst, uint32_t col_stride_bytes, uint32_t c0,
                                             const uint32_t (&acc)[NC]) {
#pragma unroll
  for (int j = 0; j < NC; ++j) ptx::st_shared_cluster_u32(dst + (c0 + j) * col_stride_bytes, acc[j]);
}

template <typename TC>
__device__ __forceinline__ void reduce_share(const EpiArgs& p, uint32_t buf, uint32_t cluster_k,
                                             uint32_t rank, uint32_t share, uint32_t tile_n,
                                             uint32_t row0, uint32_t col0, uint32_t tid) {
  const uint32_t q_per_col = share >> 2;          // float4 pieces per column (share: 16 .. 128)
  const uint32_t q_sh = 31u - __clz(q_per_col);
  const uint32_t pieces = tile_n * q_per_col;
  const uint32_t src_stride = tile_n * share * 4u;  // bytes between two sources' images
  for (uint32_t i = tid; i < pieces; i += 128u) {
    const uint32_t col = i >> q_sh, q = i & (q_per_col - 1u);   // share is a power of two
    const uint32_t at = buf + (col * share + 4u * q) * 4u;
    float4 x[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < (int)cluster_k) x[k] = ptx::ld_shared_f32x4(at + k * src_stride);
    float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (k < (int)cluster_k) {
        sum.x += x[k].x;
        sum.y += x[k].y;
        sum.z += x[k].z;
        sum.w += x[k].w;
      }
    }
    store_rows4<TC>(p, row0 + rank * share + 4u * q, col0 + col, sum);
  }
}

// kSplit selects the K-split (stream-K) code at compile time.  The whole-tile instantiation carries
// none of it: with the slot reduction inlined the kernel needs 200+ registers and measurably slows
// the whole-tile main loop (8192^3 bf16: 0.98 ms against 0.83 ms), so the two are kept apart.
// kTf32 (whole tiles, C fp32) issues kind::tf32 MMAs: the 3xTF32 plan of fp32 GEMMs.
template <typename TC, bool kSplit, bool kTf32 = false>
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
  __shared__ uint32_t last_flag;
  __shared__ uint32_t contrib_n;
  __shared__ uint32_t contrib_slots[kMaxContrib];
  __shared__ __align__(8) uint64_t bar_epilogue;

  // The broadcast tells the compiler that the warp index is the same in every lane, so the role
  // branches below are uniform and the code inside them may use the uniform datapath (which the
  // TMA and tcgen05 instructions take their operands from).
  const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const uint32_t lane = threadIdx.x & 31;
  volatile uint32_t* abort_flag = &abort_word;

  // tiles live in dynamic shared memory, 1024-byte aligned (one swizzle atom)
  const uint32_t tiles_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t full0 = ptx::smem_u32(&bar_full[0]);
  const uint32_t empty0 = ptx::smem_u32(&bar_empty[0]);
  const uint32_t acc_full0 = ptx::smem_u32(&bar_acc_full[0]);
  const uint32_t acc_empty0 = ptx::smem_u32(&bar_acc_empty[0]);

  // fields every role needs, held in registers from here on
  const uint32_t stages = p.stages;
  const uint32_t stage_bytes = p.stage_bytes;
  const uint32_t mi = p.mi;
  const uint32_t tile_n = p.tile_n;
  const uint32_t acc_bufs = p.acc_bufs;
  const uint32_t tmem_cols = p.tmem_cols;
  const uint32_t tiles_r = p.tiles_r, tiles_c = p.tiles_c, group_r = p.group_r;
  const uint32_t debug_mode = kMeasureBuild ? p.debug_mode : 0u;
  int32_t* const status = p.status;
  const bool cluster_sync = kSplit && p.split_mode == 3 && p.cluster_k > 1;
  // with the overlaid reduce region every warp passes the cluster barrier twice
  const bool cluster_sync2 = cluster_sync && p.red_overlay != 0;
  // (measurement builds only) clock stamps of CTA 0, each relative to the stamping thread's own
  // clock at kernel entry, and the wall-clock entry and exit of every CTA at [1024 + 2 * CTA]
  FRISK_MEASURE_ONLY(
      long long* const trace = blockIdx.x == 0 ? p.trace : nullptr;
      const long long t_entry = trace ? clock64() : 0;
      if (p.trace && threadIdx.x == 64) p.trace[1024 + 2 * blockIdx.x] = (long long)ptx::globaltimer_ns();
      if (trace && threadIdx.x == 64) {
        trace[320] = 0;
        trace[324] = (long long)ptx::globaltimer_ns();
      })
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (uint32_t s = 0; s < stages; ++s) {
      ptx::mbar_init(full0 + 8 * s, 1);
      ptx::mbar_init(empty0 + 8 * s, 1);
    }
    for (uint32_t i = 0; i < 2; ++i) {
      ptx::mbar_init(acc_full0 + 8 * i, 1);
      ptx::mbar_init(acc_empty0 + 8 * i, 4);  // one arrival per epilogue warp
    }
    ptx::mbar_init(ptx::smem_u32(&bar_epilogue), 128);
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), tmem_cols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  // broadcast: a value loaded from shared memory is not warp-uniform for the compiler otherwise
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_base_slot, 0);
  // Everything above touched only this CTA's shared and tensor memory, so it may overlap the tail
  // of the previous kernel in the stream; global memory (operands a previous GEMM may have
  // written, the workspace a previous launch of this plan still uses) is touched only from here.
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();
  FRISK_STAMP(threadIdx.x == 64, 321);

  WorkIter work;
  work.init(p.num_kb, kSplit ? p.split_mode : 0u, tiles_r * tiles_c, kSplit ? p.cluster_k : 1u);

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------- TMA producer
    // The whole warp walks the loop (uniform control flow); one elected lane issues.
    {
      const uint32_t a_boxes = p.a.num_boxes, a_box_bytes = p.a.box_bytes, a_box_mn = p.a.box_mn;
      const uint32_t b_boxes = p.b.num_boxes, b_box_bytes = p.b.box_bytes, b_box_mn = p.b.box_mn;
      const uint32_t a_mn_major = p.a.mn_major, b_mn_major = p.b.mn_major;
      const uint32_t a_stage_bytes = p.a.stage_bytes;
      const uint32_t bk_elems = p.bk_elems;
      const uint32_t my_turn = warp == 0 ? 0u : 1u;
      uint32_t stage = 0, phase = 0, issued = 0, turn = 0;
      bool ok = true;
      while (ok && work.next()) {
        uint32_t tr, tc;
        tile_coords(group_r, tiles_r, tiles_c, work.tile, tr, tc);
        const int32_t r0 = (int32_t)(tr * 128u * mi);
        const int32_t c0 = (int32_t)(tc * tile_n);
        for (uint32_t kb = work.kb0; kb < work.kb1; ++kb) {
          if (turn != my_turn) {  // the other producer warp loads this k-block
            turn ^= 1u;
            if (++stage == stages) {
              stage = 0;
              phase ^= 1;
            }
            continue;
          }
          turn ^= 1u;
          ok = bounded_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, status,
                            kStatusProducerTimeout, kProducerBackoffNs);
          if (!ok) break;
          const uint32_t full = full0 + 8 * stage;
          FRISK_MEASURE_ONLY(const bool tr_on = trace && issued < 32 && warp == 0;)
          FRISK_STAMP(tr_on && ptx::elect_one(), 2 * issued);
          if (debug_mode & 1u) {
            if (ptx::elect_one()) ptx::mbar_arrive(full);
          } else {
            if (ptx::elect_one()) ptx::mbar_arrive_expect_tx(full, stage_bytes);
            FRISK_STAMP(tr_on && ptx::elect_one(), 256 + 4 * issued);
            const uint32_t a_dst = tiles_base + stage * stage_bytes;
            const uint32_t b_dst = a_dst + a_stage_bytes;
            // (3xTF32: the k-blocks of segment 0 read A_lo B_hi, of segment 1 A_hi B_lo, of segment 2
            // A_hi B_hi, out of A' = [lo | hi] and B' = [hi | lo])
            int32_t k0 = (int32_t)(kb * bk_elems), k0b = k0;
            if (kTf32) {
              const uint32_t seg = kb / p.seg_kb, kk = kb - seg * p.seg_kb;
              k0 = (int32_t)(((seg == 0u ? 0u : p.seg_kb) + kk) * bk_elems);
              k0b = (int32_t)(((seg == 1u ? p.seg_kb : 0u) + kk) * bk_elems);
            }
            for (uint32_t bx = 0; bx < a_boxes; ++bx) {
              const int32_t mn = r0 + (int32_t)(bx * a_box_mn);
              const int32_t x = a_mn_major ? mn : k0, y = a_mn_major ? k0 : mn;
              if (ptx::elect_one()) ptx::tma_load_2d(a_dst + bx * a_box_bytes, &tmap_a, full, x, y);
            }
            FRISK_STAMP(tr_on && ptx::elect_one(), 256 + 4 * issued + 1);
            for (uint32_t bx = 0; bx < b_boxes; ++bx) {
              const int32_t mn = c0 + (int32_t)(bx * b_box_mn);
              const int32_t x = b_mn_major ? mn : k0b, y = b_mn_major ? k0b : mn;
              if (ptx::elect_one()) ptx::tma_load_2d(b_dst + bx * b_box_bytes, &tmap_b, full, x, y);
            }
          }
          FRISK_STAMP(tr_on && ptx::elect_one(), 2 * issued + 1);
          // Reconverge here: without it the warp stays split after the elected-lane issues above
          // and walks the next wait that way (measured: 8192^3 bf16 0.89 ms without, 0.82 ms with).
          __syncwarp();
          ++issued;
          if (++stage == stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if (!ok) {
        // Give copies that are still in flight time to land before the CTA exits (a copy takes
        // a few microseconds at most; this waits about 50).
        const long long t0 = clock64();
        while (clock64() - t0 < 100000ll) {
        }
      }
    }
    __syncwarp();
    if (cluster_sync2) {  // see the epilogue role
      ptx::cluster_arrive();
      ptx::cluster_wait();
    }
    if (cluster_sync) {
      ptx::cluster_arrive();
      ptx::cluster_wait();
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    {
      const uint64_t a_desc_base = p.a.desc_base, b_desc_base = p.b.desc_base;
      const uint32_t a_k_step = p.a.k_step_bytes, b_k_step = p.b.k_step_bytes;
      const uint32_t a_sub_stride = p.a.sub_stride_bytes;
      const uint32_t a_stage_bytes = p.a.stage_bytes;
      const uint32_t idesc = p.idesc;
      const uint32_t kind_f8 = p.kind_f8;
      uint32_t stage = 0, phase = 0, item = 0;
      bool ok = true;
      while (ok && work.next()) {
        const uint32_t acc = item % acc_bufs;
        const uint32_t acc_phase = (item / acc_bufs) & 1u;
        ok = bounded_wait(acc_empty0 + 8 * acc, acc_phase ^ 1, abort_flag, status,
                          kStatusMmaTimeout);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t d_base = tmem_base + acc * (mi * tile_n);
        // The tensor pipe queues only a little work, so the time between the last MMA of one
        // k-block and the first of the next is idle time.  To keep it short the stage of k-block
        // i is released (tcgen05.commit) only after the first MMA of k-block i+1 has been issued,
        // and the barrier of k-block i+1 is polled before the last MMA of k-block i.
        uint32_t prev_stage = 0;
        bool have_prev = false;
        uint32_t ready = __all_sync(0xffffffffu, ptx::mbar_try_wait(full0 + 8 * stage, phase));
        for (uint32_t kb = work.kb0; kb < work.kb1; ++kb) {
          if (!ready) {
            ok = bounded_wait_slow(full0 + 8 * stage, phase, abort_flag, status, kStatusMmaTimeout,
                                   0);
            if (!ok) break;
          }
          ptx::tc_fence_after();
          // Everything below is computed by the whole warp (uniform values); only the issuing
          // instructions themselves sit under the elected lane.
          const uint32_t a_addr = tiles_base + stage * stage_bytes;
          const uint32_t b_addr = a_addr + a_stage_bytes;
          const uint64_t adesc0 = a_desc_base | (uint64_t)((a_addr & 0x3FFFFu) >> 4);
          const uint64_t bdesc0 = b_desc_base | (uint64_t)((b_addr & 0x3FFFFu) >> 4);
          const uint32_t first = (kb > work.kb0) ? 1u : 0u;
          FRISK_MEASURE_ONLY(const bool tr_on = trace && item == 0 && (kb - work.kb0) < 32;)
          FRISK_STAMP(tr_on && ptx::elect_one(), 64 + 3 * (kb - work.kb0));
          uint32_t next_stage = stage + 1, next_phase = phase;
          if (next_stage == stages) {
            next_stage = 0;
            next_phase ^= 1;
          }
          if (debug_mode & 2u) {
            if (ptx::elect_one()) ptx::mbar_arrive(empty0 + 8 * stage);
            ready = __all_sync(0xffffffffu, ptx::mbar_test_wait(full0 + 8 * next_stage, next_phase));
          } else {
            // the start-address field advances by whole 16-byte units and never carries out of
            // its 14 bits (the tiles end below 256 KiB), so the step is added to the low word
#pragma unroll
            for (uint32_t ks = 0; ks < 4; ++ks) {
              const uint64_t bdesc = bdesc0 + (uint64_t)((ks * b_k_step) >> 4);
              const uint64_t adesc = adesc0 + (uint64_t)((ks * a_k_step) >> 4);
              const uint32_t accumulate = first | (ks > 0 ? 1u : 0u);
              // (test_wait, not try_wait: try_wait suspends the warp for microseconds when the
              // phase is not complete, and after the CTA's last k-block it never completes)
              if (ks == 3)
                ready = __all_sync(0xffffffffu, ptx::mbar_test_wait(full0 + 8 * next_stage, next_phase));
              if (kTf32) {
                if (ptx::elect_one()) ptx::mma_tf32(d_base, adesc, bdesc, idesc, accumulate);
              } else if (kind_f8) {
                if (ptx::elect_one()) ptx::mma_f8(d_base, adesc, bdesc, idesc, accumulate);
                if (mi > 1 && ptx::elect_one())
                  ptx::mma_f8(d_base + tile_n, adesc + (a_sub_stride >> 4), bdesc, idesc, accumulate);
              } else {
                if (ptx::elect_one()) ptx::mma_f16(d_base, adesc, bdesc, idesc, accumulate);
                if (mi > 1 && ptx::elect_one())
                  ptx::mma_f16(d_base + tile_n, adesc + (a_sub_stride >> 4), bdesc, idesc, accumulate);
              }
              if (ks == 0 && have_prev && ptx::elect_one()) ptx::tc_commit(empty0 + 8 * prev_stage);
            }
            FRISK_STAMP(tr_on && ptx::elect_one(), 64 + 3 * (kb - work.kb0) + 1);
            prev_stage = stage;
            have_prev = true;
          }
          FRISK_STAMP(tr_on && ptx::elect_one(), 64 + 3 * (kb - work.kb0) + 2);
          stage = next_stage;
          phase = next_phase;
        }
        if (!ok) break;
        // release the last stage of this work item
        if (have_prev && ptx::elect_one()) ptx::tc_commit(empty0 + 8 * prev_stage);
        if (!ok) break;
        if (ptx::elect_one()) ptx::tc_commit(acc_full0 + 8 * acc);
        FRISK_STAMP(item == 0 && ptx::elect_one(), 323);
        __syncwarp();
        ++item;
      }
    }
    __syncwarp();
    if (cluster_sync2) {  // see the epilogue role
      ptx::cluster_arrive();
      ptx::cluster_wait();
    }
    if (cluster_sync) {
      ptx::cluster_arrive();
      ptx::cluster_wait();
    }
  } else {
    // ------------------------------------------------------------- epilogue
    if constexpr (!kSplit) {
      // whole tiles of 128 rows (mi == 1): lane = row, columns 128 bytes of C at a time
      EpiArgs ep;
      ep.C = p.C;
      ep.ws = nullptr;
      ep.row_scale = p.row_scale;
      ep.col_scale = p.col_scale;
      ep.ldc = p.ldc;
      ep.ws_ld = 0;
      ep.rows = p.rows;
      ep.cols = p.cols;
      ep.split_mode = 0;
      ep.transposed_out = 0;
      ep.clear_accum = p.clear_accum;
      ep.c_vec_ok = p.c_vec_ok;
      EpiExt ex;
      ex.staged = p.epi_staged;
      ex.n_peers = p.n_peers;
      ex.rr_kind = p.rr_kind;
      ex.peers = p.peer_c;
      RowFold rf;
      rf.kind = p.rr_kind;
      rf.nslots = 2u * tiles_c;
      rf.partials = p.rr_partials;
      const uint32_t quarter = warp & 3u;  // TMEM lanes 32*quarter .. +31 belong to this warp
      const uint32_t stage_area = tiles_base + stages * stage_bytes + quarter * kEpiStageBytesPerWarp;
      const uint32_t epi_backoff = p.epilogue_backoff_ns;
      uint32_t item = 0;
      bool ok = true;
      while (ok && work.next()) {
        const uint32_t acc = item % acc_bufs;
        const uint32_t acc_phase = (item / acc_bufs) & 1u;
        uint32_t tr, tc;
        tile_coords(group_r, tiles_r, tiles_c, work.tile, tr, tc);
        // the tcgen05.ld below is warp-collective: leave the loop only as a whole warp
        ok = bounded_wait(acc_full0 + 8 * acc, acc_phase, abort_flag, status, kStatusEpilogueTimeout,
                          epi_backoff);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t t_row = tmem_base + ((quarter * 32u) << 16) + acc * tile_n;
        float red = fold_identity(rf.kind);
        epilogue_item<TC>(ep, ex, stage_area, lane, tr * 128u + quarter * 32u, tc * tile_n, tile_n,
                          t_row, red);
        ptx::tc_fence_before();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(acc_empty0 + 8 * acc);
        if (rf.kind) row_fold_store(rf, tr * 128u + quarter * 32u + lane, ep.rows, 2u * tc, 2u, red);
        ++item;
      }
      __syncwarp();
    } else {
    EpiArgs ep;
    ep.C = p.C;
    ep.ws = p.ws;
    ep.row_scale = p.row_scale;
    ep.col_scale = p.col_scale;
    ep.ldc = p.ldc;
    ep.ws_ld = p.ws_ld;
    ep.rows = p.rows;
    ep.cols = p.cols;
    ep.split_mode = kSplit ? p.split_mode : 0u;
    ep.transposed_out = p.transposed_out;
    ep.clear_accum = p.clear_accum;
    ep.c_vec_ok = p.c_vec_ok;
    const uint32_t quarter = warp & 3u;  // TMEM lanes 32*quarter .. +31 belong to this warp
    const uint32_t split_mode = kSplit ? p.split_mode : 0u, max_items = p.max_items, num_kb_all = p.num_kb;
    const uint32_t tile_rows = 128u * mi, tile_elems = tile_rows * tile_n;
    const uint32_t total_units = tiles_r * tiles_c * num_kb_all;
    const uint32_t epi_bar = ptx::smem_u32(&bar_epilogue);
    const uint32_t epi_backoff = p.epilogue_backoff_ns;
    const uint32_t cluster_k = kSplit ? p.cluster_k : 1u;
    // (the cluster size is a power of two)
    const uint32_t cluster_sh = 31u - __clz(cluster_k);
    const uint32_t my_rank = blockIdx.x & (cluster_k - 1u), share = tile_rows >> cluster_sh;
    const uint32_t share_sh = 31u - __clz(share);
    const uint32_t red_base = cluster_sync2 ? tiles_base : tiles_base + stages * stage_bytes;
    bool passed_first = false;   // overlaid reduce region: this warp has been through the first barrier
    uint32_t epi_phase = 0;
    uint32_t item = 0;
    bool ok = true;
    while (ok && work.next()) {
      const uint32_t acc = item % acc_bufs;
      const uint32_t acc_phase = (item / acc_bufs) & 1u;
      uint32_t tr, tc;
      tile_coords(group_r, tiles_r, tiles_c, work.tile, tr, tc);
      // split mode 2: a work item that covers all of K is written straight to C; a partial one goes
      // to this CTA's private slot and the last CTA to arrive for the tile sums the slots
      const bool whole = work.kb0 == 0 && work.kb1 == num_kb_all;
      const bool to_slot = split_mode == 2 && !whole;
      EpiArgs ep_item = ep;
      if (split_mode >= 2) ep_item.split_mode = 0;
      float* slot = nullptr;
      // split mode 3: the partial is pushed into the shared memory of the tile's owners, into a
      // region behind the stage buffers that nothing else uses (an owner may still be streaming)
      const bool to_smem = split_mode == 3 && !whole;
      if (to_slot) {
        // worked out while the item's MMAs still run: where the partial goes, and (one thread) who
        // else holds a partial of this tile, in case this CTA turns out to be the last to arrive
        const uint32_t first_tile =
            unit_begin(total_units, blockIdx.x, gridDim.x) / num_kb_all;
        slot = ep.ws + (size_t)(blockIdx.x * max_items + (work.tile - first_tile)) * tile_elems;
        if (threadIdx.x == 64)
          contrib_n = list_contributors(work.tile, num_kb_all, total_units, gridDim.x, max_items,
                                        contrib_slots, kMaxContrib);
      }
      // the tcgen05.ld below is warp-collective: leave the loop only as a whole warp
      ok = bounded_wait(acc_full0 + 8 * acc, acc_phase, abort_flag, status, kStatusEpilogueTimeout,
                        epi_backoff);
      if (!ok) break;
      ptx::tc_fence_after();
      FRISK_STAMP(threadIdx.x == 64 && item < 4, 330 + 8 * item);
      if (cluster_sync2 && !passed_first) {
        // The partials land on the owners' stage buffers: nobody may push before every CTA of the
        // cluster has seen its last MMA complete (this warp just has, for its own CTA).
        ptx::cluster_arrive();
        ptx::cluster_wait();
        passed_first = true;
      }
      for (uint32_t sub = 0; sub < mi; ++sub) {
        const uint32_t r_local = sub * 128u + quarter * 32u + lane;
        const uint32_t row = tr * tile_rows + r_local;
        const uint32_t t_row =
            tmem_base + ((quarter * 32u) << 16) + acc * (mi * tile_n) + sub * tile_n;
        uint32_t push_dst = 0;
        if (to_smem) {
          const uint32_t owner = r_local >> share_sh, rr = r_local - owner * share;
          push_dst = ptx::mapa(red_base + ((my_rank * tile_n) * share + rr) * 4u, owner);
        }
        if ((tile_n & 31u) == 0) {
          for (uint32_t cc = 0; cc < tile_n; cc += 32) {
            uint32_t v[32];
            ptx::tmem_ld_32x32b_x32(t_row + cc, v);
            ptx::tmem_ld_wait();
            if (to_smem) cluster_push<32>(push_dst, share * 4u, cc, v);
            else if (to_slot) slot_store<32>(slot, tile_rows, r_local, cc, v);
            else epilogue_store<TC, 32>(ep_item, row, tc * tile_n + cc, v);
          }
        } else {
          for (uint32_t cc = 0; cc < tile_n; cc += 16) {
            uint32_t v[16];
            ptx::tmem_ld_32x32b_x16(t_row + cc, v);
            ptx::tmem_ld_wait();
            if (to_smem) cluster_push<16>(push_dst, share * 4u, cc, v);
            else if (to_slot) slot_store<16>(slot, tile_rows, r_local, cc, v);
            else epilogue_store<TC, 16>(ep_item, row, tc * tile_n + cc, v);
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(acc_empty0 + 8 * acc);
      FRISK_STAMP(threadIdx.x == 64 && item < 4, 330 + 8 * item + 1);
      if (to_slot) {
        __threadfence();      // this thread's partial is visible device-wide ...
        // ... and so is every epilogue thread's, before the count goes up
        ok = epilogue_rendezvous(epi_bar, epi_phase, abort_flag, status);
        if (!ok) break;
        if (threadIdx.x == 64) {
          const uint32_t mine = work.kb1 - work.kb0;
          const uint32_t before = atomicAdd(p.counters + work.tile, mine);
          last_flag = (before + mine == num_kb_all) ? 1u : 0u;
        }
        ok = epilogue_rendezvous(epi_bar, epi_phase, abort_flag, status);
        if (!ok) break;
        FRISK_STAMP(threadIdx.x == 64 && item < 4, 330 + 8 * item + 2);
        if (last_flag) {
          __threadfence();
          if (contrib_n <= kMaxContrib) {
            reduce_tile<TC>(ep_item, contrib_slots, contrib_n, tile_rows, tile_elems,
                            tr * tile_rows, tc * tile_n, threadIdx.x - 64u);
          } else {
            for (uint32_t sub = 0; sub < mi; ++sub) {
              const uint32_t r_local = sub * 128u + quarter * 32u + lane;
              const uint32_t row = tr * tile_rows + r_local;
              for (uint32_t cc = 0; cc < tile_n; cc += 16) {
                uint32_t v[16];
                reduce_slots_x16(ep.ws, work.tile, num_kb_all, total_units, gridDim.x, max_items,
                                 tile_rows, tile_elems, r_local, cc, v);
                epilogue_store<TC, 16>(ep_item, row, tc * tile_n + cc, v);
              }
            }
          }
          if (threadIdx.x == 64) p.counters[work.tile] = 0;  // ready for the next launch
          FRISK_STAMP(threadIdx.x == 64 && item < 4, 330 + 8 * item + 3);
        }
        // last_flag is rewritten by the next item
        ok = epilogue_rendezvous(epi_bar, epi_phase, abort_flag, status);
        if (!ok) break;
      }
      FRISK_STAMP(threadIdx.x == 64 && item < 4, 330 + 8 * item + 5);
      ++item;
    }
    __syncwarp();
    if (cluster_sync2 && !passed_first) {  // a warp that gave up before its item still takes part
      ptx::cluster_arrive();
      ptx::cluster_wait();
    }
    if (cluster_sync) {
      // Split mode 3.  Every warp of every CTA of the cluster passes this barrier exactly once
      // (and the one before the pushes, when the reduce region is overlaid on the stage buffers),
      // whatever happened in its role (all waits above are bounded), so a CTA that gave up cannot
      // strand its peers.  After it every partial has reached its owner, and nobody touches
      // another CTA's shared memory again, so each CTA leaves on its own.
      ptx::cluster_arrive();
      ptx::cluster_wait();
      FRISK_STAMP(threadIdx.x == 64, 326);
      if (!*abort_flag) {
        uint32_t tr, tc;
        tile_coords(group_r, tiles_r, tiles_c, blockIdx.x >> cluster_sh, tr, tc);
        EpiArgs ep_out = ep;
        ep_out.split_mode = 0;
        reduce_share<TC>(ep_out, red_base, cluster_k, my_rank, share, tile_n, tr * tile_rows,
                         tc * tile_n, threadIdx.x - 64u);
      }
      FRISK_STAMP(threadIdx.x == 64, 327);
    }
    }  // kSplit
  }

  // ---------------------------------------------------------------- tear-down
  ptx::tc_fence_before();
  __syncthreads();
  FRISK_MEASURE_ONLY(
      if (p.trace && threadIdx.x == 64) p.trace[1024 + 2 * blockIdx.x + 1] = (long long)ptx::globaltimer_ns();
      if (trace && threadIdx.x == 64) {
        trace[322] = clock64() - t_entry;
        trace[325] = (long long)ptx::globaltimer_ns();
      })
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, tmem_cols);
  }
}

// dst[row] = (clear ? fold : dst[row] (op) fold) of partials[0 .. nslots)[row], in slot order.
// Launched behind the GEMM as a programmatic dependent launch: it may be scheduled while the GEMM
// drains and waits here until the GEMM's writes are visible.
template <typename TC>
__global__ void __launch_bounds__(256) row_fold_finalize_kernel(const float* __restrict__ partials,
                                                                TC* __restrict__ dst, uint32_t rows,
                                                                uint32_t nslots, uint32_t kind,
                                                                uint32_t clear) {
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();
  const uint32_t row = blockIdx.x * blockDim.x + threadIdx.x;
  if (row >= rows) return;
  float r = fold_identity(kind);
  for (uint32_t sl = 0; sl < nslots; ++sl) r = fold_step(kind, r, __ldcg(partials + (size_t)sl * rows + row));
  if (!clear) r = fold_step(kind, cast_in<TC>(dst[row]), r);
  dst[row] = cast_out<TC>(r);
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

// The second launch of a K-planes plan: C = cast(scale_m * scale_n * (plane 0 + plane 1 + ...)
// (+ C)), the planes summed in their order, four columns per thread.  `ldp` (the planes' pitch) is
// a multiple of 4; `vec_ok`: four elements of C at a column that is a multiple of 4 may leave as
// one store.  Launched as a programmatic dependent of the GEMM, like row_fold_finalize_kernel.
template <typename TC>
__global__ void __launch_bounds__(256) kplanes_sum_kernel(const float* __restrict__ planes,
                                                          uint64_t plane_elems, uint32_t parts,
                                                          int64_t ldp, TC* __restrict__ C, int64_t ldc,
                                                          int64_t M, int64_t N,
                                                          const float* __restrict__ scale_m,
                                                          const float* __restrict__ scale_n,
                                                          int clear_accum, int vec_ok) {
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();
  const int64_t n4 = (N + 3) / 4;
  const int64_t total = M * n4;
  for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t m = i / n4;
    const int64_t n0 = (i - m * n4) * 4;
    const float* src = planes + m * ldp + n0;
    float4 s = __ldcg(reinterpret_cast<const float4*>(src));
    // (unrolled so that eight loads are in flight per thread; the adds keep the planes' order)
#pragma unroll 8
    for (uint32_t z = 1; z < parts; ++z) {
      const float4 t = __ldcg(reinterpret_cast<const float4*>(src + (size_t)z * plane_elems));
      s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
    }
    float v[4] = {s.x, s.y, s.z, s.w};
    const float sm = scale_m ? __ldg(scale_m + m) : 1.0f;
    TC* dst = C + m * ldc + n0;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);   // four elements of C (the first 8 bytes for 16-bit types)
    TC* e = reinterpret_cast<TC*>(&raw);
    const bool whole = vec_ok && n0 + 4 <= N;
    if (whole && !clear_accum) {
      if (sizeof(TC) == 4) raw = *reinterpret_cast<const uint4*>(dst);
      else *reinterpret_cast<uint2*>(&raw) = *reinterpret_cast<const uint2*>(dst);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (n0 + j < N) {
        float x = v[j] * sm;
        if (scale_n) x *= __ldg(scale_n + n0 + j);
        if (!clear_accum) x += cast_in<TC>(whole ? e[j] : dst[j]);
        e[j] = cast_out<TC>(x);
        if (!whole) dst[j] = e[j];
      }
    }
    if (whole) {
      if (sizeof(TC) == 4) *reinterpret_cast<uint4*>(dst) = raw;
      else *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(&raw);
    }
  }
}

}  // namespace frisk
