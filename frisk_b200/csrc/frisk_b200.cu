// C ABI of libfrisk_b200.so: plan creation, kernel choice, TMA descriptor encoding, launches.
// See include/frisk_b200.h for the contract of every entry point.
#include "../../include/frisk_b200.h"

#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>

#include "abi_internal.h"
#include "gemm_simt.cuh"
#include "gemm_tcgen05.cuh"
#include "gemm_tcgen05_pair.cuh"
#include "gemm_tcgen05_pair_ksplit.cuh"
#include "mma_peak.cuh"
#include "tf32_split.cuh"

namespace {

thread_local std::string g_last_error;

}  // namespace

void frisk_internal_set_error(const char* text) { g_last_error = text ? text : ""; }

namespace {

int cuda_fail(cudaError_t e, const char* what) {
  g_last_error = std::string(what) + ": " + cudaGetErrorString(e);
  return FRISK_ERR_CUDA;
}
#define FRISK_CUDA(call)                                   \
  do {                                                     \
    cudaError_t e__ = (call);                              \
    if (e__ != cudaSuccess) return cuda_fail(e__, #call);  \
  } while (0)

int elem_size(int dt) {
  switch (dt) {
    case FRISK_DT_F32: return 4;
    case FRISK_DT_F16: return 2;
    case FRISK_DT_BF16: return 2;
    case FRISK_DT_E4M3: return 1;
    case FRISK_DT_E5M2: return 1;
    default: return 0;
  }
}
bool is_fp8(int dt) { return dt == FRISK_DT_E4M3 || dt == FRISK_DT_E5M2; }

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The driver entry point is looked up through the runtime, so the library links against
// libcudart only and loads on machines without a driver.
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// One GEMM operand as the tcgen05 kernel sees it: `mn` rows of the product dimension, K deep.
struct OperandView {
  const void* ptr;
  int64_t mn, k, ld;  // extents and leading dimension in elements
  bool mn_major;      // the M/N dimension is contiguous in memory
};

}  // namespace

struct frisk_gemm_plan {
  frisk_gemm_desc d;   // the caller's problem
  // The problem the tensor-core kernel sees.  Equal to `d` except for a 3xTF32 plan, where A and B
  // are the split operands in the workspace: K three times as long, their own leading dimensions.
  frisk_gemm_desc kd;
  bool tf32 = false;
  bool tf32_pair = false;        // which whole-tile kernel runs the split problem
  int pair_cluster = 0;          // > 0: the CTA-pair kernel with K split over this many pairs per cluster
  size_t tf32_a_bytes = 0, tf32_b_bytes = 0;
  // Operands whose row pitch is not a multiple of 16 bytes (no tensor map can describe them) are
  // copied into the front of the workspace at a padded pitch (kd.lda / kd.ldb) before every run.
  size_t repack_a_bytes = 0, repack_b_bytes = 0;
  int device = -1;
  int sm_count = 148;
  bool have_device = false;
  frisk_gemm_plan_info info;
  frisk::GemmParams gp;  // everything but pointers
  size_t ws_bytes = 0;
  size_t slot_bytes = 0;  // split mode 2: bytes of partial-tile slots before the counters
  // fused row reduce: [2 * tiles_c][M] fp32 folds, one per row and half tile
  size_t rr_partial_bytes = 0;
  size_t dyn_smem = 0;
  frisk_tma_params lay_a, lay_b;  // the layout mapper's description of the staged operand tiles
  int plan_error = 0;
  // run-time caches
  CUtensorMap tmap_a, tmap_b;
  const void* cached_a = nullptr;
  const void* cached_b = nullptr;
  frisk::CStoreMaps c_maps;      // TMA-store epilogue: C and the peers' copies
  const void* cached_c[1 + frisk::kMaxPeers] = {};
  int64_t simt_fallback_runs = 0;  // runs a tensor-core plan sent to the CUDA-core kernel
  // device buffers of frisk_b200_gemm_run_host
  void *hA = nullptr, *hB = nullptr, *hC = nullptr, *hWs = nullptr, *hRr = nullptr;
  float *hSa = nullptr, *hSb = nullptr;
  int32_t* hStatus = nullptr;
  cudaStream_t hstream = nullptr;
  // pipelined form of frisk_b200_gemm_run_host: row chunks on three streams
  static constexpr int kMaxChunks = 16;
  cudaStream_t s_in = nullptr, s_out = nullptr;
  cudaEvent_t ev_in[kMaxChunks] = {}, ev_done[kMaxChunks] = {}, ev_start = nullptr;
  frisk_gemm_plan* chunk_plan = nullptr;  // the same GEMM over chunk_rows rows
  frisk_gemm_plan* tail_plan = nullptr;   // ... over the rows left after the last full chunk
  int64_t chunk_rows = 0;
  int n_chunks = 0;                       // 0: not decided yet; 1: no pipelining
};

namespace {

// UMMA shared-memory descriptor without the start address: leading / stride byte offsets in
// 16-byte units, the sm_100 descriptor version, and the swizzle (layout type) in bits 61..63.
uint64_t make_desc_base(uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout_type) {
  uint64_t d = 0;
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version of sm_100
  d |= (uint64_t)(layout_type & 7u) << 61;
  return d;
}

// Fills the shared-memory side of one operand for a tile of `tile_mn` rows and 128 bytes of K
// from what the layout mapper (frisk_b200_layout_to_tma: the reference's swizzle selection carried
// to TMA / UMMA fields) says about that tile, and keeps the mapper's answer in `lay`: there is one
// description of a staged tile, and the kernels run on it.
int fill_operand(frisk::OperandParams& o, frisk_tma_params& lay, bool mn_major, uint32_t tile_mn,
                 uint32_t es, uint32_t bk_elems) {
  frisk_layout_desc l;
  l.elem_bits = (int32_t)(8 * es);
  l.k_inner = mn_major ? 0 : 1;
  uint32_t mn_boxes = 1;  // K-major tiles taller than a TMA box (256 rows) are cut along M/N
  if (mn_major) {
    l.rows = bk_elems;    // the tile as stored: K rows of tile_mn contiguous elements
    l.cols = tile_mn;
  } else {
    mn_boxes = tile_mn > 256 ? 2 : 1;
    l.rows = tile_mn / mn_boxes;
    l.cols = bk_elems;
  }
  int rc = frisk_b200_layout_to_tma(&l, &lay);
  if (rc) return rc;
  // the kernels stage 128 bytes of K (or of M/N) per box row: the mapper must agree
  if (lay.swizzle_bytes != 128) return FRISK_ERR_UNSUPPORTED;
  o.mn_major = (uint32_t)lay.umma_major;
  o.stage_bytes = tile_mn * 128u;  // tile_mn x bk_elems elements either way
  o.box_bytes = (uint32_t)lay.box_outer * (uint32_t)lay.swizzle_bytes;
  o.desc_base = make_desc_base((uint32_t)lay.leading_byte_offset, (uint32_t)lay.stride_byte_offset,
                               (uint32_t)lay.umma_layout_type);
  o.k_step_bytes = (uint32_t)lay.k_step_bytes;
  if (mn_major) {
    // boxes of (128 bytes of M/N) x (bk rows of K); each box is one column of swizzle atoms
    o.box_mn = (uint32_t)lay.box_inner;
    o.num_boxes = (uint32_t)lay.num_boxes;
    o.sub_stride_bytes = (128u / o.box_mn) * o.box_bytes;   // 128 rows further along M/N
  } else {
    o.box_mn = (uint32_t)lay.box_outer;
    o.num_boxes = mn_boxes;
    o.sub_stride_bytes = 128u * 128u;
  }
  return FRISK_OK;
}

uint32_t make_idesc(int ab_type, bool a_mn_major, bool b_mn_major, uint32_t m, uint32_t n) {
  uint32_t fmt = 0;  // kind::f16: 0 = f16, 1 = bf16; kind::f8f6f4: 0 = e4m3, 1 = e5m2; kind::tf32: 2 = tf32
  if (ab_type == FRISK_DT_BF16 || ab_type == FRISK_DT_E5M2) fmt = 1;
  if (ab_type == FRISK_DT_F32) fmt = 2;
  uint32_t d = 0;
  d |= 1u << 4;  // fp32 accumulator
  d |= fmt << 7;
  d |= fmt << 10;
  d |= (a_mn_major ? 1u : 0u) << 15;
  d |= (b_mn_major ? 1u : 0u) << 16;
  d |= (n >> 3) << 17;
  d |= (m >> 4) << 24;
  return d;
}

int encode_operand_map(CUtensorMap* map, const OperandView& v, int dtype, uint32_t box_mn,
                       uint32_t bk_elems, int swizzle_bytes) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) {
    g_last_error = "cuTensorMapEncodeTiled not available from the driver";
    return FRISK_ERR_CUDA;
  }
  const uint32_t es = elem_size(dtype);
  CUtensorMapDataType dt = dtype == FRISK_DT_F16    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                           : dtype == FRISK_DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : dtype == FRISK_DT_F32  ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                                    : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t dims[2], strides[1];
  cuuint32_t box[2], estr[2] = {1, 1};
  if (v.mn_major) {
    dims[0] = (cuuint64_t)v.mn;
    dims[1] = (cuuint64_t)v.k;
    box[0] = box_mn;
    box[1] = bk_elems;
  } else {
    dims[0] = (cuuint64_t)v.k;
    dims[1] = (cuuint64_t)v.mn;
    box[0] = bk_elems;
    box[1] = box_mn;
  }
  strides[0] = (cuuint64_t)v.ld * es;
  CUresult r = fn(map, dt, 2, const_cast<void*>(v.ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle_bytes == 128  ? CU_TENSOR_MAP_SWIZZLE_128B
                  : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B
                  : swizzle_bytes == 32 ? CU_TENSOR_MAP_SWIZZLE_32B
                                        : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[160];
    snprintf(buf, sizeof buf,
             "cuTensorMapEncodeTiled failed (%d): dims %llu x %llu, stride %llu, box %u x %u", (int)r,
             (unsigned long long)dims[0], (unsigned long long)dims[1],
             (unsigned long long)strides[0], box[0], box[1]);
    g_last_error = buf;
    return FRISK_ERR_CUDA;
  }
  return FRISK_OK;
}

// Tensor map of a destination of the TMA-store epilogue: `rows` x `cols` elements of `dtype` at
// pitch `ld`, stored in boxes of 32 rows x 128 bytes out of 128-byte-swizzled shared memory.
int encode_store_map(CUtensorMap* map, void* ptr, int dtype, int64_t rows, int64_t cols, int64_t ld) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) {
    g_last_error = "cuTensorMapEncodeTiled not available from the driver";
    return FRISK_ERR_CUDA;
  }
  const uint32_t es = elem_size(dtype);
  CUtensorMapDataType dt = dtype == FRISK_DT_F16    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                           : dtype == FRISK_DT_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                    : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * es};
  cuuint32_t box[2] = {128u / es, 32u}, estr[2] = {1, 1};
  CUresult r = fn(map, dt, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[160];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed (%d) for C: %lld x %lld, pitch %lld",
             (int)r, (long long)rows, (long long)cols, (long long)ld);
    g_last_error = buf;
    return FRISK_ERR_CUDA;
  }
  return FRISK_OK;
}

uint32_t next_pow2_cols(uint32_t c) {
  uint32_t v = 32;
  while (v < c) v <<= 1;
  return v;
}

// Most dynamic shared memory a plan may use, and the opt-in value every kernel function is set
// to: the 227 KiB of an SM less room for the kernels' static barriers and flags.
constexpr size_t kMaxDynSmem = 227 * 1024 - 1024;
// Every tensor-core launch asks for all of it, whatever the plan's pipeline depth needs: that
// keeps the kernels at one CTA per SM, so a CTA never waits in tcgen05.alloc for tensor memory
// another CTA on its SM holds (with CTA pairs such a wait could close a cycle across two SMs).
constexpr size_t kLaunchDynSmem = kMaxDynSmem;

// Why a problem cannot take the tensor-core kernels (FRISK_TC_*; 0 = it can).
int tcgen05_ineligible_reason(const frisk_gemm_desc& d) {
  if (d.a_type != FRISK_DT_F16 && d.a_type != FRISK_DT_BF16 && !is_fp8(d.a_type))
    return FRISK_TC_INPUT_TYPE;
  const int es = elem_size(d.a_type);
  if ((d.lda * es) % 16 || (d.ldb * es) % 16) return FRISK_TC_PITCH;
  if (d.M >= (1ll << 31) || d.N >= (1ll << 31) || d.K >= (1ll << 31)) return FRISK_TC_EXTENT;
  // 8-bit operands are taken K-major only (A row-major, B column-major)
  if (is_fp8(d.a_type) && (d.transA || !d.transB)) return FRISK_TC_FP8_ORDER;
  return FRISK_TC_OK;
}
bool tcgen05_eligible(const frisk_gemm_desc& d) { return tcgen05_ineligible_reason(d) == FRISK_TC_OK; }

// fp32 problems the 3xTF32 plan can take: fp32 C, 16-byte row pitches (TMA), extents that stay
// below 2^31 after K is tripled, no scales, plain C = or += (the fold and the peers would work
// too; they are not wired to this plan).
bool tf32_eligible(const frisk_gemm_desc& d) {
  if (d.a_type != FRISK_DT_F32 || d.c_type != FRISK_DT_F32) return false;
  if ((d.lda % 4) || (d.ldb % 4)) return false;
  if (d.M >= (1ll << 31) || d.N >= (1ll << 31) || 3 * d.K + 4 >= (1ll << 31)) return false;
  if (d.scale_mode != FRISK_SCALE_NONE || d.row_reduce) return false;
  return true;
}
// ... and the ones it pays for: the split costs a pass over A and B and two more launches, and the
// tensor-core tiles are coarse; measured against the CUDA-core kernel the break-even is near
// 1 GFLOP (fp32 512^3, 0.27 GFLOP: 22 us on CUDA cores).
bool tf32_worthwhile(const frisk_gemm_desc& d) {
  return 2.0 * (double)d.M * (double)d.N * (double)d.K >= 1.0e9 && d.N >= 64 && d.K >= 64;
}

// Few rows of A against a wide B: the shape the swapped, K-split plan is for.  The kernel counts
// (tile, k-block) units in 32 bits and multiplies the count by the grid size, so the product has
// to stay below 2^32 (conservatively: the smallest tile and k-block the plan could pick).
bool skinny_shape(const frisk_gemm_desc& d, int sm_count) {
  if (!(d.M <= 128 && d.N >= 256 && !d.transA)) return false;
  const uint64_t units = (uint64_t)((d.N + 127) / 128) * (uint64_t)((d.K + 31) / 32);
  return units * (uint64_t)(sm_count + 1) < (1ull << 32);
}

bool skinny_clusters_fit(frisk_gemm_plan* pl);

// Whether the pair kernel cuts the tiles of its last wave in two (see plan_tcgen05).
bool pair_tail_split(uint64_t tile_n, uint64_t tiles, uint64_t pairs) {
  const uint64_t rest = tiles % pairs;
  return tile_n == 256 && rest > 0 && 2 * rest <= pairs;
}

// cluster_try: which cluster candidate of a K-split plan to take (-1: none, plan stream-K).
// ksplit: the K-split forms of the few-row plan (a cluster per tile, or stream-K) for a problem
// that is NOT swapped: few tiles of C against a long K (512 x 512 x 65536 has 8 tiles for 148 SMs).
// kparts > 1 (CTA-pair plans only): K planes -- K cut into that many parts at most, one work item
// per (tile, part), the partial tiles written as fp32 planes into the workspace and folded into C
// by a second launch (kplanes_sum_kernel).
void plan_tcgen05(frisk_gemm_plan* pl, bool swap, bool pair, int cluster_try = 0, bool ksplit = false,
                  int kparts = 0, int pair_cluster = 0) {
  const bool split = swap || ksplit;
  const bool planes = pair && !split && kparts > 1 && !pl->kd.row_reduce && !pl->tf32;
  // K split over the pairs of a cluster (gemm_tcgen05_pair_ksplit.cuh): 256 x 128 tiles
  const bool pcl = pair && !split && !planes && pair_cluster > 1 && !pl->kd.row_reduce && !pl->tf32;
  pl->pair_cluster = pcl ? pair_cluster : 0;
  const frisk_gemm_desc& d = pl->kd;
  frisk::GemmParams& g = pl->gp;
  memset(&g, 0, sizeof g);
  pl->plan_error = 0;
  const uint32_t es = elem_size(d.a_type);
  const uint32_t bk = 128u / es;
  bool a_mn, b_mn;  // majors of the kernel's a-role / b-role operands
  uint32_t cluster_mi = 1, cluster_k = 1;
  bool use_cluster = false;
  int64_t rows, cols;
  if (!swap) {
    a_mn = d.transA != 0;  // A stored K x M
    b_mn = d.transB == 0;  // B stored K x N
    rows = d.M;
    cols = d.N;
    g.mi = (ksplit && rows > 128) ? 2 : 1;
    uint32_t tn = d.tile_n ? (uint32_t)d.tile_n : (cols > 128 ? 256u : (cols > 64 ? 128u : 64u));
    if (pair && tn < 128) tn = 128;
    // 256-wide tiles that fill at most half of the pairs would run as half-width items anyway
    // (pair_tail_split); planned as 128-wide tiles the same items get stages of 24 instead of
    // 32 KiB, eight of them instead of six, and it is bytes in flight that such an operand-streaming
    // shape waits for (256 x 8192 x 8192: 39.3 -> 35.5 us, 256 x 4096 x 4096: 21.6 -> 18.8 us,
    // 8192 x 256 x 8192: 40.1 -> 37.1 us).
    if (pcl) tn = 128;
    if (pair && !planes && !pcl && !d.tile_n && tn == 256 &&
        2 * ((rows + 255) / 256) * ((cols + 255) / 256) <= (int64_t)std::max(1, pl->sm_count / 2))
      tn = 128;
    g.tile_n = tn;
  } else {
    // D = C^T: rows run over N (the weights), columns over M (the few activations rows)
    a_mn = d.transB == 0;  // B stored K x N: N contiguous
    b_mn = false;          // A stored M x K (transA == 0 is a precondition of this plan)
    rows = d.N;
    cols = d.M;
    g.mi = rows > 128 ? 2 : 1;
    g.tile_n = (uint32_t)((cols + 15) / 16 * 16);
  }
  if (split) {
    // Split mode 3 (a cluster per tile, a K slice per CTA, partials summed through distributed
    // shared memory) needs tiles x cluster size CTAs to cover most of the SMs; otherwise the
    // stream-K plan (mode 2) spreads the work evenly over all of them.
    // Candidates: 256- or 128-row tiles with the largest power-of-two cluster that keeps the grid
    // within the SMs, most CTAs first, then the larger tile (fewer, larger TMA boxes).
    // `cluster_try` skips the candidates the device could not place.
    const uint32_t kbs = (uint32_t)((d.K + bk - 1) / bk);
    // percent of the SMs a cluster plan has to use: measured, 64 CTAs in clusters still beat
    // stream-K over all SMs (16x2048x2048: 10.4 against 15.5 us; 32x2048x8192: 18.7 against 25.7)
    uint32_t min_cover = 40;
#ifdef FRISK_B200_MEASURE
    if (const char* e = getenv("FRISK_B200_MIN_COVER")) min_cover = (uint32_t)atoi(e);
#endif
    struct Cand {
      uint32_t ctas, mi, s;
    } cand[8];
    int n_cand = 0;
    for (uint32_t mi = (rows > 128 ? 2u : 1u); mi >= 1; --mi) {
      // tiles of the plan (the swapped plan has one tile column: all of M fits its tile width)
      const uint32_t t = (uint32_t)((rows + 128 * mi - 1) / (128 * mi)) *
                         (uint32_t)((cols + g.tile_n - 1) / g.tile_n);
      // the pushed-partials region and at least four pipeline stages have to fit beside each
      // other, or the region on top of four stages (red_overlay)
      const size_t stage = (size_t)(128 * mi + g.tile_n) * 128u;
      const size_t red = (size_t)128 * mi * g.tile_n * sizeof(float);
      if (1024 + 4 * stage > kMaxDynSmem) continue;
      if (red + 1024 + 4 * stage > kMaxDynSmem && red > 4 * stage) continue;
      for (uint32_t s = 8; s >= 2; s >>= 1) {
        if (s > kbs || (uint64_t)t * s > (uint64_t)pl->sm_count) continue;
        if (t * s * 100u >= (uint32_t)pl->sm_count * min_cover) cand[n_cand++] = Cand{t * s, mi, s};
      }
    }
    std::sort(cand, cand + n_cand, [](const Cand& x, const Cand& y) {
      return x.ctas != y.ctas ? x.ctas > y.ctas : x.mi > y.mi;
    });
    use_cluster = cluster_try >= 0 && cluster_try < n_cand && d.num_ctas == 0;
    if (use_cluster) {
      cluster_mi = cand[cluster_try].mi;
      cluster_k = cand[cluster_try].s;
    }
#ifdef FRISK_B200_MEASURE
    if (const char* e = getenv("FRISK_B200_SKINNY_CLUSTER")) {
      const int t = cluster_try + atoi(e);   // skip that many more candidates; negative: none
      use_cluster = atoi(e) >= 0 && t < n_cand && d.num_ctas == 0;
      if (use_cluster) {
        cluster_mi = cand[t].mi;
        cluster_k = cand[t].s;
      }
    }
#endif
    if (use_cluster) g.mi = cluster_mi;
  }
  g.bk_elems = bk;
  g.k_steps = 4;
  // a CTA of a pair stages its own 128 rows of A and half of the tile's B columns
  if (fill_operand(g.a, pl->lay_a, a_mn, 128u * g.mi, es, bk) ||
      fill_operand(g.b, pl->lay_b, b_mn, pair ? g.tile_n / 2 : g.tile_n, es, bk)) {
    pl->plan_error = FRISK_ERR_UNSUPPORTED;
    return;
  }
  if (pair && !b_mn && g.b.num_boxes == 1 && g.tile_n == 256) {
    // two boxes of 64 rows instead of one of 128 (same bytes in shared memory): a half-width item
    // of the last wave loads just the first
    g.b.num_boxes = 2;
    g.b.box_mn /= 2;
    g.b.box_bytes /= 2;
  }
  g.stage_bytes = g.a.stage_bytes + g.b.stage_bytes;
  // split mode 3 keeps one fp32 tile behind the stage buffers: the region the cluster's partials
  // are pushed into
  size_t red_bytes = (split && use_cluster) ? (size_t)128 * g.mi * g.tile_n * sizeof(float) : 0;
  // The region may instead lie ON the stage buffers (the kernel then holds the pushes back until
  // every CTA of the cluster has finished its main loop): taken when that buys at least a quarter
  // more pipeline stages -- measured, bf16 N = K = 8192: the time of a few-row plan follows the
  // weight bytes it keeps in flight (16 rows: 47 / 30 / 25.5 / 24.5 us at 64 / 96 / 128 / 160 KiB
  // per CTA), and from 64 rows on the region takes a third of the shared memory or more.
  bool red_overlay = false;
  if (red_bytes) {
    const size_t room = kMaxDynSmem - 1024;
    size_t st_sep = red_bytes < room ? (room - red_bytes) / g.stage_bytes : 0;
    size_t st_ovl = room / g.stage_bytes;
    st_sep = std::min<size_t>(st_sep, frisk::kMaxStages);
    st_ovl = std::min<size_t>(st_ovl, frisk::kMaxStages);
    if (d.stages > 0) {
      st_sep = std::min<size_t>(st_sep, (size_t)d.stages);
      st_ovl = std::min<size_t>(st_ovl, (size_t)d.stages);
    }
    red_overlay = red_bytes <= st_ovl * g.stage_bytes && (st_sep < 2 || 4 * st_ovl >= 5 * st_sep);
#ifdef FRISK_B200_MEASURE
    if (const char* e = getenv("FRISK_B200_RED_OVERLAY"))
      red_overlay = atoi(e) != 0 && red_bytes <= st_ovl * g.stage_bytes;
#endif
    if (red_overlay) red_bytes = 0;
  }
  g.red_overlay = red_overlay ? 1u : 0u;
  // Whole-tile plans stage the rows of C through 16 KiB of shared memory behind the pipeline
  // stages and store them as 128-byte pieces (measured on bf16 8192^3 and e4m3 8192^3: five, six
  // or seven stages of 32 KiB run within 1 % of each other, so the stage this costs the CTA-pair
  // kernel is free).  desc.epilogue = 1 stores per thread instead.
  // The area is reserved either way: the element-wise path of a C without 16-byte alignment goes
  // through it too.
  // desc.epilogue = 4 on a CTA-pair plan: TMA tensor stores out of two staging buffers per warp
  // (needs rows of C that start on 16-byte boundaries, like every tensor map).
  // Taken by default when K is short (at most 32 k-blocks): the epilogue of a tile then takes
  // longer than its main loop, and the tensor stores need a fraction of the instructions
  // (measured, bf16 8192 x 8192 x K: K = 256 58.6 -> 41.4 us, K = 512 65.3 -> 54.3 us, equal from
  // K = 1024 on; cuBLAS: 41.2 and 58.5 us).
  // ... and when every pair has a single tile, whose epilogue nothing hides (1024 x 1024 x 4096
  // 18.5 -> 18.1 us, 2048 x 2048 x 4096 29.5 -> 27.5 us, 2304 x 2048 x 8192 53.2 -> 51.9 us).
  const bool short_k = (d.K + bk - 1) / bk <= 32;
  const bool one_wave = pair && 2 * ((rows + 255) / 256) * ((cols + g.tile_n - 1) / g.tile_n) <=
                                    (int64_t)(d.num_ctas > 1 ? std::min(d.num_ctas, pl->sm_count) : pl->sm_count);
  const bool want_tma = d.epilogue == 4 || (d.epilogue == 0 && (short_k || one_wave));
  const bool epi_tma = pair && !planes && !pcl && !pl->tf32 && want_tma &&
                       (d.ldc * (int64_t)elem_size(d.c_type)) % 16 == 0;
  const size_t epi_bytes = (split || pcl) ? 0 : (epi_tma ? 2 : 1) * frisk::kEpiStageBytes;
  // (the other pairs' images of the rows a CTA owns: [pair][row of the share][tile_n + 4] fp32)
  if (pcl) red_bytes = ((size_t)(pair_cluster - 1) * (128 / pair_cluster) * (g.tile_n + 4) * sizeof(float) + 1023) / 1024 * 1024;
  g.epi_staged = split ? 0u : epi_tma ? 3u : planes ? 1u : d.epilogue == 1 ? 0u : d.epilogue == 3 ? 2u : 1u;
  // stages * stage_bytes + 1024 (alignment slack) + red_bytes + epi_bytes stays within kMaxDynSmem
  uint32_t stages = (uint32_t)((kMaxDynSmem - 1024 - red_bytes - epi_bytes) / g.stage_bytes);
  stages = std::min<uint32_t>(stages, frisk::kMaxStages);
  if (d.stages > 0) stages = std::min<uint32_t>(stages, (uint32_t)d.stages);
  // at least two: a stage is released only after the first MMA of the NEXT k-block was issued,
  // so with a single stage the producer and the MMA warp would wait for each other
  g.stages = std::max<uint32_t>(stages, 2);
  g.acc_bufs = (2 * g.mi * g.tile_n <= 512) ? 2 : 1;
  g.tmem_cols = next_pow2_cols(g.acc_bufs * g.mi * g.tile_n);
  g.idesc = make_idesc(d.a_type, a_mn, b_mn, pair ? 256u : 128u, g.tile_n);
  g.kind_f8 = is_fp8(d.a_type);
  g.rows = (uint32_t)rows;
  g.cols = (uint32_t)cols;
  const uint32_t tile_rows = pair ? 256u : 128u * g.mi;
  g.tiles_r = (uint32_t)((rows + tile_rows - 1) / tile_rows);
  g.tiles_c = (uint32_t)((cols + g.tile_n - 1) / g.tile_n);
  g.num_kb = (uint32_t)((d.K + bk - 1) / bk);
  // tile rows walked together: 2048 rows of A either way.  Measured on bf16 8192^3 with the pair
  // kernel (DRAM bytes read per launch): bands of 4 / 6 / 8 / 10 / 12 / 16 tile rows give
  // 1.58 / 1.26 / 1.07 / 1.15 / 1.11 / 1.21 GB
  g.group_r = d.band_tiles > 0 ? (uint32_t)d.band_tiles : (pair ? 8u : 16u);
  g.group_c = (pair && d.panel_tiles > 0) ? (uint32_t)d.panel_tiles : 0u;
  g.l2_hints = pair ? (uint32_t)d.l2_hints : 0u;
  g.split_mode = split ? 1 : 0;
  // a split plan has one or two work items per CTA, so the wake-up delay of a sleeping epilogue
  // warp is paid at the end of the kernel; a whole-tile plan hides it behind the next tile
  g.epilogue_backoff_ns = (split || planes || pcl) ? 0u : frisk::kEpilogueBackoffNs;
#ifdef FRISK_B200_MEASURE
  if (const char* e = getenv("FRISK_B200_EPI_BACKOFF")) g.epilogue_backoff_ns = (uint32_t)atoi(e);
#endif
  g.transposed_out = swap ? 1 : 0;
  g.clear_accum = d.clear_accum ? 1 : 0;
  g.c_type = d.c_type;
  g.ldc = d.ldc;
  g.ws_ld = d.N;
  size_t planes_bytes = 0;
  if (planes) {
    // the GEMM launch writes fp32 partial tiles, whole, without scales, at a pitch that keeps
    // every row of every plane on a 16-byte boundary
    g.kb_per = (g.num_kb + (uint32_t)kparts - 1) / (uint32_t)kparts;
    g.k_parts = (g.num_kb + g.kb_per - 1) / g.kb_per;   // no empty part
    const int64_t ldp = (d.N + 3) / 4 * 4;
    g.plane_elems = (uint64_t)d.M * (uint64_t)ldp;
    g.c_type = FRISK_DT_F32;
    g.ldc = ldp;
    g.clear_accum = 1;
    planes_bytes = ((size_t)g.k_parts * g.plane_elems * sizeof(float) + 255) / 256 * 256;
  }

  const uint64_t tiles = (uint64_t)g.tiles_r * g.tiles_c;
  const uint64_t units = split ? tiles * g.num_kb : tiles;
  uint32_t ctas = (uint32_t)std::min<uint64_t>(units, (uint64_t)pl->sm_count);
  if (d.num_ctas > 0) ctas = (uint32_t)std::min<uint64_t>(units, (uint64_t)d.num_ctas);
  g.n_items = g.narrow_from = (uint32_t)(planes ? tiles * g.k_parts : tiles);
  if (pcl) {
    g.cluster_k = (uint32_t)pair_cluster;
    g.kb_per = (g.num_kb + g.cluster_k - 1) / g.cluster_k;
    if ((g.cluster_k - 1) * g.kb_per >= g.num_kb) pl->plan_error = FRISK_ERR_UNSUPPORTED;   // an empty part
    ctas = (uint32_t)tiles * 2u * g.cluster_k;
  } else if (pair) {  // one cluster of two CTAs per tile in flight
    uint64_t slots = (uint64_t)pl->sm_count / 2;
    if (d.num_ctas > 1) slots = std::min<uint64_t>(slots, (uint64_t)d.num_ctas / 2);
    slots = std::max<uint64_t>(slots, 1);
    // Tiles that fill the last wave of pairs at most half are cut into two half-width items each:
    // the wave then takes about 0.56 of a whole-tile wave instead of a full one.
    const uint64_t rest = tiles % slots;
    if (!planes && pair_tail_split(g.tile_n, tiles, slots)) {
      g.narrow_from = (uint32_t)(tiles - rest);
      g.n_items = (uint32_t)(tiles + rest);
      g.idesc_narrow = make_idesc(d.a_type, a_mn, b_mn, 256u, g.tile_n / 2);
    }
    const uint64_t pairs = std::min<uint64_t>((uint64_t)g.n_items, slots);
    ctas = (uint32_t)(2 * pairs);
  }
  pl->dyn_smem = (size_t)g.stages * g.stage_bytes + 1024 + red_bytes + epi_bytes;
  pl->ws_bytes = planes_bytes;
  pl->rr_partial_bytes = 0;
  if (!split && d.row_reduce) {
    g.rr_kind = (uint32_t)d.row_reduce;
    pl->rr_partial_bytes = ((size_t)2 * g.tiles_c * (size_t)rows * sizeof(float) + 15) / 16 * 16;
    pl->ws_bytes = pl->rr_partial_bytes;
  }
  if (split && use_cluster) {
    g.split_mode = 3;
    g.cluster_k = cluster_k;
    ctas = (uint32_t)tiles * cluster_k;
  } else if (split) {
    // Split mode 2: every CTA writes the partial tiles of its unit range into private slots; the
    // workspace is [ctas * max_items slots of tile_rows x tile_n fp32][one arrival counter per tile].
    g.split_mode = 2;
    // the vector reduction sums at most kMaxContrib partials per tile: a tile's k-blocks spread
    // over ctas / tiles CTAs plus one at each end
    if (d.num_ctas == 0 && tiles * (frisk::kMaxContrib - 2) < ctas)
      ctas = (uint32_t)(tiles * (frisk::kMaxContrib - 2));
    // Tiles enough for five eighths of the SMs or more: whole tiles, the same number for every CTA,
    // so that nothing goes through the slots (measured, bf16, few rows against a wide B: 125 tiles
    // 73.0 -> 54.0 us, 112 tiles 85.6 -> 77.9, 96 tiles 54.5 -> 45.8, 196 tiles 52.0 -> 49.6;
    // 80 tiles 41.1 -> 43.3, which is why the rule stops there).
    if (d.num_ctas == 0 && tiles * 8 >= (uint64_t)pl->sm_count * 5) {
      const uint64_t per = (tiles + (uint64_t)pl->sm_count - 1) / (uint64_t)pl->sm_count;
      ctas = (uint32_t)((tiles + per - 1) / per);
    }
    const uint64_t per_cta = (units + ctas - 1) / ctas;
    g.max_items = (uint32_t)((per_cta + g.num_kb - 1) / g.num_kb + 1);
    const size_t tile_elems = (size_t)128 * g.mi * g.tile_n;
    pl->slot_bytes = (size_t)ctas * g.max_items * tile_elems * sizeof(float);
    pl->ws_bytes = pl->slot_bytes + (size_t)tiles * sizeof(uint32_t);
  }

  frisk_gemm_plan_info& in = pl->info;
  in.kernel = swap ? FRISK_KERNEL_SKINNY : (pair ? FRISK_KERNEL_TCGEN05_PAIR : FRISK_KERNEL_TCGEN05);
  in.tile_m = swap ? (int)g.tile_n : (int)tile_rows;
  in.tile_n = swap ? 128 * (int)g.mi : (int)g.tile_n;
  in.tile_k = (int)bk;
  in.stages = (int)g.stages;
  in.num_ctas = (int)ctas;
  in.swap_ab = swap;
  in.split_k = split || planes || pcl;
  in.smem_bytes = (int)pl->dyn_smem;
  in.launches = ((!split && d.row_reduce) || planes) ? 2 : 1;   // the fold's finalize launch / the planes' sum
  in.swizzle_a = pl->lay_a.swizzle_bytes;
  in.swizzle_b = pl->lay_b.swizzle_bytes;
  // the clusters must all be resident at once for the plan to make sense; if this device cannot
  // place them, plan again without
  if (split && use_cluster && pl->have_device && !skinny_clusters_fit(pl))
    plan_tcgen05(pl, swap, pair, cluster_try + 1, ksplit);
}

constexpr int kMaxDevices = 64;

// Opts a kernel function into the large dynamic shared memory, once per function and device.
// The limit belongs to the kernel function, not to a plan: every plan asks for the same value
// (the most any plan uses), so plans with different pipeline depths do not lower it under one
// another, and a plan that lives on the caller's stack does not pay for the call every time.
// `Tag` names the kernel function: instantiations of one kernel template share a function TYPE, so
// the flags cannot hang on the type of `kern`.
template <typename Tag, typename Kern>
int ensure_dyn_smem(Kern kern, int device) {
  static bool done[kMaxDevices] = {};  // one array per Tag
  const bool tracked = device >= 0 && device < kMaxDevices;
  if (tracked && __atomic_load_n(&done[device], __ATOMIC_ACQUIRE)) return FRISK_OK;
  FRISK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  (int)kMaxDynSmem));
  if (tracked) __atomic_store_n(&done[device], true, __ATOMIC_RELEASE);
  return FRISK_OK;
}
template <typename TC, bool kSplit, bool kTf32 = false> struct OneCtaKernelTag {};
template <typename TC, bool kTf32 = false> struct PairKernelTag {};

template <typename TC, bool kSplit, bool kTf32 = false>
int launch_tcgen05_ts(frisk_gemm_plan* pl, const frisk::GemmParams& g, cudaStream_t st) {
  auto kern = frisk::gemm_tcgen05_kernel<TC, kSplit, kTf32>;
  if (int rc = ensure_dyn_smem<OneCtaKernelTag<TC, kSplit, kTf32>>(kern, pl->device)) return rc;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3((unsigned)pl->info.num_ctas, 1, 1);
  cfg.blockDim = dim3(frisk::kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = kLaunchDynSmem;
  cfg.stream = st;
  // the kernel's set-up may start while the previous kernel of the stream drains; it waits
  // (griddepcontrol.wait) before it touches global memory
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (kSplit && g.split_mode == 3 && g.cluster_k > 1) {
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = g.cluster_k;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.numAttrs = 2;
  }
  FRISK_CUDA(cudaLaunchKernelEx(&cfg, kern, pl->tmap_a, pl->tmap_b, g));
  return FRISK_OK;
}

// How many clusters of the plan's size the device can hold at once, for one C type.
template <typename TC>
int max_active_clusters_t(frisk_gemm_plan* pl, int* out) {
  auto kern = frisk::gemm_tcgen05_kernel<TC, true>;
  if (int rc = ensure_dyn_smem<OneCtaKernelTag<TC, true>>(kern, pl->device)) return rc;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3((unsigned)pl->info.num_ctas, 1, 1);
  cfg.blockDim = dim3(frisk::kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = kLaunchDynSmem;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = pl->gp.cluster_k;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  FRISK_CUDA(cudaOccupancyMaxActiveClusters(out, kern, &cfg));
  return FRISK_OK;
}

bool skinny_clusters_fit(frisk_gemm_plan* pl) {
  int n = 0, rc;
  switch (pl->d.c_type) {
    case FRISK_DT_F32: rc = max_active_clusters_t<float>(pl, &n); break;
    case FRISK_DT_F16: rc = max_active_clusters_t<__half>(pl, &n); break;
    case FRISK_DT_BF16: rc = max_active_clusters_t<__nv_bfloat16>(pl, &n); break;
    default: return false;
  }
  if (rc != FRISK_OK) {
    cudaGetLastError();
    return false;
  }
  return (uint32_t)n * pl->gp.cluster_k >= (uint32_t)pl->info.num_ctas;
}

template <typename TC>
int launch_tcgen05_t(frisk_gemm_plan* pl, const frisk::GemmParams& g, cudaStream_t st) {
  return g.split_mode ? launch_tcgen05_ts<TC, true>(pl, g, st) : launch_tcgen05_ts<TC, false>(pl, g, st);
}

template <typename TC, bool kTf32 = false>
int launch_pair_tf(frisk_gemm_plan* pl, const frisk::GemmParams& g, cudaStream_t st) {
  auto kern = frisk::gemm_tcgen05_pair_kernel<TC, kTf32>;
  if (int rc = ensure_dyn_smem<PairKernelTag<TC, kTf32>>(kern, pl->device)) return rc;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3((unsigned)pl->info.num_ctas, 1, 1);
  cfg.blockDim = dim3(frisk::kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = kLaunchDynSmem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  FRISK_CUDA(cudaLaunchKernelEx(&cfg, kern, pl->tmap_a, pl->tmap_b, g, pl->c_maps));
  return FRISK_OK;
}

template <typename TC>
int launch_pair_t(frisk_gemm_plan* pl, const frisk::GemmParams& g, cudaStream_t st) {
  return launch_pair_tf<TC>(pl, g, st);
}

// The CTA-pair kernel with K split over the pairs of a cluster: one cluster of 2 x cluster_k CTAs
// per tile.  `occupancy`: ask how many such clusters the device holds at once instead of launching.
template <typename TC> struct PairKsplitKernelTag {};
template <typename TC>
int launch_pair_ksplit_t(frisk_gemm_plan* pl, const frisk::GemmParams& g, cudaStream_t st,
                         int* occupancy = nullptr) {
  auto kern = frisk::gemm_tcgen05_pair_ksplit_kernel<TC>;
  if (int rc = ensure_dyn_smem<PairKsplitKernelTag<TC>>(kern, pl->device)) return rc;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3((unsigned)pl->info.num_ctas, 1, 1);
  cfg.blockDim = dim3(frisk::kGemmThreads, 1, 1);
  cfg.dynamicSmemBytes = kLaunchDynSmem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2u * g.cluster_k;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  if (occupancy) {
    cfg.numAttrs = 1;
    FRISK_CUDA(cudaOccupancyMaxActiveClusters(occupancy, kern, &cfg));
    return FRISK_OK;
  }
  cfg.numAttrs = 2;
  FRISK_CUDA(cudaLaunchKernelEx(&cfg, kern, pl->tmap_a, pl->tmap_b, g));
  return FRISK_OK;
}

int launch_pair_ksplit(frisk_gemm_plan* pl, const frisk::GemmParams& g, cudaStream_t st, int* occupancy = nullptr) {
  switch (pl->d.c_type) {
    case FRISK_DT_F32: return launch_pair_ksplit_t<float>(pl, g, st, occupancy);
    case FRISK_DT_F16: return launch_pair_ksplit_t<__half>(pl, g, st, occupancy);
    case FRISK_DT_BF16: return launch_pair_ksplit_t<__nv_bfloat16>(pl, g, st, occupancy);
    default: return FRISK_ERR_UNSUPPORTED;
  }
}

// Whether the device can hold all of the plan's clusters at once (they wait for one another).
bool pair_clusters_fit(frisk_gemm_plan* pl) {
  int n = 0;
  if (launch_pair_ksplit(pl, pl->gp, nullptr, &n) != FRISK_OK) {
    cudaGetLastError();
    return false;
  }
  return (int64_t)n * 2 * pl->gp.cluster_k >= (int64_t)pl->info.num_ctas;
}

// The second launch of a plan with a fused row reduce: folds the per-tile results of every row.
template <typename TC>
int launch_row_fold_t(const frisk_gemm_plan* pl, const frisk::GemmParams& g, void* dst, cudaStream_t st) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  cfg.gridDim = dim3((g.rows + 255u) / 256u, 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  FRISK_CUDA(cudaLaunchKernelEx(&cfg, frisk::row_fold_finalize_kernel<TC>, (const float*)g.rr_partials,
                                reinterpret_cast<TC*>(dst), g.rows, 2u * g.tiles_c, g.rr_kind,
                                (uint32_t)(pl->d.row_reduce_clear ? 1 : 0)));
  return FRISK_OK;
}

// The second launch of a K-planes plan: sums the fp32 planes into the caller's C.
template <typename TC>
int launch_kplanes_sum_t(const frisk_gemm_plan* pl, const frisk::GemmParams& g, const float* planes,
                         void* C, const float* sa, const float* sb, cudaStream_t st) {
  const frisk_gemm_desc& d = pl->d;
  const int64_t work = d.M * ((d.N + 3) / 4);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof cfg);
  const int64_t blocks = std::min<int64_t>((work + 255) / 256, 8 * (int64_t)pl->sm_count);
  cfg.gridDim = dim3((unsigned)std::max<int64_t>(1, blocks), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.stream = st;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  const int vec_ok = ((uintptr_t)C % (4 * sizeof(TC)) == 0) && (d.ldc % 4 == 0);
  FRISK_CUDA(cudaLaunchKernelEx(&cfg, frisk::kplanes_sum_kernel<TC>, planes, (uint64_t)g.plane_elems,
                                (uint32_t)g.k_parts, (int64_t)g.ldc, reinterpret_cast<TC*>(C), (int64_t)d.ldc,
                                (int64_t)d.M, (int64_t)d.N, sa, sb, (int)(d.clear_accum ? 1 : 0), vec_ok));
  return FRISK_OK;
}

template <typename TC>
int launch_finalize_t(const frisk_gemm_plan* pl, float* ws, void* C, const float* sa,
                      const float* sb, cudaStream_t st) {
  const frisk_gemm_desc& d = pl->d;
  const int64_t work = d.M * ((d.N + 3) / 4);
  const int threads = 256;
  const int blocks = (int)std::min<int64_t>((work + threads - 1) / threads, 4 * (int64_t)pl->sm_count);
  frisk::splitk_finalize_kernel<TC><<<blocks, threads, 0, st>>>(
      ws, d.N, reinterpret_cast<TC*>(C), d.ldc, d.M, d.N, sa, sb, d.clear_accum);
  FRISK_CUDA(cudaGetLastError());
  return FRISK_OK;
}

// Copies `rows` rows of `row_bytes` bytes from pitch `src_pitch` to pitch `dst_pitch` (a multiple
// of 16, like dst itself), zero behind the end of a row.  The source may start anywhere: it is
// read in 2-byte or 1-byte units (`unit`), the destination written 16 bytes at a time.
__global__ void __launch_bounds__(256) repack_rows_kernel(const unsigned char* __restrict__ src,
                                                          unsigned char* __restrict__ dst, int64_t rows,
                                                          int64_t row_bytes, int64_t src_pitch,
                                                          int64_t dst_pitch, int unit) {
  const int64_t chunks = dst_pitch >> 4;
  const int64_t total = rows * chunks;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t r = i / chunks, c = (i - r * chunks) << 4;
    const unsigned char* s = src + r * src_pitch + c;
    union {
      uint4 v;
      unsigned short h[8];
      unsigned char b[16];
    } u;
    u.v = make_uint4(0, 0, 0, 0);
    const int64_t left = row_bytes - c;
    if (left >= 16 && (reinterpret_cast<uintptr_t>(s) & 15) == 0) {
      u.v = *reinterpret_cast<const uint4*>(s);
    } else if (unit == 2) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        if (2 * j < left) u.h[j] = *reinterpret_cast<const unsigned short*>(s + 2 * j);
    } else {
#pragma unroll
      for (int j = 0; j < 16; ++j)
        if (j < left) u.b[j] = s[j];
    }
    *reinterpret_cast<uint4*>(dst + r * dst_pitch + c) = u.v;
  }
}

int launch_repack(const void* src, void* dst, int64_t rows, int64_t cols, int64_t ld_src, int64_t ld_dst,
                  int es, int sm_count, cudaStream_t st) {
  const int64_t work = rows * (ld_dst * es / 16);
  const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((work + 255) / 256, 8 * (int64_t)sm_count));
  repack_rows_kernel<<<blocks, 256, 0, st>>>(static_cast<const unsigned char*>(src), static_cast<unsigned char*>(dst),
                                             rows, cols * es, ld_src * es, ld_dst * es, es);
  FRISK_CUDA(cudaGetLastError());
  return FRISK_OK;
}

// One operand of a 3xTF32 plan (`mn` x `k` logically) into its two K segments of `seg` columns
// (k rounded up to a k-block), K innermost.
// `k_along_rows`: the source is stored [k, mn] (mn contiguous) and is transposed on the way.
int launch_tf32_split(const float* src, float* dst, int64_t mn, int64_t k, int64_t seg, int64_t ld_src,
                      int64_t ld_dst, bool k_along_rows, uint32_t lo_mask, int sm_count,
                      cudaStream_t st) {
  if (k_along_rows) {
    const dim3 grid((unsigned)((mn + 31) / 32), (unsigned)(seg / 32));
    if (grid.y > 65535) return FRISK_ERR_UNSUPPORTED;
    frisk::tf32_split_transpose_kernel<<<grid, dim3(32, 8), 0, st>>>(src, dst, k, mn, seg, ld_src, ld_dst, lo_mask);
  } else {
    const int64_t work = mn * (seg / 4);
    const int blocks = (int)std::max<int64_t>(1, std::min<int64_t>((work + 255) / 256, 8 * (int64_t)sm_count));
    frisk::tf32_split_kernel<<<blocks, 256, 0, st>>>(src, dst, mn, k, seg, ld_src, ld_dst, lo_mask);
  }
  FRISK_CUDA(cudaGetLastError());
  return FRISK_OK;
}

template <typename TIn, int TM>
int launch_simt_tm(const frisk_gemm_desc& d, const frisk::SimtParams& sp, cudaStream_t st) {
  dim3 grid((unsigned)((d.N + frisk::kSimtTile - 1) / frisk::kSimtTile), (unsigned)((d.M + TM - 1) / TM));
  switch (d.c_type) {
    case FRISK_DT_F32: frisk::gemm_simt_kernel<TIn, float, TM><<<grid, TM * 4, 0, st>>>(sp); break;
    case FRISK_DT_F16: frisk::gemm_simt_kernel<TIn, __half, TM><<<grid, TM * 4, 0, st>>>(sp); break;
    case FRISK_DT_BF16: frisk::gemm_simt_kernel<TIn, __nv_bfloat16, TM><<<grid, TM * 4, 0, st>>>(sp); break;
    default: return FRISK_ERR_UNSUPPORTED;
  }
  FRISK_CUDA(cudaGetLastError());
  return FRISK_OK;
}

// fp32 problems the pipelined CUDA-core kernel takes (gemm_simt.cuh): the tile of the generic
// kernel's 32-row form without edges, rows of A and B that cp.async can read 16 bytes at a time.
bool simt_f32_pipelined_ok(const frisk_gemm_desc& d, const frisk::SimtParams& sp) {
  if (d.a_type != FRISK_DT_F32 || d.transA || d.transB) return false;
  if (d.M % 32 || d.N % frisk::kSimtTile || d.K % frisk::kSimtPipeBK) return false;
  if (d.lda % 4 || d.ldb % 4 || (uintptr_t)sp.A % 16 || (uintptr_t)sp.B % 16) return false;
  // where the generic kernel would take 32-row tiles (launch_simt_in; plan_info reports that tile)
  const int64_t ctas64 = ((d.N + 63) / 64) * ((d.M + 63) / 64);
  return d.M > 32 && ctas64 < 148;
}

int launch_simt_f32_pipelined(const frisk_gemm_desc& d, const frisk::SimtParams& sp, cudaStream_t st) {
  const dim3 grid((unsigned)(d.N / frisk::kSimtTile), (unsigned)(d.M / 32));
  switch (d.c_type) {
    case FRISK_DT_F32: frisk::gemm_simt_f32_pipelined_kernel<float><<<grid, 128, 0, st>>>(sp); break;
    case FRISK_DT_F16: frisk::gemm_simt_f32_pipelined_kernel<__half><<<grid, 128, 0, st>>>(sp); break;
    case FRISK_DT_BF16: frisk::gemm_simt_f32_pipelined_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>(sp); break;
    default: return FRISK_ERR_UNSUPPORTED;
  }
  FRISK_CUDA(cudaGetLastError());
  return FRISK_OK;
}

template <typename TIn>
int launch_simt_in(const frisk_gemm_desc& d, const frisk::SimtParams& sp, cudaStream_t st) {
  // 32-row tiles when 64-row tiles would leave SMs idle (fp32 512^3: 64 CTAs for 148 SMs)
  const int64_t ctas64 = ((d.N + 63) / 64) * ((d.M + 63) / 64);
  if (d.M > 32 && ctas64 < 148) return launch_simt_tm<TIn, 32>(d, sp, st);
  return launch_simt_tm<TIn, 64>(d, sp, st);
}

int launch_simt(const frisk_gemm_desc& d, const void* A, const void* B, void* C, const float* sa,
                const float* sb, cudaStream_t st) {
  if ((d.M + 31) / 32 > 65535) return FRISK_ERR_UNSUPPORTED;  // grid.y limit
  frisk::SimtParams sp;
  sp.A = A; sp.B = B; sp.C = C;
  sp.scale_a = d.scale_mode ? sa : nullptr;
  sp.scale_b = d.scale_mode ? sb : nullptr;
  sp.M = d.M; sp.N = d.N; sp.K = d.K;
  sp.lda = d.lda; sp.ldb = d.ldb; sp.ldc = d.ldc;
  sp.transA = d.transA; sp.transB = d.transB; sp.clear_accum = d.clear_accum;
  if (simt_f32_pipelined_ok(d, sp)) return launch_simt_f32_pipelined(d, sp, st);
  switch (d.a_type) {
    case FRISK_DT_F32: return launch_simt_in<float>(d, sp, st);
    case FRISK_DT_F16: return launch_simt_in<__half>(d, sp, st);
    case FRISK_DT_BF16: return launch_simt_in<__nv_bfloat16>(d, sp, st);
    case FRISK_DT_E4M3: return launch_simt_in<frisk::e4m3_t>(d, sp, st);
    case FRISK_DT_E5M2: return launch_simt_in<frisk::e5m2_t>(d, sp, st);
    default: return FRISK_ERR_UNSUPPORTED;
  }
}

size_t a_bytes(const frisk_gemm_desc& d) {
  return (size_t)(d.transA ? d.K : d.M) * d.lda * elem_size(d.a_type);
}
size_t b_bytes(const frisk_gemm_desc& d) {
  return (size_t)(d.transB ? d.N : d.K) * d.ldb * elem_size(d.b_type);
}
size_t c_bytes(const frisk_gemm_desc& d) { return (size_t)d.M * d.ldc * elem_size(d.c_type); }

// Host -> device copies of the operands.  Only the elements of each stored row are read: a host
// buffer sized the BLAS way, (rows - 1) * ld + row length, ends before rows * ld.
int upload_rows(void* dst, const void* src, size_t pitch, size_t row_bytes, int64_t row0,
                int64_t rows, cudaStream_t st) {
  char* d = static_cast<char*>(dst) + (size_t)row0 * pitch;
  const char* s = static_cast<const char*>(src) + (size_t)row0 * pitch;
  if (pitch == row_bytes)
    FRISK_CUDA(cudaMemcpyAsync(d, s, (size_t)rows * pitch, cudaMemcpyHostToDevice, st));
  else
    FRISK_CUDA(cudaMemcpy2DAsync(d, pitch, s, pitch, row_bytes, (size_t)rows,
                                 cudaMemcpyHostToDevice, st));
  return FRISK_OK;
}
// stored rows [row0, row0 + rows) of A: rows of M (transA == 0) or of K
int upload_a(const frisk_gemm_desc& d, void* dst, const void* src, int64_t row0, int64_t rows,
             cudaStream_t st) {
  const size_t es = elem_size(d.a_type);
  return upload_rows(dst, src, (size_t)d.lda * es, (size_t)(d.transA ? d.M : d.K) * es, row0, rows, st);
}
int upload_b(const frisk_gemm_desc& d, void* dst, const void* src, cudaStream_t st) {
  const size_t es = elem_size(d.b_type);
  return upload_rows(dst, src, (size_t)d.ldb * es, (size_t)(d.transB ? d.K : d.N) * es, 0,
                     d.transB ? d.N : d.K, st);
}
int upload_c(const frisk_gemm_desc& d, void* dst, const void* src, int64_t row0, int64_t rows,
             cudaStream_t st) {
  const size_t es = elem_size(d.c_type);
  return upload_rows(dst, src, (size_t)d.ldc * es, (size_t)d.N * es, row0, rows, st);
}

}  // namespace

extern "C" {

int frisk_b200_gemm_plan_create(const frisk_gemm_desc* desc, frisk_gemm_plan** out) {
  if (!desc || !out) return FRISK_ERR_INVALID_ARGUMENT;
  *out = nullptr;
  frisk_gemm_desc d = *desc;
  if (d.M <= 0 || d.N <= 0 || d.K <= 0) return FRISK_ERR_INVALID_ARGUMENT;
  if (!elem_size(d.a_type) || !elem_size(d.b_type) || !elem_size(d.c_type))
    return FRISK_ERR_INVALID_ARGUMENT;
  if (is_fp8(d.c_type)) return FRISK_ERR_UNSUPPORTED;
  if (d.a_type != d.b_type) return FRISK_ERR_INVALID_ARGUMENT;  // ffi/ir.cpp:357-359
  if (d.scale_mode != FRISK_SCALE_NONE && d.scale_mode != FRISK_SCALE_ROW_COL)
    return FRISK_ERR_INVALID_ARGUMENT;
  d.transA = d.transA != 0;
  d.transB = d.transB != 0;
  if (d.lda == 0) d.lda = d.transA ? d.M : d.K;
  if (d.ldb == 0) d.ldb = d.transB ? d.K : d.N;
  if (d.ldc == 0) d.ldc = d.N;
  if (d.lda < (d.transA ? d.M : d.K) || d.ldb < (d.transB ? d.K : d.N) || d.ldc < d.N)
    return FRISK_ERR_INVALID_ARGUMENT;
  if (d.tile_n != 0 && d.tile_n != 64 && d.tile_n != 128 && d.tile_n != 256)
    return FRISK_ERR_INVALID_ARGUMENT;
  if (d.force_kernel < 0 || d.force_kernel > 5 || d.stages < 0 || d.num_ctas < 0 || d.band_tiles < 0)
    return FRISK_ERR_INVALID_ARGUMENT;
  if (d.epilogue < 0 || d.epilogue > 4 || d.row_reduce < 0 || d.row_reduce > 4 ||
      d.panel_tiles < 0 || d.l2_hints < 0 || d.l2_hints > 3 || d.k_split < -1 || d.k_split > 3)
    return FRISK_ERR_INVALID_ARGUMENT;
  d.row_reduce_clear = d.row_reduce_clear != 0;

  frisk_gemm_plan* pl = new (std::nothrow) frisk_gemm_plan();
  if (!pl) return FRISK_ERR_INVALID_ARGUMENT;
  pl->d = d;
  pl->kd = d;
  memset(&pl->info, 0, sizeof pl->info);
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) == cudaSuccess) {
      pl->device = dev;
      pl->sm_count = prop.multiProcessorCount;
      pl->have_device = prop.major == 10;
    }
  } else {
    cudaGetLastError();  // plans can be made (and inspected) on a machine without a GPU
  }

  // fp32 inputs: three tf32 products on the tensor cores when the problem is large enough
  if ((d.force_kernel == 1 + FRISK_KERNEL_TF32X3) ||
      (!d.force_kernel && tf32_eligible(d) && tf32_worthwhile(d))) {
    if (!tf32_eligible(d)) {
      delete pl;
      return d.a_type == FRISK_DT_F32 ? FRISK_ERR_MISALIGNED : FRISK_ERR_UNSUPPORTED;
    }
    frisk_gemm_desc& k = pl->kd;
    // A' = [A_lo | A_hi] is [M, 2 Ks] and B' = [B_hi | B_lo] is [N, 2 Ks], K innermost (kind::tf32
    // reads 32-bit operands K-inner only) whatever the order A and B are stored in, Ks = K rounded
    // up to a k-block of 32; the kernel walks 3 Ks of K (tf32_split.cuh)
    const int64_t ks = (d.K + 31) / 32 * 32;
    k.K = 3 * ks;
    k.transA = 0;
    k.transB = 1;
    k.lda = k.ldb = 2 * ks;
    k.force_kernel = 0;
    pl->tf32 = true;
    pl->tf32_a_bytes = ((size_t)d.M * k.lda * sizeof(float) + 255) / 256 * 256;
    pl->tf32_b_bytes = ((size_t)d.N * k.ldb * sizeof(float) + 255) / 256 * 256;
    pl->tf32_pair = d.M > 128 && d.N > 64 && d.tile_n != 64 && pl->sm_count >= 2;
    plan_tcgen05(pl, /*swap=*/false, pl->tf32_pair);
    if (pl->plan_error) {
      const int rc = pl->plan_error;
      delete pl;
      return rc;
    }
    pl->gp.seg_kb = (uint32_t)(ks / 32);
    pl->info.kernel = FRISK_KERNEL_TF32X3;
    pl->info.launches = 3;   // the split of A, the split of B, the GEMM
    pl->ws_bytes = pl->tf32_a_bytes + pl->tf32_b_bytes;
    *out = pl;
    return FRISK_OK;
  }
  // A row pitch of A or B that is not a multiple of 16 bytes rules out tensor maps on the caller's
  // buffers, not the tensor cores: the plan copies such an operand into the workspace at a padded
  // pitch before every run (one more launch each; the copy reads and writes the operand once,
  // against a CUDA-core kernel about 100 x slower on the whole problem).
  if (tcgen05_ineligible_reason(d) == FRISK_TC_PITCH && d.force_kernel != 1 + FRISK_KERNEL_SIMT) {
    const int64_t es = elem_size(d.a_type), q = 16 / es;
    frisk_gemm_desc& k = pl->kd;
    if ((d.lda * es) % 16) {
      k.lda = ((d.transA ? d.M : d.K) + q - 1) / q * q;
      pl->repack_a_bytes = ((size_t)(d.transA ? d.K : d.M) * k.lda * es + 255) / 256 * 256;
    }
    if ((d.ldb * es) % 16) {
      k.ldb = ((d.transB ? d.K : d.N) + q - 1) / q * q;
      pl->repack_b_bytes = ((size_t)(d.transB ? d.N : d.K) * k.ldb * es + 255) / 256 * 256;
    }
    d = k;   // the choices below are made for the repacked problem
  }
  const bool tc_ok = tcgen05_eligible(d);
  const bool skinny_ok = tc_ok && skinny_shape(d, pl->sm_count);
  const bool pair_ok = tc_ok && d.M > 128 && d.N > 64 && d.tile_n != 64 && pl->sm_count >= 2;
  int kind;
  if (d.force_kernel) {
    kind = d.force_kernel - 1;
    if ((kind == FRISK_KERNEL_TCGEN05 && !tc_ok) || (kind == FRISK_KERNEL_SKINNY && !skinny_ok) ||
        (kind == FRISK_KERNEL_TCGEN05_PAIR && !pair_ok)) {
      delete pl;
      return tc_ok ? FRISK_ERR_UNSUPPORTED : FRISK_ERR_MISALIGNED;
    }
  } else {
    // Two SMs on one 256-row tile (each stages half of B) run about 1.12x faster per tile than
    // two one-CTA tiles, so the pair kernel is taken unless its coarser tiles lose more than that
    // to the last, partly filled wave (desc.force_kernel overrides the estimate).
    bool use_pair = false;
    if (pair_ok) {
      const uint64_t tn = d.tile_n ? (uint64_t)d.tile_n : (d.N > 128 ? 256u : 128u);
      const uint64_t cols_t = ((uint64_t)d.N + tn - 1) / tn;
      const uint64_t one_tiles = (((uint64_t)d.M + 127) / 128) * cols_t;
      const uint64_t two_tiles = (((uint64_t)d.M + 255) / 256) * cols_t;
      const uint64_t sms = (uint64_t)pl->sm_count, pairs = sms / 2;
      const double one_cost = (double)((one_tiles + sms - 1) / sms);
      double two_waves = (double)((two_tiles + pairs - 1) / pairs);
      if (pair_tail_split(tn, two_tiles, pairs)) two_waves -= 0.44;  // a wave of half-width items
      const double two_cost = two_waves / 1.12;
      use_pair = two_cost < one_cost;
#ifdef FRISK_B200_MEASURE
      if (const char* want_pair = getenv("FRISK_B200_PAIR")) use_pair = want_pair[0] == '1';
#endif
    }
    kind = (skinny_ok && !d.row_reduce) ? FRISK_KERNEL_SKINNY
           : use_pair                    ? FRISK_KERNEL_TCGEN05_PAIR
           : tc_ok                       ? FRISK_KERNEL_TCGEN05
                                         : FRISK_KERNEL_SIMT;
  }
  // the row reduce lives in the whole-tile epilogue of the tensor-core kernels
  if (d.row_reduce && kind != FRISK_KERNEL_TCGEN05 && kind != FRISK_KERNEL_TCGEN05_PAIR) {
    delete pl;
    g_last_error = "a fused row reduce needs a whole-tile tensor-core plan (fp16 / bf16 / e4m3 "
                   "inputs with 16-byte row pitches)";
    return FRISK_ERR_UNSUPPORTED;
  }
  if (kind == FRISK_KERNEL_SIMT) {
    pl->info.kernel = FRISK_KERNEL_SIMT;
    pl->info.cuda_core_reason = d.force_kernel ? FRISK_TC_FORCED : tcgen05_ineligible_reason(d);
    // the same choice launch_simt_in makes: 32-row tiles when 64-row tiles would not fill the SMs
    const int64_t ctas64 = ((d.N + 63) / 64) * ((d.M + 63) / 64);
    const int tm = (d.M > 32 && ctas64 < 148) ? 32 : frisk::kSimtTile;
    pl->info.tile_m = tm;
    pl->info.tile_n = frisk::kSimtTile;
    pl->info.tile_k = frisk::kSimtBK;
    pl->info.stages = 1;
    pl->info.num_ctas = (int)(((d.M + tm - 1) / tm) * ((d.N + 63) / 64));
    pl->info.launches = 1;
  } else {
    plan_tcgen05(pl, kind == FRISK_KERNEL_SKINNY, kind == FRISK_KERNEL_TCGEN05_PAIR);
    // Between 65 and 128 rows the few-row plan pays only in its cluster form (128 x 8192 x 8192:
    // 35 us against 59 us for whole tiles on 32 SMs); where clusters do not apply (few tiles, or
    // more tiles than SMs) whole tiles are as good or better (128 x 28672 x 4096: 45 against 79 us).
    if (kind == FRISK_KERNEL_SKINNY && d.M > 64 && !d.force_kernel && pl->gp.split_mode != 3)
      plan_tcgen05(pl, /*swap=*/false, /*pair=*/false);
    // Few tiles of C against a long K: whole tiles would leave most SMs idle (512 x 512 x 65536:
    // 8 tiles; measured 227 us against 43 us for cuBLAS), so K is split over clusters or, where
    // no cluster shape fits, over all SMs (stream-K), as in the few-row plan but without the swap.
    // Considered when the whole-tile plan would use at most a quarter of the SMs and K has at least
    // 48 k-blocks, or at most half of them and K has at least 192 (8192 x 128 x 8192 on 64 SMs:
    // 34.1 us whole, 36.9 us split over 128; 1024 x 1024 x 16384 on 64: 62.7 whole, 44.5 split)
    // (1024^3 with 16 k-blocks: 15.4 us split against 10.1 us whole -- the fold of the partials
    // costs more than the idle SMs); taken when it puts more CTAs to work.
    const bool force_split = d.k_split == 1;
    const bool consider_split = d.k_split >= 0 && (d.k_split > 0 || 2 * pl->info.num_ctas <= pl->sm_count);
    if (!d.force_kernel && !d.row_reduce && !d.num_ctas && !d.tile_n &&
        (pl->info.kernel == FRISK_KERNEL_TCGEN05 || pl->info.kernel == FRISK_KERNEL_TCGEN05_PAIR) &&
        consider_split) {
      const uint64_t kbs = (uint64_t)((d.K + pl->info.tile_k - 1) / pl->info.tile_k);
      const uint64_t t128 = (uint64_t)((d.M + 127) / 128) * (uint64_t)((d.N + 63) / 64);
      const bool few = 4 * pl->info.num_ctas <= pl->sm_count;
      // K planes on the CTA-pair kernel: 256-row tiles, as many K parts as there are pairs for
      // (at least eight k-blocks each)
      const uint64_t tn256 = d.N > 128 ? 256 : 128;
      const uint64_t tiles256 = (uint64_t)((d.M + 255) / 256) * (((uint64_t)d.N + tn256 - 1) / tn256);
      const uint64_t kparts = std::min<uint64_t>((uint64_t)(pl->sm_count / 2) / tiles256, kbs / 8);
      const bool planes_ok = pair_ok && kparts >= 2;
      bool planes = planes_ok && d.k_split == 2;
      // K split over the pairs of a cluster (gemm_tcgen05_pair_ksplit.cuh): 256 x 128 tiles, at
      // least eight k-blocks per pair.  Taken where measured ahead, for K up to 128 k-blocks
      // (deeper: the forms below) and tiles that are not mostly padding:
      //   six to nine tiles, four pairs per cluster (bf16, before -> after (cuBLAS)):
      //     512 x 512 x 4096 12.8 -> 12.8 us (13.2), x 8192 18.8 -> 16.2 us (14.6);
      //   twelve tiles up to a quarter of the SMs, two pairs per cluster, from 48 k-blocks on:
      //     1024 x 1024 x 4096 18.2 -> 15.0 us (12.9), 768 x 768 x 4096 17.7 -> 14.9 us (10.4),
      //     1024 x 512 x 4096 15.4 -> 14.1 us (10.4), 512 x 1024 x 8192 21.5 -> 20.3 us (15.9),
      //     256 x 4096 x 4096 18.7 -> 15.5 us (14.3), 2304 x 256 x 4096 18.2 -> 14.9 us (11.0);
      //     1024 x 1024 x 2048 (32 k-blocks) 12.0 -> 11.6 us: not worth a second form;
      //     512 x 640 x 8192 (ten tiles, 40 CTAs) 19.6 -> 20.4 us: left to the forms below.
      // With four tiles or fewer the single-CTA clusters below stay ahead (256 x 256 x 4096: 9.0
      // against 11.5 us).  Clusters of eight CTAs with 214 KB of shared memory each are placed
      // about a dozen at a time, which is why larger problems get two pairs per cluster.
      const bool deep = force_split || (few ? kbs >= 48 : kbs >= 192);
      const uint64_t tiles128 = (uint64_t)((d.M + 255) / 256) * (uint64_t)((d.N + 127) / 128);
      const int whole_kernel = pl->info.kernel;
      const int64_t rows_pad = (d.M + 255) / 256 * 256, cols_pad = (d.N + 127) / 128 * 128;
      const bool full_tiles = 4 * (rows_pad - d.M) <= rows_pad && 4 * (cols_pad - d.N) <= cols_pad;
      int pcl = 0;
      if (d.k_split == 3) {   // forced: four pairs per cluster where the SMs allow, else two
        for (int sp : {4, 2})
          if (!pcl && pair_ok && tiles128 * 2 * sp <= (uint64_t)pl->sm_count && kbs >= 8u * sp) pcl = sp;
      } else if (d.k_split == 0 && pair_ok && full_tiles && kbs <= 128) {
        if (tiles128 >= 6 && tiles128 <= 9 && kbs >= 32) pcl = 4;
        else if (tiles128 >= 12 && tiles128 * 4 <= (uint64_t)pl->sm_count && kbs >= 48) pcl = 2;
      }
      bool took_pcl = false;
      if (pcl) {
        plan_tcgen05(pl, /*swap=*/false, /*pair=*/true, 0, false, 0, pcl);
        took_pcl = !pl->plan_error && (!pl->have_device || pair_clusters_fit(pl));
        if (!took_pcl && d.k_split == 3 && pcl == 4) {   // forced: two pairs per cluster will do
          plan_tcgen05(pl, /*swap=*/false, /*pair=*/true, 0, false, 0, 2);
          took_pcl = !pl->plan_error && (!pl->have_device || pair_clusters_fit(pl));
        }
        // no cluster shape the device can place: back to whole tiles, and to the choices below
        if (!took_pcl) plan_tcgen05(pl, /*swap=*/false, whole_kernel == FRISK_KERNEL_TCGEN05_PAIR);
      }
      if (!took_pcl && !planes && deep && t128 * kbs * (uint64_t)(pl->sm_count + 1) < (1ull << 32)) {
        // narrower tiles give a small C more of them: the width with the most CTAs wins, a
        // cluster plan (the reduction stays on chip) before a stream-K one
        const frisk_gemm_plan_info whole = pl->info;
        int best_score = whole.num_ctas, best_tn = -1;
        for (int tn : {0, 128, 64}) {
          if (tn && d.N <= tn) continue;
          pl->kd.tile_n = tn;
          plan_tcgen05(pl, /*swap=*/false, /*pair=*/false, /*cluster_try=*/0, /*ksplit=*/true);
          const int score = pl->info.num_ctas + (pl->gp.split_mode == 3 ? 1000 : 0);
          const bool better = score > best_score || (force_split && best_tn < 0);
          if (!pl->plan_error && better) {
            best_score = score;
            best_tn = tn;
          }
        }
        pl->kd.tile_n = best_tn > 0 ? best_tn : 0;
        if (best_tn >= 0) plan_tcgen05(pl, /*swap=*/false, /*pair=*/false, /*cluster_try=*/0, /*ksplit=*/true);
        else plan_tcgen05(pl, /*swap=*/false, whole.kernel == FRISK_KERNEL_TCGEN05_PAIR);   // nothing gained
        // The split forms above fill the SMs with small tiles, and small tiles pull many bytes from
        // L2 per FLOP: their time follows tiles x (tile rows + tile columns) x K bytes at 7 - 9 TB/s
        // (512 x 512 x 65536 as 128 x 64 tiles: 805 MB, 100 us).  K planes keep 256 x 256 tiles and
        // pay a second launch that cannot start before the first has drained (about 10 us more on a
        // problem of a few microseconds), so they are taken when they save more L2 traffic than
        // that costs.  bf16, K split over clusters -> K planes (cuBLAS): 512 x 512 x 65536
        // 100 -> 40 us (44), 1024 x 1024 x 16384 43 -> 35 us (36), 512 x 1024 x 8192 20.9 -> 19.4 us
        // (16); 129 x 1000 x 8192 18.2 -> 21.8 us and 512 x 512 x 4096 12.3 -> 17.0 us are what the
        // rule keeps out.
        if (best_tn >= 0 && planes_ok && d.k_split == 0) {
          const frisk::GemmParams& sg = pl->gp;
          const double es = (double)elem_size(d.a_type), kk = (double)d.K;
          const double split_bytes = (double)sg.tiles_r * sg.tiles_c * (128.0 * sg.mi + sg.tile_n) * kk * es;
          const double planes_bytes = (double)tiles256 * (256.0 + (double)tn256) * kk * es;
          planes = split_bytes - planes_bytes > 80.0e6;
        }
      }
      if (planes) {
        pl->kd.tile_n = 0;
        plan_tcgen05(pl, /*swap=*/false, /*pair=*/true, 0, false, (int)kparts);
      }
    }
    if (pl->info.kernel == FRISK_KERNEL_SKINNY && d.row_reduce) {  // a forced few-row plan
      delete pl;
      return FRISK_ERR_UNSUPPORTED;
    }
  }
  if (pl->plan_error) {
    const int rc = pl->plan_error;
    delete pl;
    return rc;
  }
  if (pl->info.kernel == FRISK_KERNEL_SIMT) {
    pl->repack_a_bytes = pl->repack_b_bytes = 0;   // (a forced or otherwise ineligible problem)
    pl->kd = pl->d;
  }
  pl->ws_bytes += pl->repack_a_bytes + pl->repack_b_bytes;
  pl->info.launches += (pl->repack_a_bytes ? 1 : 0) + (pl->repack_b_bytes ? 1 : 0);
  *out = pl;
  return FRISK_OK;
}

int frisk_b200_gemm_plan_operand_layout(const frisk_gemm_plan* pl, int32_t operand,
                                        frisk_tma_params* layout, uint64_t* umma_desc_base,
                                        int32_t* tma_boxes_per_stage) {
  if (!pl || operand < 0 || operand > 1) return FRISK_ERR_INVALID_ARGUMENT;
  if (pl->info.kernel == FRISK_KERNEL_SIMT) return FRISK_ERR_UNSUPPORTED;  // nothing is staged by TMA
  const frisk::OperandParams& o = operand ? pl->gp.b : pl->gp.a;
  if (layout) *layout = operand ? pl->lay_b : pl->lay_a;
  if (umma_desc_base) *umma_desc_base = o.desc_base;
  if (tma_boxes_per_stage) *tma_boxes_per_stage = (int32_t)o.num_boxes;
  return FRISK_OK;
}

void frisk_b200_gemm_plan_destroy(frisk_gemm_plan* pl) {
  if (!pl) return;
  cudaFree(pl->hA); cudaFree(pl->hB); cudaFree(pl->hC); cudaFree(pl->hWs);
  cudaFree(pl->hSa); cudaFree(pl->hSb); cudaFree(pl->hStatus); cudaFree(pl->hRr);
  if (pl->hstream) cudaStreamDestroy(pl->hstream);
  if (pl->s_in) cudaStreamDestroy(pl->s_in);
  if (pl->s_out) cudaStreamDestroy(pl->s_out);
  if (pl->ev_start) cudaEventDestroy(pl->ev_start);
  for (int i = 0; i < frisk_gemm_plan::kMaxChunks; ++i) {
    if (pl->ev_in[i]) cudaEventDestroy(pl->ev_in[i]);
    if (pl->ev_done[i]) cudaEventDestroy(pl->ev_done[i]);
  }
  frisk_b200_gemm_plan_destroy(pl->chunk_plan);
  frisk_b200_gemm_plan_destroy(pl->tail_plan);
  cudaGetLastError();
  delete pl;
}

int frisk_b200_gemm_plan_info(const frisk_gemm_plan* pl, frisk_gemm_plan_info* out) {
  if (!pl || !out) return FRISK_ERR_INVALID_ARGUMENT;
  *out = pl->info;
  out->cuda_core_runs = pl->simt_fallback_runs;
  return FRISK_OK;
}

int frisk_b200_gemm_workspace_bytes(const frisk_gemm_plan* pl, size_t* out) {
  if (!pl || !out) return FRISK_ERR_INVALID_ARGUMENT;
  *out = pl->ws_bytes;
  return FRISK_OK;
}

int frisk_b200_gemm_run(frisk_gemm_plan* pl, const void* A, const void* B, void* C,
                        const float* scale_a, const float* scale_b, void* workspace,
                        size_t workspace_bytes, int32_t* device_status, void* stream) {
  frisk_gemm_run_args a;
  memset(&a, 0, sizeof a);
  a.A = A; a.B = B; a.C = C;
  a.scale_a = scale_a; a.scale_b = scale_b;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  a.device_status = device_status;
  a.stream = stream;
  return frisk_b200_gemm_run_ex(pl, &a);
}

int frisk_b200_gemm_run_ex(frisk_gemm_plan* pl, const frisk_gemm_run_args* args) {
  if (!pl || !args) return FRISK_ERR_INVALID_ARGUMENT;
  const void *A = args->A, *B = args->B;
  void* C = args->C;
  void* workspace = args->workspace;
  if (!A || !B || !C) return FRISK_ERR_INVALID_ARGUMENT;
  const frisk_gemm_desc& d = pl->d;
  if (d.scale_mode == FRISK_SCALE_ROW_COL && (!args->scale_a || !args->scale_b))
    return FRISK_ERR_INVALID_ARGUMENT;
  if (args->n_peers < 0 || args->n_peers > frisk::kMaxPeers) return FRISK_ERR_INVALID_ARGUMENT;
  for (int q = 0; q < args->n_peers; ++q)
    if (!args->peer_c[q]) return FRISK_ERR_INVALID_ARGUMENT;
  if (d.row_reduce && !args->row_reduce_dst) return FRISK_ERR_INVALID_ARGUMENT;
  if (!pl->have_device) return FRISK_ERR_NO_DEVICE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(args->stream);
  const float* sa = d.scale_mode ? args->scale_a : nullptr;
  const float* sb = d.scale_mode ? args->scale_b : nullptr;
  const bool whole_tile_tc = pl->gp.split_mode == 0 && pl->gp.k_parts <= 1u && !pl->pair_cluster && (pl->info.kernel == FRISK_KERNEL_TCGEN05 ||
                                                        pl->info.kernel == FRISK_KERNEL_TCGEN05_PAIR);

  if (pl->tf32) {
    // fp32 on the tensor cores: split A and B into the workspace, then run the tensor-core
    // kernel on the split operands (K three times as long).  Any alignment of A and B will do:
    // the split reads them with plain loads.
    if (args->n_peers > 0) return FRISK_ERR_UNSUPPORTED;
    if (!workspace || args->workspace_bytes < pl->ws_bytes) return FRISK_ERR_WORKSPACE;
    if ((uintptr_t)workspace % 256) return FRISK_ERR_MISALIGNED;
    float* a3 = reinterpret_cast<float*>(workspace);
    float* b3 = reinterpret_cast<float*>(static_cast<char*>(workspace) + pl->tf32_a_bytes);
    const frisk_gemm_desc& k = pl->kd;
    // A' = [A_lo | A_hi], B' = [B_hi | B_lo] along K
    const int64_t ks = k.K / 3;
    int rc = launch_tf32_split(static_cast<const float*>(A), a3, d.M, d.K, ks, d.lda, k.lda,
                               /*k_along_rows=*/d.transA != 0, 0x1u, pl->sm_count, st);
    if (rc) return rc;
    rc = launch_tf32_split(static_cast<const float*>(B), b3, d.N, d.K, ks, d.ldb, k.ldb,
                           /*k_along_rows=*/d.transB == 0, 0x2u, pl->sm_count, st);
    if (rc) return rc;
    frisk::GemmParams g = pl->gp;
    OperandView va{a3, k.M, 2 * ks, k.lda, k.transA != 0};
    OperandView vb{b3, k.N, 2 * ks, k.ldb, k.transB == 0};
    rc = encode_operand_map(&pl->tmap_a, va, FRISK_DT_F32, g.a.box_mn, g.bk_elems, pl->lay_a.swizzle_bytes);
    if (rc) return rc;
    rc = encode_operand_map(&pl->tmap_b, vb, FRISK_DT_F32, g.b.box_mn, g.bk_elems, pl->lay_b.swizzle_bytes);
    if (rc) return rc;
    g.C = C;
    g.status = args->device_status;
    g.c_vec_ok = ((uintptr_t)C % 16 == 0) && ((d.ldc * elem_size(d.c_type)) % 16 == 0);
    return pl->tf32_pair ? launch_pair_tf<float, true>(pl, g, st)
                         : launch_tcgen05_ts<float, false, true>(pl, g, st);
  }

  // operands with an odd row pitch are copied into the front of the workspace first
  const void *A0 = A, *B0 = B;
  const size_t repack_bytes = pl->repack_a_bytes + pl->repack_b_bytes;
  const frisk_gemm_desc& k = pl->kd;
  if (repack_bytes) {
    if (!workspace || args->workspace_bytes < pl->ws_bytes) return FRISK_ERR_WORKSPACE;
    if ((uintptr_t)workspace % 16) return FRISK_ERR_MISALIGNED;
    const int es = elem_size(d.a_type);
    char* w = static_cast<char*>(workspace);
    if (pl->repack_a_bytes) {
      if (int rc = launch_repack(A, w, d.transA ? d.K : d.M, d.transA ? d.M : d.K, d.lda, k.lda, es,
                                 pl->sm_count, st))
        return rc;
      A = w;
    }
    if (pl->repack_b_bytes) {
      char* wb = w + pl->repack_a_bytes;
      if (int rc = launch_repack(B, wb, d.transB ? d.N : d.K, d.transB ? d.K : d.N, d.ldb, k.ldb, es,
                                 pl->sm_count, st))
        return rc;
      B = wb;
    }
    workspace = w + repack_bytes;   // what follows is the kernels' own scratch
  }
  const bool ptr_aligned = ((uintptr_t)A % 16 == 0) && ((uintptr_t)B % 16 == 0);
  if ((args->n_peers > 0 || d.row_reduce) && !(whole_tile_tc && ptr_aligned)) {
    g_last_error = "peer copies of C and the fused row reduce exist only in the whole-tile "
                   "tensor-core kernels (16-byte aligned A and B; a plan that splits K is kept to "
                   "whole tiles by desc.k_split = -1)";
    return FRISK_ERR_UNSUPPORTED;
  }
  if (pl->info.kernel != FRISK_KERNEL_SIMT && !ptr_aligned) {
    // TMA needs 16-byte aligned bases; the run still gives the right answer, about 100x slower,
    // so it is counted (plan_info.cuda_core_runs) and noted where the caller can read it
    ++pl->simt_fallback_runs;
    g_last_error = "A or B is not 16-byte aligned: this run used the CUDA-core kernel";
  }
  if (pl->info.kernel == FRISK_KERNEL_SIMT || !ptr_aligned)
    return launch_simt(d, A0, B0, C, sa, sb, st);  // the CUDA-core kernel has no alignment rule

  const bool swap = pl->info.kernel == FRISK_KERNEL_SKINNY;
  const size_t own_ws_bytes = pl->ws_bytes - repack_bytes;
  if (own_ws_bytes) {
    if (!workspace || args->workspace_bytes < pl->ws_bytes) return FRISK_ERR_WORKSPACE;
    if ((uintptr_t)workspace % 16) return FRISK_ERR_MISALIGNED;
  }
  frisk::GemmParams g = pl->gp;
  if (A != pl->cached_a || B != pl->cached_b) {
    OperandView va{A, d.M, d.K, k.lda, d.transA != 0};
    OperandView vb{B, d.N, d.K, k.ldb, d.transB == 0};
    const OperandView& ra = swap ? vb : va;  // a-role: the 128-row operand
    const OperandView& rb = swap ? va : vb;
    int rc = encode_operand_map(&pl->tmap_a, ra, d.a_type, g.a.box_mn, g.bk_elems, pl->lay_a.swizzle_bytes);
    if (rc) return rc;
    rc = encode_operand_map(&pl->tmap_b, rb, d.a_type, g.b.box_mn, g.bk_elems, pl->lay_b.swizzle_bytes);
    if (rc) return rc;
    pl->cached_a = A;
    pl->cached_b = B;
  }
  g.C = C;
  g.status = args->device_status;
#ifdef FRISK_B200_MEASURE
  if (const char* dbg = getenv("FRISK_B200_DEBUG_MODE")) g.debug_mode = (uint32_t)atoi(dbg);
  if (const char* tr = getenv("FRISK_B200_TRACE")) g.trace = reinterpret_cast<long long*>(strtoull(tr, nullptr, 0));
#endif
  g.c_vec_ok = ((uintptr_t)C % 16 == 0) && ((d.ldc * elem_size(d.c_type)) % 16 == 0);
  g.n_peers = (uint32_t)args->n_peers;
  for (int q = 0; q < args->n_peers; ++q) {
    g.peer_c[q] = args->peer_c[q];
    // a peer copy that cannot take 16-byte stores switches every copy to element stores
    if ((uintptr_t)args->peer_c[q] % 16) g.c_vec_ok = 0;
  }
  if (g.epi_staged == 3u) {
    if (!g.c_vec_ok) {
      g.epi_staged = 1u;  // a base off the 16-byte grid: this run stores without TMA
    } else {
      // one map per destination: [rows of this plan, N] of C's type at pitch ldc, boxes of
      // 32 rows x 128 bytes in the 128-byte swizzle the staging buffers are written in
      for (int q = 0; q <= args->n_peers; ++q) {
        void* dst = q == 0 ? C : args->peer_c[q - 1];
        if (dst == pl->cached_c[q]) continue;
        if (int rc = encode_store_map(&pl->c_maps.m[q], dst, d.c_type, d.M, d.N, d.ldc)) return rc;
        pl->cached_c[q] = dst;
      }
    }
  }
  if (g.split_mode) {
    // (swapped: D is C transposed, its rows run over N (scale_b), its columns over M (scale_a))
    g.row_scale = swap ? sb : sa;
    g.col_scale = swap ? sa : sb;
    if (own_ws_bytes) {
      g.ws = reinterpret_cast<float*>(workspace);
      g.counters = reinterpret_cast<uint32_t*>(static_cast<char*>(workspace) + pl->slot_bytes);
    }
    // The arrival counters must start at zero.  The kernel leaves them at zero when it completes,
    // but nothing guarantees what the caller hands in: a scratch buffer that was given to other
    // code between two runs, one buffer shared by two plans, a run that gave up on a bounded wait.
    // They are a few bytes per tile, so they are cleared on every run, in stream order.
    if (own_ws_bytes)
      FRISK_CUDA(cudaMemsetAsync(g.counters, 0, own_ws_bytes - pl->slot_bytes, st));
  } else {
    g.row_scale = sa;
    g.col_scale = sb;
    if (d.row_reduce) g.rr_partials = reinterpret_cast<float*>(workspace);
  }
  const bool planes = g.k_parts > 1u;
  if (planes) {   // the GEMM launch writes raw fp32 planes; scales, += C and the cast follow in the sum
    g.C = workspace;
    g.c_vec_ok = 1;
    g.row_scale = g.col_scale = nullptr;
  }
  int rc;
  if (pl->pair_cluster) {
    rc = launch_pair_ksplit(pl, g, st);
  } else if (planes) {
    rc = launch_pair_t<float>(pl, g, st);
    if (!rc) {
      const float* w = static_cast<const float*>(workspace);
      switch (d.c_type) {
        case FRISK_DT_F32: rc = launch_kplanes_sum_t<float>(pl, g, w, C, sa, sb, st); break;
        case FRISK_DT_F16: rc = launch_kplanes_sum_t<__half>(pl, g, w, C, sa, sb, st); break;
        case FRISK_DT_BF16: rc = launch_kplanes_sum_t<__nv_bfloat16>(pl, g, w, C, sa, sb, st); break;
        default: rc = FRISK_ERR_UNSUPPORTED;
      }
    }
  } else if (pl->info.kernel == FRISK_KERNEL_TCGEN05_PAIR) {
    switch (d.c_type) {
      case FRISK_DT_F32: rc = launch_pair_t<float>(pl, g, st); break;
      case FRISK_DT_F16: rc = launch_pair_t<__half>(pl, g, st); break;
      case FRISK_DT_BF16: rc = launch_pair_t<__nv_bfloat16>(pl, g, st); break;
      default: rc = FRISK_ERR_UNSUPPORTED;
    }
  } else {
    switch (d.c_type) {
      case FRISK_DT_F32: rc = launch_tcgen05_t<float>(pl, g, st); break;
      case FRISK_DT_F16: rc = launch_tcgen05_t<__half>(pl, g, st); break;
      case FRISK_DT_BF16: rc = launch_tcgen05_t<__nv_bfloat16>(pl, g, st); break;
      default: rc = FRISK_ERR_UNSUPPORTED;
    }
  }
  if (!rc && d.row_reduce) {
    switch (d.c_type) {
      case FRISK_DT_F32: rc = launch_row_fold_t<float>(pl, g, args->row_reduce_dst, st); break;
      case FRISK_DT_F16: rc = launch_row_fold_t<__half>(pl, g, args->row_reduce_dst, st); break;
      case FRISK_DT_BF16: rc = launch_row_fold_t<__nv_bfloat16>(pl, g, args->row_reduce_dst, st); break;
      default: rc = FRISK_ERR_UNSUPPORTED;
    }
  }
  return rc;
}

int frisk_b200_peer_alloc(size_t bytes, void** ptr, unsigned char handle[64]) {
  if (!ptr || !handle || bytes == 0) return FRISK_ERR_INVALID_ARGUMENT;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle crosses the ABI as 64 bytes");
  *ptr = nullptr;
  void* p = nullptr;
  FRISK_CUDA(cudaMalloc(&p, bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    cudaFree(p);
    return cuda_fail(e, "cudaIpcGetMemHandle");
  }
  memcpy(handle, &h, sizeof h);
  *ptr = p;
  return FRISK_OK;
}

int frisk_b200_peer_open(const unsigned char handle[64], void** ptr) {
  if (!ptr || !handle) return FRISK_ERR_INVALID_ARGUMENT;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof h);
  *ptr = nullptr;
  FRISK_CUDA(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return FRISK_OK;
}

int frisk_b200_peer_close(void* ptr) {
  if (!ptr) return FRISK_OK;
  FRISK_CUDA(cudaIpcCloseMemHandle(ptr));
  return FRISK_OK;
}

int frisk_b200_peer_free(void* ptr) {
  if (!ptr) return FRISK_OK;
  FRISK_CUDA(cudaFree(ptr));
  return FRISK_OK;
}

namespace {

// Decides once per plan whether frisk_b200_gemm_run_host runs as a pipeline of row chunks.  With
// the operands in host memory the call is bound by the PCIe copies (cfg5: 1.2 GB up, 1 GB down
// against 6 ms of GEMM), and the two directions are independent links: while chunk i is computed
// chunk i+1 is on its way up and chunk i-1 on its way down.  Needs A stored row-major (a row chunk
// is then one contiguous block) and enough rows for at least two chunks of 2048.
int plan_host_pipeline(frisk_gemm_plan* pl) {
  const frisk_gemm_desc& d = pl->d;
  pl->n_chunks = 1;
  if (d.transA || d.M < 4096) return FRISK_OK;
  int n = (int)std::min<int64_t>(frisk_gemm_plan::kMaxChunks, d.M / 2048);
  int64_t rows = ((d.M + n - 1) / n + 255) / 256 * 256;
  n = (int)((d.M + rows - 1) / rows);
  if (n < 2) return FRISK_OK;
  frisk_gemm_desc dc = d;
  dc.M = rows;
  int rc = frisk_b200_gemm_plan_create(&dc, &pl->chunk_plan);
  if (rc) return rc;
  const int64_t tail = d.M - (int64_t)(n - 1) * rows;
  if (tail != rows) {
    dc.M = tail;
    rc = frisk_b200_gemm_plan_create(&dc, &pl->tail_plan);
    if (rc) return rc;
  }
  // the chunk plans must not need a workspace of their own (they are never few-row plans)
  if (pl->chunk_plan->ws_bytes || (pl->tail_plan && pl->tail_plan->ws_bytes)) return FRISK_OK;
  FRISK_CUDA(cudaStreamCreateWithFlags(&pl->s_in, cudaStreamNonBlocking));
  FRISK_CUDA(cudaStreamCreateWithFlags(&pl->s_out, cudaStreamNonBlocking));
  FRISK_CUDA(cudaEventCreateWithFlags(&pl->ev_start, cudaEventDisableTiming));
  for (int i = 0; i < n; ++i) {
    FRISK_CUDA(cudaEventCreateWithFlags(&pl->ev_in[i], cudaEventDisableTiming));
    FRISK_CUDA(cudaEventCreateWithFlags(&pl->ev_done[i], cudaEventDisableTiming));
  }
  pl->chunk_rows = rows;
  pl->n_chunks = n;
  return FRISK_OK;
}

int run_host_pipelined(frisk_gemm_plan* pl, const void* A, const void* B, void* C,
                       const float* scale_a, const float* scale_b) {
  const frisk_gemm_desc& d = pl->d;
  const size_t a_pitch = (size_t)d.lda * elem_size(d.a_type);
  const size_t c_pitch = (size_t)d.ldc * elem_size(d.c_type);
  const size_t c_row = (size_t)d.N * elem_size(d.c_type);
  cudaStream_t s_in = pl->s_in, s_cmp = pl->hstream, s_out = pl->s_out;
  // up: status word, B, scales, then the chunks of A (and of C when the GEMM accumulates into it)
  FRISK_CUDA(cudaMemsetAsync(pl->hStatus, 0, sizeof(int32_t), s_in));
  if (int rc = upload_b(d, pl->hB, B, s_in)) return rc;
  if (d.scale_mode) {
    FRISK_CUDA(cudaMemcpyAsync(pl->hSa, scale_a, d.M * sizeof(float), cudaMemcpyHostToDevice, s_in));
    FRISK_CUDA(cudaMemcpyAsync(pl->hSb, scale_b, d.N * sizeof(float), cudaMemcpyHostToDevice, s_in));
  }
  for (int i = 0; i < pl->n_chunks; ++i) {
    const int64_t r0 = (int64_t)i * pl->chunk_rows;
    const int64_t rows = std::min<int64_t>(pl->chunk_rows, d.M - r0);
    frisk_gemm_plan* sub = (rows == pl->chunk_rows) ? pl->chunk_plan : pl->tail_plan;
    char* a_dst = static_cast<char*>(pl->hA) + r0 * a_pitch;
    char* c_host = static_cast<char*>(C) + r0 * c_pitch;
    char* c_dev = static_cast<char*>(pl->hC) + r0 * c_pitch;
    if (int rc = upload_a(d, pl->hA, A, r0, rows, s_in)) return rc;
    if (!d.clear_accum)
      if (int rc = upload_c(d, pl->hC, C, r0, rows, s_in)) return rc;
    FRISK_CUDA(cudaEventRecord(pl->ev_in[i], s_in));
    // compute
    FRISK_CUDA(cudaStreamWaitEvent(s_cmp, pl->ev_in[i], 0));
    int rc = frisk_b200_gemm_run(sub, a_dst, pl->hB, c_dev, pl->hSa ? pl->hSa + r0 : nullptr,
                                 pl->hSb, nullptr, 0, pl->hStatus, s_cmp);
    if (rc) {
      cudaDeviceSynchronize();  // nothing of this call may still be in flight when it returns
      return rc;
    }
    FRISK_CUDA(cudaEventRecord(pl->ev_done[i], s_cmp));
    // down: only the N columns of each row, the caller's padding stays as it was
    FRISK_CUDA(cudaStreamWaitEvent(s_out, pl->ev_done[i], 0));
    FRISK_CUDA(cudaMemcpy2DAsync(c_host, c_pitch, c_dev, c_pitch, c_row, (size_t)rows,
                                 cudaMemcpyDeviceToHost, s_out));
  }
  // the next call reuses the device buffers: its first copy must not overtake this call's last
  // GEMM or copy-back, so everything drains here (the call is synchronous anyway)
  FRISK_CUDA(cudaStreamSynchronize(s_cmp));
  return frisk_b200_check_status(pl->hStatus, s_out);
}

}  // namespace

int frisk_b200_gemm_run_host(frisk_gemm_plan* pl, const void* A, const void* B, void* C,
                             const float* scale_a, const float* scale_b) {
  return frisk_b200_gemm_run_host_ex(pl, A, B, C, scale_a, scale_b, nullptr);
}

int frisk_b200_gemm_run_host_ex(frisk_gemm_plan* pl, const void* A, const void* B, void* C,
                                const float* scale_a, const float* scale_b, void* row_reduce_dst) {
  if (!pl || !A || !B || !C) return FRISK_ERR_INVALID_ARGUMENT;
  if (!pl->have_device) return FRISK_ERR_NO_DEVICE;
  const frisk_gemm_desc& d = pl->d;
  if (d.scale_mode == FRISK_SCALE_ROW_COL && (!scale_a || !scale_b))
    return FRISK_ERR_INVALID_ARGUMENT;
  if ((d.row_reduce != 0) != (row_reduce_dst != nullptr)) return FRISK_ERR_INVALID_ARGUMENT;
  if (!pl->hA) {
    FRISK_CUDA(cudaStreamCreateWithFlags(&pl->hstream, cudaStreamNonBlocking));
    FRISK_CUDA(cudaMalloc(&pl->hA, a_bytes(d)));
    FRISK_CUDA(cudaMalloc(&pl->hB, b_bytes(d)));
    FRISK_CUDA(cudaMalloc(&pl->hC, c_bytes(d)));
    FRISK_CUDA(cudaMalloc(&pl->hStatus, sizeof(int32_t)));
    if (pl->ws_bytes) FRISK_CUDA(cudaMalloc(&pl->hWs, pl->ws_bytes));
    if (d.scale_mode) {
      FRISK_CUDA(cudaMalloc(&pl->hSa, d.M * sizeof(float)));
      FRISK_CUDA(cudaMalloc(&pl->hSb, d.N * sizeof(float)));
    }
    if (d.row_reduce) FRISK_CUDA(cudaMalloc(&pl->hRr, (size_t)d.M * elem_size(d.c_type)));
  }
  cudaStream_t st = pl->hstream;
  if (pl->n_chunks == 0) {
    if (d.row_reduce) {
      pl->n_chunks = 1;  // the fold's workspace belongs to the whole problem: no row chunks
    } else {
      int rc = plan_host_pipeline(pl);
      if (rc) return rc;
    }
  }
  if (pl->n_chunks > 1) return run_host_pipelined(pl, A, B, C, scale_a, scale_b);
  FRISK_CUDA(cudaMemsetAsync(pl->hStatus, 0, sizeof(int32_t), st));
  if (int rc = upload_a(d, pl->hA, A, 0, d.transA ? d.K : d.M, st)) return rc;
  if (int rc = upload_b(d, pl->hB, B, st)) return rc;
  if (!d.clear_accum)
    if (int rc = upload_c(d, pl->hC, C, 0, d.M, st)) return rc;
  if (d.scale_mode) {
    FRISK_CUDA(cudaMemcpyAsync(pl->hSa, scale_a, d.M * sizeof(float), cudaMemcpyHostToDevice, st));
    FRISK_CUDA(cudaMemcpyAsync(pl->hSb, scale_b, d.N * sizeof(float), cudaMemcpyHostToDevice, st));
  }
  const size_t rr_bytes = (size_t)d.M * elem_size(d.c_type);
  if (d.row_reduce && !d.row_reduce_clear)
    FRISK_CUDA(cudaMemcpyAsync(pl->hRr, row_reduce_dst, rr_bytes, cudaMemcpyHostToDevice, st));
  frisk_gemm_run_args ra;
  memset(&ra, 0, sizeof ra);
  ra.A = pl->hA; ra.B = pl->hB; ra.C = pl->hC;
  ra.scale_a = pl->hSa; ra.scale_b = pl->hSb;
  ra.workspace = pl->hWs; ra.workspace_bytes = pl->ws_bytes;
  ra.device_status = pl->hStatus;
  ra.stream = st;
  ra.row_reduce_dst = pl->hRr;
  int rc = frisk_b200_gemm_run_ex(pl, &ra);
  if (rc) return rc;
  if (d.row_reduce)
    FRISK_CUDA(cudaMemcpyAsync(row_reduce_dst, pl->hRr, rr_bytes, cudaMemcpyDeviceToHost, st));
  // only the N columns of each row come back: padding beyond them in the caller's C stays as it was
  const size_t c_pitch = (size_t)d.ldc * elem_size(d.c_type);
  FRISK_CUDA(cudaMemcpy2DAsync(C, c_pitch, pl->hC, c_pitch, (size_t)d.N * elem_size(d.c_type),
                               (size_t)d.M, cudaMemcpyDeviceToHost, st));
  return frisk_b200_check_status(pl->hStatus, st);
}

// ------------------------------------------------------------------------------------------
// Skinny GEMM for callers that cannot allocate device memory.
//
// Some hosts of this library are not allowed to call cudaMalloc: a plugin that runs inside
// another framework's memory pool and must not grow the process's footprint behind its back, a
// service whose memory budget is fixed at start-up, a replay of pre-recorded work where every
// buffer has to exist beforehand.  The skinny (few-row) plan needs fp32 scratch for its partial
// sums; here that scratch is a fixed array inside the library image instead of a buffer the
// caller (or the library) would have to allocate.  Every GPU that loads the library holds the
// array until the process exits.
constexpr size_t kStaticScratchFloats = 1u << 20;  // 4 MiB: M * N <= 1,048,576 outputs
static __device__ __align__(256) float g_skinny_scratch[kStaticScratchFloats];

namespace {
// Device address of g_skinny_scratch per device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel could use; the address is asked for once per
// device, with that device current.
float* g_scratch_addr[kMaxDevices] = {nullptr};

int static_scratch_for_current_device(float** out) {
  int dev = 0;
  FRISK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return FRISK_ERR_UNSUPPORTED;
  float* p = __atomic_load_n(&g_scratch_addr[dev], __ATOMIC_ACQUIRE);
  if (!p) {
    void* sym = nullptr;
    FRISK_CUDA(cudaGetSymbolAddress(&sym, g_skinny_scratch));
    p = static_cast<float*>(sym);
    __atomic_store_n(&g_scratch_addr[dev], p, __ATOMIC_RELEASE);  // same value from any thread
  }
  *out = p;
  return FRISK_OK;
}
}  // namespace

int frisk_b200_gemm_skinny_static(const frisk_gemm_desc* desc, const void* A, const void* B,
                                  void* C, const float* scale_a, const float* scale_b,
                                  int32_t* device_status, void* stream) {
  if (!desc || !A || !B || !C) return FRISK_ERR_INVALID_ARGUMENT;
  frisk_gemm_desc d = *desc;
  if (d.M <= 0 || d.N <= 0 || d.K <= 0) return FRISK_ERR_INVALID_ARGUMENT;
  if (!elem_size(d.a_type) || d.a_type != d.b_type || !elem_size(d.c_type) ||
      is_fp8(d.c_type))
    return FRISK_ERR_INVALID_ARGUMENT;
  if (d.scale_mode != FRISK_SCALE_NONE && d.scale_mode != FRISK_SCALE_ROW_COL)
    return FRISK_ERR_INVALID_ARGUMENT;
  if (d.scale_mode == FRISK_SCALE_ROW_COL && (!scale_a || !scale_b))
    return FRISK_ERR_INVALID_ARGUMENT;
  if ((uint64_t)d.M * (uint64_t)d.N > kStaticScratchFloats) {
    char buf[160];
    snprintf(buf, sizeof buf,
             "M * N = %lld exceeds the %zu outputs the built-in scratch array holds; use "
             "frisk_b200_gemm_run with a workspace",
             (long long)(d.M * d.N), kStaticScratchFloats);
    g_last_error = buf;
    return FRISK_ERR_TOO_LARGE;
  }
  d.transA = d.transA != 0;
  d.transB = d.transB != 0;
  if (d.lda == 0) d.lda = d.transA ? d.M : d.K;
  if (d.ldb == 0) d.ldb = d.transB ? d.K : d.N;
  if (d.ldc == 0) d.ldc = d.N;
  if (d.lda < (d.transA ? d.M : d.K) || d.ldb < (d.transB ? d.K : d.N) || d.ldc < d.N)
    return FRISK_ERR_INVALID_ARGUMENT;
  d.force_kernel = 0;
  d.tile_n = 0;
  d.band_tiles = 0;
  // only the few-row plan uses scratch; everything else has no reason to come through here
  // (this entry point keeps the 64-row limit the few-row plan had when it was written)
  if (!(tcgen05_eligible(d) && d.M <= 64 && skinny_shape(d, 1024))) return FRISK_ERR_UNSUPPORTED;
  if (((uintptr_t)A % 16) || ((uintptr_t)B % 16)) return FRISK_ERR_MISALIGNED;

  frisk_gemm_plan pl;  // lives on the stack: nothing is allocated on the host heap either
  pl.d = d;
  pl.kd = d;
  memset(&pl.info, 0, sizeof pl.info);
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return FRISK_ERR_NO_DEVICE;
  }
  int major = 0, sms = 0;
  FRISK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  FRISK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (major != 10) return FRISK_ERR_NO_DEVICE;
  pl.device = dev;
  pl.sm_count = sms;
  pl.have_device = true;
  plan_tcgen05(&pl, /*swap=*/true, /*pair=*/false, /*cluster_try=*/-1);
  if (pl.plan_error) return pl.plan_error;
  // this entry point keeps the atomic split (mode 1): its scratch is M x N fp32, independent of
  // the grid, which is what lets a fixed array serve it
  pl.gp.split_mode = 1;
  pl.ws_bytes = (size_t)d.M * d.N * sizeof(float);

  float* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch);
  if (rc) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  // the array keeps whatever the previous call (or an interrupted one) left: start from zero
  FRISK_CUDA(cudaMemsetAsync(scratch, 0, pl.ws_bytes, st));

  frisk::GemmParams g = pl.gp;
  OperandView va{A, d.M, d.K, d.lda, false};
  OperandView vb{B, d.N, d.K, d.ldb, d.transB == 0};
  rc = encode_operand_map(&pl.tmap_a, vb, d.a_type, g.a.box_mn, g.bk_elems, pl.lay_a.swizzle_bytes);  // weights: 128-row role
  if (rc) return rc;
  rc = encode_operand_map(&pl.tmap_b, va, d.a_type, g.b.box_mn, g.bk_elems, pl.lay_b.swizzle_bytes);
  if (rc) return rc;
  g.C = C;
  g.status = device_status;
  g.c_vec_ok = ((uintptr_t)C % 16 == 0) && ((d.ldc * elem_size(d.c_type)) % 16 == 0);
  g.ws = scratch;
  g.row_scale = nullptr;
  g.col_scale = nullptr;
  const float* sa = d.scale_mode ? scale_a : nullptr;
  const float* sb = d.scale_mode ? scale_b : nullptr;
  switch (d.c_type) {
    case FRISK_DT_F32:
      rc = launch_tcgen05_t<float>(&pl, g, st);
      if (!rc) rc = launch_finalize_t<float>(&pl, scratch, C, sa, sb, st);
      break;
    case FRISK_DT_F16:
      rc = launch_tcgen05_t<__half>(&pl, g, st);
      if (!rc) rc = launch_finalize_t<__half>(&pl, scratch, C, sa, sb, st);
      break;
    case FRISK_DT_BF16:
      rc = launch_tcgen05_t<__nv_bfloat16>(&pl, g, st);
      if (!rc) rc = launch_finalize_t<__nv_bfloat16>(&pl, scratch, C, sa, sb, st);
      break;
    default: rc = FRISK_ERR_UNSUPPORTED;
  }
  return rc;
}

size_t frisk_b200_gemm_skinny_static_capacity(void) { return kStaticScratchFloats; }

int frisk_b200_measure_mma_peak(int32_t ab_type, int32_t pair, int32_t k_blocks, int32_t reps,
                                double* tflops, double* ms_per_launch) {
  if (!tflops || k_blocks < 32 || k_blocks % 32 || reps < 1) return FRISK_ERR_INVALID_ARGUMENT;
  if (!elem_size(ab_type)) return FRISK_ERR_UNSUPPORTED;   // fp32 is measured as kind::tf32
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return FRISK_ERR_NO_DEVICE;
  }
  int major = 0, sms = 0;
  FRISK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  FRISK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  if (major != 10) return FRISK_ERR_NO_DEVICE;
  const uint32_t es = (uint32_t)elem_size(ab_type);
  const uint32_t m = pair ? 256u : 128u, n = 256u, k_step = 32u / es;
  const uint32_t idesc = make_idesc(ab_type, false, false, m, n);
  const int ctas = pair ? (sms / 2) * 2 : sms;
  const size_t smem = 4 * (128 * 128 + (pair ? 128 : 256) * 128) + 1024;
  int32_t* status = nullptr;
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  FRISK_CUDA(cudaMalloc(&status, sizeof(int32_t)));
  int rc = FRISK_OK;
  auto fail = [&](cudaError_t e, const char* what) { rc = cuda_fail(e, what); };
  cudaError_t e = cudaMemset(status, 0, sizeof(int32_t));
  if (e != cudaSuccess) fail(e, "cudaMemset");
  if (!rc && (e = cudaEventCreate(&e0)) != cudaSuccess) fail(e, "cudaEventCreate");
  if (!rc && (e = cudaEventCreate(&e1)) != cudaSuccess) fail(e, "cudaEventCreate");
  auto launch = [&]() -> cudaError_t {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDim = dim3((unsigned)ctas, 1, 1);
    cfg.blockDim = dim3(128, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = pair ? 2 : 1;
    attr.val.clusterDim.y = attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    const uint32_t kind = is_fp8(ab_type) ? 1u : ab_type == FRISK_DT_F32 ? 2u : 0u;
    if (pair)
      return cudaLaunchKernelEx(&cfg, frisk::mma_peak_kernel<1>, (uint32_t)k_blocks, idesc, kind, es, status);
    return cudaLaunchKernelEx(&cfg, frisk::mma_peak_kernel<0>, (uint32_t)k_blocks, idesc, kind, es, status);
  };
  if (!rc) {
    e = pair ? cudaFuncSetAttribute(frisk::mma_peak_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
             : cudaFuncSetAttribute(frisk::mma_peak_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) fail(e, "cudaFuncSetAttribute");
  }
  for (int i = 0; !rc && i < 2; ++i)   // warm-up
    if ((e = launch()) != cudaSuccess) fail(e, "mma_peak_kernel launch");
  if (!rc && (e = cudaEventRecord(e0, 0)) != cudaSuccess) fail(e, "cudaEventRecord");
  for (int i = 0; !rc && i < reps; ++i)
    if ((e = launch()) != cudaSuccess) fail(e, "mma_peak_kernel launch");
  if (!rc && (e = cudaEventRecord(e1, 0)) != cudaSuccess) fail(e, "cudaEventRecord");
  if (!rc && (e = cudaEventSynchronize(e1)) != cudaSuccess) fail(e, "cudaEventSynchronize");
  float ms = 0.f;
  if (!rc && (e = cudaEventElapsedTime(&ms, e0, e1)) != cudaSuccess) fail(e, "cudaEventElapsedTime");
  if (!rc) rc = frisk_b200_check_status(status, nullptr);
  if (!rc) {
    const double issuers = pair ? ctas / 2 : ctas;
    const double flop = issuers * (double)k_blocks * 4.0 * 2.0 * m * n * k_step * reps;
    *tflops = flop / (ms * 1e-3) / 1e12;
    if (ms_per_launch) *ms_per_launch = ms / reps;
  }
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(status);
  return rc;
}

int frisk_b200_check_status(const int32_t* device_status, void* stream) {
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  int32_t h = 0;
  if (device_status)
    FRISK_CUDA(cudaMemcpyAsync(&h, device_status, sizeof h, cudaMemcpyDeviceToHost, st));
  FRISK_CUDA(cudaStreamSynchronize(st));
  if (h != 0) {
    char buf[64];
    snprintf(buf, sizeof buf, "device status word 0x%x", (unsigned)h);
    g_last_error = buf;
    return FRISK_ERR_DEVICE_TIMEOUT;
  }
  return FRISK_OK;
}

const char* frisk_b200_strerror(int code) {
  switch (code) {
    case FRISK_OK: return "ok";
    case FRISK_ERR_INVALID_ARGUMENT: return "invalid argument";
    case FRISK_ERR_UNSUPPORTED: return "unsupported dtype or layout";
    case FRISK_ERR_MISALIGNED: return "pointer or leading dimension is not 16-byte aligned";
    case FRISK_ERR_WORKSPACE: return "workspace missing or too small";
    case FRISK_ERR_CUDA: return "CUDA call failed";
    case FRISK_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
    case FRISK_ERR_NO_DEVICE: return "no sm_100 device";
    case FRISK_ERR_SHARD: return "invalid rank or rank count";
    case FRISK_ERR_TOO_LARGE: return "problem exceeds the capacity of this entry point";
    default: return "unknown error";
  }
}

const char* frisk_b200_last_error(void) { return g_last_error.c_str(); }

int frisk_b200_shard_rows(int64_t M, int nranks, int rank, int64_t* row0, int64_t* rows) {
  if (!row0 || !rows || M < 0) return FRISK_ERR_INVALID_ARGUMENT;
  if (nranks <= 0 || rank < 0 || rank >= nranks) return FRISK_ERR_SHARD;
  const int64_t base = M / nranks, extra = M % nranks;
  *rows = base + (rank < extra ? 1 : 0);
  *row0 = rank * base + std::min<int64_t>(rank, extra);
  return FRISK_OK;
}

int frisk_b200_device_sm_count(void) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return FRISK_ERR_NO_DEVICE;
  }
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    cudaGetLastError();
    return FRISK_ERR_CUDA;
  }
  return n;
}

const char* frisk_b200_version(void) { return "frisk_b200 0.1 (sm_100a)"; }

}  // extern "C"
