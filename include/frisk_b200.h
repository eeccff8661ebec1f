/*
 * frisk_b200.h -- C ABI of libfrisk_b200.so, the execution back end for `frisk.gemm`.
 *
 * The reference (Xiebaokang/frisk) can build a `frisk.gemm` op but has no way to run it:
 * there is no lowering, kernel or runtime below its pybind11 IR builder.  This library is
 * what a binding of that builder calls to execute the op on an NVIDIA B200 (sm_100a).
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns 0 or a negative
 * FRISK_ERR_* code and never throws.  Unless stated otherwise, matrix pointers are DEVICE
 * pointers owned by the caller.  A plan is bound to the CUDA device that was current when it
 * was created and may be used from one host thread at a time.
 *
 * Operand convention (the one the reference's builder enforces, ffi/ir.cpp:339-359):
 *   A is a logical [M,K] matrix, B a logical [K,N] matrix, C a logical [M,N] matrix,
 *   whatever the trans flags say.  The trans flags select the memory order of the buffer
 *   (lib/Dialect/Frisk/IR/FriskOps.cpp:1359-1360 and 1376-1377 derive "K is the inner
 *   dimension" as !transA for A and transB for B):
 *     transA == 0 : A[m,k] at  A + m*lda + k      (K contiguous)
 *     transA == 1 : A[m,k] at  A + k*lda + m      (M contiguous)
 *     transB == 0 : B[k,n] at  B + k*ldb + n      (N contiguous)
 *     transB == 1 : B[k,n] at  B + n*ldb + k      (K contiguous, "column-major B")
 *   C[m,n] at C + m*ldc + n always.
 * Semantics (include/Dialect/Frisk/IR/FriskOps.td:248-289):
 *   C = (clear_accum ? 0 : C) + scale_a[m] * scale_b[n] * sum_k A[m,k] * B[k,n]
 * with the products and the sum in fp32 and one round-to-nearest-even cast to C's type.
 * The scales are an addition to the reference op (it has no fp8 GEMM); they are optional.
 */
#ifndef FRISK_B200_H_
#define FRISK_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------- */
enum {
  FRISK_OK = 0,
  FRISK_ERR_INVALID_ARGUMENT = -1, /* NULL pointer, non-positive size, bad enum            */
  FRISK_ERR_UNSUPPORTED = -2,      /* dtype / layout combination no kernel covers          */
  FRISK_ERR_MISALIGNED = -3,       /* pointer or leading dimension breaks an alignment rule */
  FRISK_ERR_WORKSPACE = -4,        /* workspace missing or smaller than workspace_bytes     */
  FRISK_ERR_CUDA = -5,             /* a CUDA runtime/driver call failed (see last_error)    */
  FRISK_ERR_DEVICE_TIMEOUT = -6,   /* a bounded device-side wait ran out (status word)      */
  FRISK_ERR_NO_DEVICE = -7,        /* no sm_100 device is visible                           */
  FRISK_ERR_SHARD = -8,            /* rank/nranks invalid for row sharding                  */
  FRISK_ERR_TOO_LARGE = -9         /* problem exceeds a fixed capacity of the entry point    */
};

/* ---- element types: the dtype vocabulary of ffi/ir.cpp:163-175, 240-245, 410-423 ----- */
typedef enum {
  FRISK_DT_F32 = 0,
  FRISK_DT_F16 = 1,
  FRISK_DT_BF16 = 2,
  FRISK_DT_E4M3 = 3, /* "e4m3fn": finite-only fp8, max 448, no inf */
  FRISK_DT_E5M2 = 4  /* "e5m2": fp8 with fp16's exponent (the top byte of an fp16), max 57344;
                        inputs of a gemm only, like e4m3 (the reference names both as buffer
                        element types: ffi/ir.cpp:411-414, 454-457)                      */
} frisk_dtype;

typedef enum { FRISK_SCALE_NONE = 0, FRISK_SCALE_ROW_COL = 1 } frisk_scale_mode;

/* Which kernel family a plan resolved to (reported by frisk_b200_gemm_plan_info). */
typedef enum {
  FRISK_KERNEL_SIMT = 0,    /* CUDA-core fp32-FMA tiles: small fp32 problems, every odd shape */
  FRISK_KERNEL_TCGEN05 = 1, /* TMA + tcgen05.mma, accumulators in TMEM, whole-tile output   */
  FRISK_KERNEL_SKINNY = 2,  /* few rows (M <= 128): operands swapped, K split over a cluster / SMs */
  FRISK_KERNEL_TCGEN05_PAIR = 3, /* CTA pairs with two-SM MMAs on 256 x tile_n output tiles  */
  FRISK_KERNEL_TF32X3 = 4   /* fp32 inputs and C: A and B split into tf32 hi + lo parts in the
                               workspace, three products in one tensor-core GEMM (fp32-level
                               accuracy: relative error about 1e-6); larger problems only      */
} frisk_kernel_kind;

/*
 * Description of one `frisk.gemm`.  Mirrors the op's attributes
 * (include/Dialect/Frisk/IR/FriskOps.td:256-262: transA, transB, M, N, K, clear_accum) plus
 * what the memref types carry (element types) and what an executor needs (leading dimensions).
 * lda/ldb/ldc are in ELEMENTS; 0 means "packed" (the natural value for the chosen order).
 */
typedef struct frisk_gemm_desc {
  int64_t M, N, K;
  int32_t a_type, b_type, c_type; /* frisk_dtype; a_type must equal b_type                  */
  int64_t lda, ldb, ldc;
  int32_t transA, transB;
  int32_t clear_accum; /* 1: C = A*B ; 0: C += A*B                                          */
  int32_t scale_mode;  /* frisk_scale_mode                                                  */
  /* Tuning overrides; 0 = let the plan choose.                                             */
  int32_t force_kernel; /* 1 + frisk_kernel_kind, or 0                                       */
  int32_t tile_n;       /* tcgen05 tile width along N: 64, 128 or 256                        */
  int32_t stages;       /* TMA pipeline depth                                                */
  int32_t num_ctas;     /* persistent grid size                                              */
  int32_t band_tiles;   /* tile rows walked together by the rasterisation (L2 reuse)         */
  int32_t epilogue;     /* whole-tile tensor-core plans (0: staged as in 2, or as in 4 on a CTA-pair
                           plan whose K has at most 32 k-blocks or whose pairs have one tile each): 1 = every thread stores its own row
                           pieces, 2 = rows staged through shared memory and stored as 128-byte
                           pieces (a C without 16-byte aligned rows is stored element-wise
                           either way), 3 = as 2 with linear instead of swizzled staging rows:
                           same results, shared-memory bank conflicts on every staging write
                           (kept so that the swizzle's effect can be measured), 4 = rows
                           staged as in 2 and stored by TMA tensor stores, one instruction per
                           32 x 128-byte piece and destination (CTA-pair plans with 16-byte
                           aligned C rows; other plans take it as 2)                            */
  /* A frisk.reduce of C over its columns (dim 1), folded inside the GEMM's epilogue (a small
   * second launch folds the per-tile results) instead of a second pass over C.  The reference's
   * sketches reduce the accumulator of a gemm this way: tmp/ir.mlir:116, 135.
   * row_reduce = 1 + frisk_reduce_kind, 0 = none.  The fold sees the
   * values of C as stored (after the cast), so it equals frisk_b200_reduce_run on the finished C
   * for min and max and differs from it only in summation order for add and mul.  The result,
   * [M] of C's element type, goes to frisk_gemm_run_args.row_reduce_dst.                      */
  int32_t row_reduce;
  int32_t row_reduce_clear; /* 1: dst = fold, 0: dst = dst (op) fold (the op's `clear`)        */
  /* More tuning overrides of the CTA-pair kernel; 0 = let the plan choose.                     */
  int32_t panel_tiles;  /* > 0: walk the tiles in panels of this many tile columns (the panel
                           of B stays in L2 while A streams past) instead of bands of rows      */
  int32_t l2_hints;     /* bit 0: loads of A evict-first in L2; bit 1: loads of B evict-last    */
  int32_t k_split;      /* the K-split forms of an unswapped problem with few tiles of C and a
                           long K: 0 = where the plan expects one to pay, -1 = never,
                           1 = a cluster per tile (or stream-K) whenever that form exists,
                           2 = K planes whenever they exist (CTA-pair kernel, one work item per
                           tile and K part, fp32 partial tiles in the workspace, summed into C
                           by a second launch; plan_info: kernel tcgen05_pair, split_k = 1,
                           launches = 2),
                           3 = K split over the CTA pairs of a cluster whenever such a plan exists
                           (256 x 128 tiles, two or four pairs per tile, partials folded through
                           distributed shared memory; kernel tcgen05_pair, split_k = 1, one
                           launch, no workspace)                                                */
} frisk_gemm_desc;

typedef struct frisk_gemm_plan frisk_gemm_plan; /* opaque */

typedef struct frisk_gemm_plan_info {
  int32_t kernel;      /* frisk_kernel_kind                                                 */
  int32_t tile_m, tile_n, tile_k;
  int32_t stages;
  int32_t num_ctas;
  int32_t swap_ab;     /* 1 when the weights feed the 128-row operand (skinny path)          */
  int32_t split_k;     /* 1 when several CTAs share a tile's K range: the few-row plan, and
                          FRISK_KERNEL_TCGEN05 / FRISK_KERNEL_TCGEN05_PAIR (K planes) plans for
                          a few tiles against a long K                                        */
  int32_t smem_bytes;  /* dynamic shared memory per CTA                                      */
  int32_t launches;    /* kernels launched per run                                           */
  int32_t swizzle_a, swizzle_b; /* TMA/UMMA swizzle width in bytes (0, 32, 64, 128)          */
  int32_t cuda_core_reason; /* FRISK_TC_*: why a plan resolved to FRISK_KERNEL_SIMT (0 if not) */
  int64_t cuda_core_runs;   /* runs of a tensor-core plan that took the CUDA-core kernel
                               because A or B was not 16-byte aligned (about 100x slower)     */
} frisk_gemm_plan_info;

/* Why a problem cannot run on the tensor-core kernels (frisk_gemm_plan_info.cuda_core_reason). */
enum {
  FRISK_TC_OK = 0,
  FRISK_TC_INPUT_TYPE = 1, /* A and B are not fp16, bf16 or e4m3                              */
  FRISK_TC_PITCH = 2,      /* a row pitch of A or B is not a multiple of 16 bytes (TMA rule)   */
  FRISK_TC_EXTENT = 3,     /* M, N or K is 2^31 or more                                        */
  FRISK_TC_FP8_ORDER = 4,  /* e4m3 operands are taken K-inner only (transA = 0, transB = 1)    */
  FRISK_TC_FORCED = 5      /* desc.force_kernel asked for the CUDA-core kernel                 */
};

/* Replaces: nothing executable in the reference.  The closest reference interface is
 * builder.create_gemm_op (ffi/ir.cpp:322-366), whose shape and dtype checks are repeated here:
 * rank-2 static shapes, matching inner dimensions, one element type for A and B.           */
int frisk_b200_gemm_plan_create(const frisk_gemm_desc* desc, frisk_gemm_plan** out);
void frisk_b200_gemm_plan_destroy(frisk_gemm_plan* plan);
int frisk_b200_gemm_plan_info(const frisk_gemm_plan* plan, frisk_gemm_plan_info* out);

/* Bytes of device scratch `run` needs.  0 for every plan but the stream-K forms of the K-split
 * plans (shapes whose tiles cannot be covered by thread-block clusters), plans with a fused row
 * reduce (one fp32 per row and half tile), K-planes plans (one fp32 copy of C per K part, at
 * most 20 MB), 3xTF32 plans (twice the bytes of A and B; 256-byte
 * aligned) and plans for an A or B whose row pitch is not a multiple of 16 bytes (a copy of that
 * operand at a padded pitch, made by one more launch before every run); `run` takes a NULL
 * workspace when it is 0. */
int frisk_b200_gemm_workspace_bytes(const frisk_gemm_plan* plan, size_t* out);

/*
 * Launch the GEMM on `stream` (a cudaStream_t passed as void*; NULL = the default stream).
 * Asynchronous and stream-ordered.  scale_a ([M] fp32) and scale_b ([N] fp32) are used only
 * when desc.scale_mode == FRISK_SCALE_ROW_COL.  `device_status` may be NULL; otherwise it
 * points to one int32 in device memory that a kernel ORs a non-zero code into when one of its
 * bounded waits ran out (read it with frisk_b200_check_status after synchronising).  With a NULL
 * device_status a wait that runs out is not reported at all: the kernel returns and C is left
 * partly written.
 * `workspace` (see frisk_b200_gemm_workspace_bytes) is scratch: it need not keep its contents
 * between runs and may be shared by plans whose runs do not overlap on the GPU.
 * The executor behind the op created by ffi/ir.cpp:362.
 */
int frisk_b200_gemm_run(frisk_gemm_plan* plan, const void* A, const void* B, void* C,
                        const float* scale_a, const float* scale_b, void* workspace,
                        size_t workspace_bytes, int32_t* device_status, void* stream);

/*
 * frisk_b200_gemm_run with every argument in one struct, plus the two things the plain call has
 * no room for: the destination of a fused row reduce, and copies of C for other GPUs.
 *
 * peer_c: the row-sharded GEMM (frisk_b200_shard_rows) with the all-gather of C folded into the
 * kernel.  Entry q points, in the memory of another GPU of the node (a peer-mapped pointer:
 * frisk_b200_peer_open, or any pointer this device can store to), to where THIS rank's rows
 * start in that GPU's copy of the whole C; same element type and ldc as C.  The epilogue stores
 * every tile to C and to each peer copy with ordinary global stores -- nothing is loaded from a
 * peer.  The caller orders the ranks: every peer buffer must be allocated before the launch,
 * and a rank may read its copy only after all ranks' launches have completed (a barrier after
 * synchronising the stream).  Whole-tile tensor-core plans only; at most 7 peers.
 */
typedef struct frisk_gemm_run_args {
  const void* A;
  const void* B;
  void* C;
  const float* scale_a;
  const float* scale_b;
  void* workspace;
  size_t workspace_bytes;
  int32_t* device_status;
  void* stream;
  void* row_reduce_dst; /* needed iff desc.row_reduce != 0                                    */
  int32_t n_peers;
  void* peer_c[7];
} frisk_gemm_run_args;
int frisk_b200_gemm_run_ex(frisk_gemm_plan* plan, const frisk_gemm_run_args* args);

/*
 * Device buffers another process of the node can store into (one process per GPU): peer_alloc
 * allocates `bytes` on the current device and fills a 64-byte handle to send to the other
 * processes (any byte transport); peer_open maps the buffer behind a handle received from another
 * process into this one and enables peer access.  Thin wrappers of cudaMalloc / cudaIpcGetMemHandle
 * / cudaIpcOpenMemHandle / cudaIpcCloseMemHandle / cudaFree.  No counterpart in the reference.
 */
int frisk_b200_peer_alloc(size_t bytes, void** ptr, unsigned char handle[64]);
int frisk_b200_peer_open(const unsigned char handle[64], void** ptr);
int frisk_b200_peer_close(void* ptr);
int frisk_b200_peer_free(void* ptr);

/*
 * The same GEMM for callers that hold HOST buffers (what a binding of the reference's Python
 * builder would be handed: numpy arrays).  Copies A, B (and C when clear_accum == 0, and the
 * scales) to the device, runs, copies C back and synchronises.  With 4096 or more rows of a
 * row-major A the rows go through in up to 16 chunks on three streams, so the upload of one chunk,
 * the GEMM of the previous and the download of the one before overlap.  Device buffers are
 * cached in the plan between calls.  Returns FRISK_ERR_DEVICE_TIMEOUT if the status word came back set.
 * Only the elements of each stored row are read and written, so a host buffer may end after the
 * last row's elements: (rows - 1) * ld + row length elements are enough.
 */
int frisk_b200_gemm_run_host(frisk_gemm_plan* plan, const void* A, const void* B, void* C,
                             const float* scale_a, const float* scale_b);
/* The same for a plan with a fused row reduce (desc.row_reduce != 0): `row_reduce_dst` is the
 * host array of M elements of C's type the fold goes to (and comes from, when clear is 0). */
int frisk_b200_gemm_run_host_ex(frisk_gemm_plan* plan, const void* A, const void* B, void* C,
                                const float* scale_a, const float* scale_b, void* row_reduce_dst);

/*
 * No counterpart in the reference.  The few-row ("skinny") GEMM for callers that may not
 * allocate device memory: code running inside someone else's memory pool, services with a
 * memory budget fixed at start-up, replays of pre-recorded work.  It always uses the K-split
 * form that adds partial sums into an M x N fp32 scratch, and that scratch is a fixed 4 MiB array
 * inside the library image (held by every GPU that loads the library until the process exits),
 * so the call allocates nothing on the device or the host.
 *   - Accepts what the skinny plan accepts: fp16 / bf16 / e4m3 inputs, M <= 64, N >= 256,
 *     transA == 0, 16-byte aligned A and B with 16-byte row pitches; anything else returns
 *     FRISK_ERR_UNSUPPORTED or FRISK_ERR_MISALIGNED.
 *   - M * N must not exceed frisk_b200_gemm_skinny_static_capacity() (1,048,576 outputs);
 *     larger problems return FRISK_ERR_TOO_LARGE (text in frisk_b200_last_error()).
 *   - The first call on a device looks up the array's device address (the device must be
 *     current); make that first call before starting any stream capture.
 *   - All calls share the one array and each clears the part it uses first, so calls that
 *     overlap on the GPU (different streams, different threads) race: serialise them.
 * A, B, C, the scales and device_status are the caller's device buffers, as for
 * frisk_b200_gemm_run; the call is asynchronous on `stream`.
 */
int frisk_b200_gemm_skinny_static(const frisk_gemm_desc* desc, const void* A, const void* B,
                                  void* C, const float* scale_a, const float* scale_b,
                                  int32_t* device_status, void* stream);
size_t frisk_b200_gemm_skinny_static_capacity(void);

/* Copies the status word to the host (synchronises `stream`) and maps it to a return code. */
int frisk_b200_check_status(const int32_t* device_status, void* stream);

const char* frisk_b200_strerror(int code);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char* frisk_b200_last_error(void);

/*
 * Row-block sharding of C = A*B over `nranks` GPUs: rank r owns rows [row0, row0+rows) of A
 * and C, B is replicated.  Rows are dealt in contiguous blocks; when M is not a multiple of
 * nranks the first M % nranks ranks get one extra row.  No counterpart in the reference,
 * which has no multi-device notion (its only "parallel" is the intra-kernel frisk.parallel,
 * include/Dialect/Frisk/IR/FriskOps.td:81-140).
 */
int frisk_b200_shard_rows(int64_t M, int nranks, int rank, int64_t* row0, int64_t* rows);

/* ---- frisk.reduce on whole buffers ------------------------------------------------------ */
/*
 * frisk.reduce (include/Dialect/Frisk/IR/FriskOps.td:413-443; builder ffi/ir.cpp:469-471):
 * `dst = (clear ? identity : dst) (op) reduce_op over dimension `dim` of src`, kind "add", "mul",
 * "min" or "max" (verifier, lib/Dialect/Frisk/IR/FriskOps.cpp:1734-1767: the destination has the
 * source's shape without `dim` and the same element type).  The reference has no lowering for
 * it; the sketches it is written for are row maxima and row sums of an online softmax
 * (tmp/ir.mlir:21-78).  A row-major source of any rank is [outer, extent, inner] around the
 * reduced dimension, the destination [outer, inner].  Arithmetic: elements decoded to fp32, fp32
 * accumulation (a fixed order: the same result on every run), one round-to-nearest-even cast at
 * the end; min and max are exact and skip NaN operands (fminf / fmaxf from the identity: a line
 * of nothing but NaN, like an empty one, gives +inf for min and -inf for max).
 */
typedef enum {
  FRISK_REDUCE_ADD = 0,
  FRISK_REDUCE_MUL = 1,
  FRISK_REDUCE_MIN = 2,
  FRISK_REDUCE_MAX = 3
} frisk_reduce_kind;

typedef struct frisk_reduce_desc {
  int64_t outer, extent, inner; /* product of the dimensions before / at / after `dim`       */
  int32_t dtype;                /* FRISK_DT_F32, _F16 or _BF16, for src and dst              */
  int32_t kind;                 /* frisk_reduce_kind                                         */
  int32_t clear;                /* 1: dst is overwritten; 0: dst is folded into the result   */
  int32_t device;               /* CUDA ordinal, -1 = current                                */
} frisk_reduce_desc;

typedef struct frisk_reduce_info {
  int32_t lines;       /* 1: the reduced dimension is the innermost one (a warp per line)    */
  int32_t vector;      /* elements per 16-byte load along the contiguous dimension, or 1     */
  int32_t chunks;      /* pieces the reduced dimension is cut into (> 1: two launches)       */
  int32_t launches;
  int64_t chunk_len;
  int64_t ctas;        /* grid of the first launch                                           */
  size_t workspace_bytes;
} frisk_reduce_info;

/* How the library would run `desc` for operands at addresses with the given alignment
 * (`src_align16` = 1 when src is 16-byte aligned).  Host arithmetic; the cut into pieces depends on
 * how many CTAs the device holds at once, which is asked of the current device when there is one
 * and assumed to be 148 SMs x 6 CTAs otherwise. */
int frisk_b200_reduce_info(const frisk_reduce_desc* desc, int src_align16, frisk_reduce_info* out);
/* Bytes of device workspace frisk_b200_reduce_run needs (0 for most shapes). */
int frisk_b200_reduce_workspace_bytes(const frisk_reduce_desc* desc, size_t* out);
/*
 * Stream-ordered, asynchronous.  src, dst, workspace are device pointers aligned to the element
 * size (16-byte alignment enables vector loads; any extent and inner size is accepted).
 * Returns FRISK_ERR_WORKSPACE if ws_bytes is below frisk_b200_reduce_workspace_bytes.
 */
int frisk_b200_reduce_run(const frisk_reduce_desc* desc, const void* src, void* dst, void* workspace,
                          size_t ws_bytes, void* stream);
/* The same on HOST buffers: allocates, copies in, runs, copies dst back, synchronises. */
int frisk_b200_reduce_run_host(const frisk_reduce_desc* desc, const void* src, void* dst);

/* ---- layout mapping ------------------------------------------------------------------- */
/*
 * A shared-memory operand layout as the reference's GemmOp::inferLayout chooses it
 * (lib/Dialect/Frisk/IR/FriskOps.cpp:589-618, buildHopperSharedLayout): a rows x cols tile of
 * `elem_bits`-wide elements, row-major, with `k_inner` telling whether the contiguous
 * dimension is the GEMM's K.
 */
typedef struct frisk_layout_desc {
  int64_t rows, cols;  /* tile shape as stored: cols is the contiguous dimension             */
  int32_t elem_bits;   /* 8, 16 or 32                                                        */
  int32_t k_inner;     /* 1: cols is K (K-major operand); 0: cols is M or N (MN-major)        */
} frisk_layout_desc;

/* What the B200 pipeline needs for that tile: TMA box + swizzle, UMMA descriptor fields. */
typedef struct frisk_tma_params {
  int32_t swizzle_bytes;     /* 0, 32, 64 or 128: CU_TENSOR_MAP_SWIZZLE_{NONE,32B,64B,128B}   */
  int32_t box_inner;         /* elements per box row (= swizzle_bytes / element size)         */
  int32_t box_outer;         /* rows per box                                                  */
  int32_t num_boxes;         /* boxes that make up the tile                                   */
  int32_t umma_layout_type;  /* bits 61..63 of the shared-memory descriptor: 0, 6, 4, 2        */
  int32_t umma_major;        /* 0 = K-major, 1 = MN-major (instruction-descriptor bit)        */
  int32_t leading_byte_offset; /* LBO in bytes                                                */
  int32_t stride_byte_offset;  /* SBO in bytes                                                */
  int32_t k_step_bytes;      /* start-address advance per UMMA K step (32 bytes of K)          */
  char reference_layout[24]; /* name of the reference swizzle: "full_bank", "half_bank", ...   */
} frisk_tma_params;

/* The selection rule of FriskOps.cpp:608-617 carried over to TMA / UMMA descriptors. */
int frisk_b200_layout_to_tma(const frisk_layout_desc* layout, frisk_tma_params* out);

/*
 * What a tensor-core plan stages per pipeline stage for its two operands (operand 0: the one
 * that feeds the 128 UMMA rows, 1: the one that feeds the UMMA N columns; for a few-row plan the
 * weights are operand 0).  `layout` is frisk_b200_layout_to_tma's answer for the staged tile --
 * the plan fills its TMA boxes and UMMA descriptors from it and from nothing else --,
 * `umma_desc_base` the 64-bit shared-memory descriptor the kernel adds start addresses to
 * (bits 16..29 LBO / 16, 32..45 SBO / 16, 46 the sm_100 version, 61..63 the swizzle), and
 * `tma_boxes_per_stage` how many copies fill the operand's part of a stage.  Any output
 * pointer may be NULL.  FRISK_ERR_UNSUPPORTED for a CUDA-core plan.
 */
int frisk_b200_gemm_plan_operand_layout(const frisk_gemm_plan* plan, int32_t operand,
                                        frisk_tma_params* layout, uint64_t* umma_desc_base,
                                        int32_t* tma_boxes_per_stage);

/*
 * Byte offset inside a swizzled rows x cols tile of element (row, col), as TMA writes it and
 * UMMA reads it (-1 on a bad argument).  The reference's makeFull/Half/QuarterBankSwizzle
 * (FriskOps.cpp:500-558) return (column atom tc, row atom ts, offset in atom) and never
 * linearise them; here the three are laid out as
 *   tc * (rows * span) + ts * (8 * span) + offset * elem_bytes,   span = swizzle_bytes,
 * i.e. one TMA box per column atom.
 */
int64_t frisk_b200_swizzled_offset(int64_t row, int64_t col, int64_t rows, int64_t cols,
                                   int32_t elem_bits, int32_t swizzle_bytes);

/*
 * Shared-memory bank-conflict model of exp/layout/gemm_layout_tool.cpp:135-208 applied to a
 * swizzle mode: walks the tile in windows of 32*lane_vector row-major elements, maps every
 * element to its bank (4-byte words, 32 banks) and reports the worst bucket per window.
 * `mode` is swizzle_bytes (0/32/64/128) or one of the Blackwell-only atoms below.
 */
enum { FRISK_SWIZZLE_128B_ATOM_32B = 1032, FRISK_SWIZZLE_128B_ATOM_64B = 1064 };
typedef struct frisk_bank_stats {
  double avg_max_conflict;
  int32_t max_conflict;
  int32_t samples;
} frisk_bank_stats;
int frisk_b200_bank_conflicts(int64_t rows, int64_t cols, int32_t elem_bits, int32_t mode,
                              int32_t lane_vector, int32_t distinct_words_only,
                              frisk_bank_stats* out);

/*
 * The access patterns the reference's model does not walk.  Its windows are 32 * lane_vector
 * consecutive ROW-MAJOR elements (gemm_layout_tool.cpp:150-176; `--ldmatrix` only widens the
 * lane vector, 407-409), which every layout with 128-byte rows serves without conflicts,
 * swizzled or not -- so it cannot tell the modes apart.  What a swizzle is for is the other
 * direction:
 *   FRISK_ACCESS_CHUNK_COLUMN  every lane a different row, all lanes the same 16-byte chunk
 *                              column: the operand fetch of ldmatrix / UMMA (8 rows x 16 bytes
 *                              per matrix) and the writes of an epilogue that stages one row per
 *                              thread;
 *   FRISK_ACCESS_ROW_PIECES    consecutive lanes walk the 16-byte chunks of a row, then the next
 *                              row: the coalesced read-back of staged rows.
 * The tile is laid out as frisk_b200_swizzled_offset lays it out (mode 0: plain rows of
 * cols * elem_bytes).  16-byte accesses are served a quarter warp at a time; `wavefronts` counts,
 * per quarter, the most distinct 4-byte words any bank has to deliver.  conflict_degree =
 * wavefronts / ideal_wavefronts: 1.0 means conflict-free.  tma_boxes / global_segment_bytes are
 * what the mode costs outside shared memory: copies to issue per tile, contiguous bytes per
 * box row in global memory.
 */
enum { FRISK_ACCESS_CHUNK_COLUMN = 1, FRISK_ACCESS_ROW_PIECES = 2 };
typedef struct frisk_access_stats {
  int64_t requests;          /* warp-wide requests of up to 32 x 16 bytes                      */
  int64_t wavefronts;        /* passes over the banks all requests took                        */
  int64_t ideal_wavefronts;  /* one per quarter warp                                           */
  double conflict_degree;
  int32_t max_wavefronts_per_request;
  int32_t tma_boxes;
  int32_t global_segment_bytes;
} frisk_access_stats;
int frisk_b200_bank_conflicts_access(int64_t rows, int64_t cols, int32_t elem_bits, int32_t mode,
                                     int32_t access, frisk_access_stats* out);

/*
 * Measures, on the current device, the rate the tensor pipes reach when every SM (pair = 0) or
 * SM pair (pair = 1: two-SM MMAs, M = 256) issues tcgen05.mma of shape M x 256 x 32 bytes of K
 * back to back on operand tiles resident in shared memory: no loads, no epilogue.  It is the
 * denominator of a GEMM kernel's tensor-pipe roofline for operand types no library peak was
 * measured for (e4m3; FRISK_DT_F32 is measured as kind::tf32, the rate behind the 3xTF32 plan).  `k_blocks` (a multiple of 32; one k-block = four MMAs) sets the length
 * of one launch -- choose it so that a launch lasts about as long as the GEMM it is compared
 * with, since the clock under the power cap depends on it; `reps` launches are timed with CUDA
 * events on the default stream.  Synchronous.  No counterpart in the reference, whose timing
 * method (exp/layout/analyze_bank_conflicts.py:112-178) has no roofline.
 */
int frisk_b200_measure_mma_peak(int32_t ab_type, int32_t pair, int32_t k_blocks, int32_t reps,
                                double* tflops, double* ms_per_launch);

/* Library / device facts: returns the SM count of the current device (or a negative code). */
int frisk_b200_device_sm_count(void);
const char* frisk_b200_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FRISK_B200_H_ */
