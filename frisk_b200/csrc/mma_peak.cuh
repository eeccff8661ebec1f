// Measurement of the tensor pipes' own rate: every SM (or SM pair) issues tcgen05.mma back to
// back on operand tiles that already sit in shared memory -- no loads, no epilogue.  What this
// kernel reaches is the ceiling for a GEMM of the same operand type, tile shape and duration on
// the same device; a GEMM kernel's tensor-pipe roofline is reported against it.
#pragma once
#include "gemm_tcgen05.cuh"

namespace frisk {

// A valid, ordinary number of the operand type from a hash of its index: random sign and
// mantissa, exponent near 1.  (All-zero or NaN operands draw less power than real data and
// would let the clock, and with it the measured rate, run higher than any GEMM sees.)
__device__ __forceinline__ uint32_t peak_hash(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352du; x ^= x >> 15; x *= 0x846ca68bu; x ^= x >> 16;
  return x;
}

template <int kPair>
__global__ void __launch_bounds__(128, 1)
mma_peak_kernel(uint32_t k_blocks, uint32_t idesc, uint32_t kind /* 0 f16, 1 f8f6f4, 2 tf32 */,
                uint32_t elem_bytes, int32_t* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_done[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ uint32_t abort_word;
  constexpr uint32_t kStages = 4;
  constexpr uint32_t kABytes = 128u * 128u;                  // 128 rows x 128 bytes of K
  constexpr uint32_t kBBytes = (kPair ? 128u : 256u) * 128u; // this CTA's share of 256 columns
  constexpr uint32_t kStageBytes = kABytes + kBBytes;
  const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const uint32_t rank = kPair ? __shfl_sync(0xffffffffu, ptx::cluster_ctarank(), 0) : 0u;
  const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  volatile uint32_t* abort_flag = &abort_word;
  uint8_t* tiles = smem_raw + (base - ptx::smem_u32(smem_raw));

  // operand tiles: 32-bit words of valid numbers of the type
  for (uint32_t i = threadIdx.x; i < kStages * kStageBytes / 4; i += blockDim.x) {
    const uint32_t h = peak_hash(i * 2654435761u + blockIdx.x);
    uint32_t w;
    if (elem_bytes == 4) {  // one fp32 with a tf32 mantissa: 0.5 .. 1, any sign
      w = (h & 0x807FE000u) | 0x3F000000u;
    } else if (elem_bytes == 2) {  // two 16-bit floats, exponent field near the bias, any sign / mantissa
      w = (h & 0x807F807Fu) | 0x3F003F00u;   // valid as bf16 (about 0.5 .. 1) and as fp16 (about 1.75)
    } else {                // four e4m3: exponent 6 .. 7, any sign / mantissa
      w = (h & 0x87878787u) | 0x30303030u;
    }
    reinterpret_cast<uint32_t*>(tiles)[i] = w;
  }
  if (threadIdx.x == 0) {
    abort_word = 0;
    ptx::mbar_init(ptx::smem_u32(&bar_done[0]), 1);
    ptx::mbar_init(ptx::smem_u32(&bar_done[1]), 1);
    ptx::fence_mbar_init();
  }
  ptx::fence_proxy_async_smem();   // the tensor pipe reads shared memory through the async proxy
  if (warp == 0) {
    if (kPair) { ptx::tmem_alloc_pair(ptx::smem_u32(&tmem_base_slot), 512); ptx::tmem_relinquish_pair(); }
    else { ptx::tmem_alloc(ptx::smem_u32(&tmem_base_slot), 512); ptx::tmem_relinquish(); }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (kPair) { ptx::cluster_arrive(); ptx::cluster_wait(); }
  ptx::tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_base_slot, 0);

  if (warp == 0 && rank == 0) {
    // K-major operands in the 128-byte swizzle: SBO = 1024, one K step = 32 bytes
    uint64_t desc = 0;
    desc |= (uint64_t)1 << 16;
    desc |= (uint64_t)(1024 >> 4) << 32;
    desc |= (uint64_t)1 << 46;
    desc |= (uint64_t)2 << 61;
    const uint32_t done0 = ptx::smem_u32(&bar_done[0]);
    bool ok = true;
    uint32_t batches = 0;
    for (uint32_t kb = 0; ok && kb < k_blocks; ++kb) {
      const uint32_t st = kb & (kStages - 1u);
      const uint32_t a_addr = base + st * kStageBytes, b_addr = a_addr + kABytes;
      const uint64_t ad = desc | (uint64_t)((a_addr & 0x3FFFFu) >> 4);
      const uint64_t bd = desc | (uint64_t)((b_addr & 0x3FFFFu) >> 4);
      const uint32_t d = tmem_base + ((kb >> 6) & 1u) * 256u;   // two accumulators, 64 k-blocks each
#pragma unroll
      for (uint32_t ks = 0; ks < 4; ++ks) {
        const uint32_t accumulate = ((kb & 63u) | ks) ? 1u : 0u;
        if (kind == 2u) {
          if (kPair) { if (ptx::elect_one()) ptx::mma_tf32_pair(d, ad + 2 * ks, bd + 2 * ks, idesc, accumulate); }
          else { if (ptx::elect_one()) ptx::mma_tf32(d, ad + 2 * ks, bd + 2 * ks, idesc, accumulate); }
        } else if (kind == 1u) {
          if (kPair) { if (ptx::elect_one()) ptx::mma_f8_pair(d, ad + 2 * ks, bd + 2 * ks, idesc, accumulate); }
          else { if (ptx::elect_one()) ptx::mma_f8(d, ad + 2 * ks, bd + 2 * ks, idesc, accumulate); }
        } else {
          if (kPair) { if (ptx::elect_one()) ptx::mma_f16_pair(d, ad + 2 * ks, bd + 2 * ks, idesc, accumulate); }
          else { if (ptx::elect_one()) ptx::mma_f16(d, ad + 2 * ks, bd + 2 * ks, idesc, accumulate); }
        }
      }
      // every 32 k-blocks: mark this point, then wait (bounded) for the mark before it, so the
      // queue of issued work stays short without the pipe ever running dry
      if ((kb & 31u) == 31u) {
        const uint32_t b = batches & 1u;
        if (kPair) { if (ptx::elect_one()) ptx::tc_commit_pair(done0 + 8 * b); }
        else { if (ptx::elect_one()) ptx::tc_commit(done0 + 8 * b); }
        if (batches > 0)
          ok = bounded_wait(done0 + 8 * (b ^ 1u), ((batches - 1u) >> 1) & 1u, abort_flag, status,
                            kStatusTestTimeout);
        ++batches;
      }
      __syncwarp();
    }
    // drain: the last mark issued (k_blocks is a multiple of 32)
    if (ok && batches > 0)
      ok = bounded_wait(done0 + 8 * ((batches - 1u) & 1u), ((batches - 1u) >> 1) & 1u, abort_flag,
                        status, kStatusTestTimeout);
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (kPair) { ptx::cluster_arrive(); ptx::cluster_wait(); }
  if (warp == 0) {
    ptx::tc_fence_after();
    if (kPair) ptx::tmem_dealloc_pair(tmem_base, 512);
    else ptx::tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace frisk
