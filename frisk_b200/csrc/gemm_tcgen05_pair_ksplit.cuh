// The CTA-pair GEMM of gemm_tcgen05_pair.cuh with K split inside a thread-block cluster, for
// problems whose 256 x 128 tiles number at most a quarter of the SMs: a cluster of 2 S CTAs
// (S = 2 or 4 pairs) owns one tile, pair q multiplies K part q with two-SM MMAs, and the S
// partial tiles meet through distributed shared memory as in the few-row plan
// (gemm_tcgen05.cuh, split mode 3), but in rows: pair `row / (128 / S)` owns a row of its side's
// 128; a CTA keeps the rows its pair owns in tensor memory and sends the others, 16 bytes per
// remote store, to their owner on the same side; one cluster barrier; each owner adds the S - 1
// images to its own partial in pair order, applies the scales and `+= C`, casts and stores whole
// row pieces.  One launch, no workspace, a fixed summation order.
//
// Cluster rank r: pair q = r >> 1, side h = r & 1 (h = 0 leads its pair and issues its MMAs).
// The barriers of the pipeline are those of the pair kernel, addressed relative to r: the
// leader's `full` barriers at rank r & ~1, the other side's `empty` / `acc_full` at rank r ^ 1.
// Every thread of the cluster passes three cluster barriers: after the set-up, before the fold
// (all partials pushed), and at the tear-down.  Every other wait is bounded.
#pragma once
#include "gemm_tcgen05_pair.cuh"

namespace frisk {

template <typename TC>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_pair_ksplit_kernel(const __grid_constant__ CUtensorMap tmap_a,
                                const __grid_constant__ CUtensorMap tmap_b,
                                const __grid_constant__ GemmParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kMaxStages];
  __shared__ __align__(8) uint64_t bar_empty[kMaxStages];
  __shared__ __align__(8) uint64_t bar_acc_full;
  __shared__ uint32_t tmem_base_slot;
  __shared__ uint32_t abort_word;

  const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const uint32_t lane = threadIdx.x & 31;
  const uint32_t crank = __shfl_sync(0xffffffffu, ptx::cluster_ctarank(), 0);
  const uint32_t side = crank & 1u;     // 0: leader of its pair
  const uint32_t part = crank >> 1;     // which K part this pair multiplies
  const uint32_t parts = p.cluster_k;   // pairs per cluster (2 or 4)
  const uint32_t tile = blockIdx.x / (2u * parts);
  volatile uint32_t* abort_flag = &abort_word;

  const uint32_t tiles_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t full0 = ptx::smem_u32(&bar_full[0]);
  const uint32_t empty0 = ptx::smem_u32(&bar_empty[0]);
  const uint32_t acc_full0 = ptx::smem_u32(&bar_acc_full);
  const uint32_t leader_full0 = __shfl_sync(0xffffffffu, ptx::mapa(full0, crank & ~1u), 0);
  const uint32_t peer_empty0 = __shfl_sync(0xffffffffu, ptx::mapa(empty0, crank ^ 1u), 0);
  const uint32_t peer_acc_full0 = __shfl_sync(0xffffffffu, ptx::mapa(acc_full0, crank ^ 1u), 0);
  const uint32_t peer_abort = __shfl_sync(0xffffffffu, ptx::mapa(ptx::smem_u32(&abort_word), crank ^ 1u), 0);

  const uint32_t stages = p.stages;
  const uint32_t stage_bytes = p.stage_bytes;  // per CTA
  const uint32_t tile_n = p.tile_n;
  const uint32_t tmem_cols = p.tmem_cols;
  int32_t* const status = p.status;
  // this pair's k-blocks (the host leaves no part empty)
  const uint32_t kb0 = part * p.kb_per, kb1 = min(p.num_kb, kb0 + p.kb_per);
  uint32_t tr, tc;
  tile_coords(p.group_r, p.tiles_r, p.tiles_c, tile, tr, tc, p.group_c);
  // the region the other pairs' partials arrive in lies behind the stage buffers: S - 1 images of
  // [row of the share][tile_n + 4] fp32
  const uint32_t red_base = tiles_base + stages * stage_bytes;

  if (threadIdx.x == 0) {
    abort_word = 0;
    for (uint32_t s = 0; s < stages; ++s) {
      ptx::mbar_init(full0 + 8 * s, 2);  // one producer arrival per CTA of the pair
      ptx::mbar_init(empty0 + 8 * s, 1);
    }
    ptx::mbar_init(acc_full0, 1);
    ptx::fence_mbar_init();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    ptx::tmem_alloc_pair(ptx::smem_u32(&tmem_base_slot), tmem_cols);
    ptx::tmem_relinquish_pair();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_arrive();   // cluster barrier 1: every CTA's barriers exist
  ptx::cluster_wait();
  ptx::tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_base_slot, 0);
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------- TMA producers (every CTA)
    const uint32_t a_boxes = p.a.num_boxes, a_box_bytes = p.a.box_bytes, a_box_mn = p.a.box_mn;
    const uint32_t b_boxes = p.b.num_boxes, b_box_bytes = p.b.box_bytes, b_box_mn = p.b.box_mn;
    const uint32_t a_mn_major = p.a.mn_major, b_mn_major = p.b.mn_major;
    const uint32_t a_stage_bytes = p.a.stage_bytes;
    const uint32_t bk_elems = p.bk_elems;
    const uint32_t my_turn = warp == 0 ? 0u : 1u;
    const int32_t r0 = (int32_t)(tr * 256u + side * 128u);
    const int32_t c0 = (int32_t)(tc * tile_n + side * (tile_n >> 1));   // each side stages half of B
    uint32_t stage = 0, phase = 0, turn = 0;
    bool ok = true;
    for (uint32_t kb = kb0; kb < kb1; ++kb) {
      if (turn == my_turn) {
        ok = bounded_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, status, kStatusProducerTimeout,
                          kProducerBackoffNs);
        if (!ok) break;
        const uint32_t full = leader_full0 + 8 * stage;
        if (ptx::elect_one()) ptx::mbar_arrive_expect_tx_cluster(full, stage_bytes);
        const uint32_t a_dst = tiles_base + stage * stage_bytes;
        const uint32_t b_dst = a_dst + a_stage_bytes;
        const int32_t k0 = (int32_t)(kb * bk_elems);
        for (uint32_t bx = 0; bx < a_boxes; ++bx) {
          const int32_t mn = r0 + (int32_t)(bx * a_box_mn);
          const int32_t x = a_mn_major ? mn : k0, y = a_mn_major ? k0 : mn;
          if (ptx::elect_one()) ptx::tma_load_2d_pair(a_dst + bx * a_box_bytes, &tmap_a, full, x, y);
        }
        for (uint32_t bx = 0; bx < b_boxes; ++bx) {
          const int32_t mn = c0 + (int32_t)(bx * b_box_mn);
          const int32_t x = b_mn_major ? mn : k0, y = b_mn_major ? k0 : mn;
          if (ptx::elect_one()) ptx::tma_load_2d_pair(b_dst + bx * b_box_bytes, &tmap_b, full, x, y);
        }
        __syncwarp();
      }
      turn ^= 1u;
      if (++stage == stages) {
        stage = 0;
        phase ^= 1;
      }
    }
    if (!ok) {
      // tell the other side, then give copies in flight time to land
      if (ptx::elect_one()) ptx::st_shared_cluster_u32(peer_abort, 1);
      const long long t0 = clock64();
      while (clock64() - t0 < 100000ll) {
      }
    }
    __syncwarp();
    ptx::cluster_arrive();   // cluster barrier 2 (see the epilogue role)
    ptx::cluster_wait();
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (leaders only)
    if (side == 0) {
      const uint64_t a_desc_base = p.a.desc_base, b_desc_base = p.b.desc_base;
      const uint32_t a_k_step = p.a.k_step_bytes, b_k_step = p.b.k_step_bytes;
      const uint32_t a_stage_bytes = p.a.stage_bytes;
      const uint32_t idesc = p.idesc, kind_f8 = p.kind_f8;
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      uint32_t prev_stage = 0;
      bool have_prev = false;
      for (uint32_t kb = kb0; kb < kb1; ++kb) {
        ok = bounded_wait(full0 + 8 * stage, phase, abort_flag, status, kStatusMmaTimeout, 0);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t a_addr = tiles_base + stage * stage_bytes;
        const uint32_t b_addr = a_addr + a_stage_bytes;
        const uint64_t adesc0 = a_desc_base | (uint64_t)((a_addr & 0x3FFFFu) >> 4);
        const uint64_t bdesc0 = b_desc_base | (uint64_t)((b_addr & 0x3FFFFu) >> 4);
        const uint32_t first = kb > kb0 ? 1u : 0u;
#pragma unroll
        for (uint32_t ks = 0; ks < 4; ++ks) {
          const uint64_t bdesc = bdesc0 + (uint64_t)((ks * b_k_step) >> 4);
          const uint64_t adesc = adesc0 + (uint64_t)((ks * a_k_step) >> 4);
          const uint32_t accumulate = first | (ks > 0 ? 1u : 0u);
          if (kind_f8) {
            if (ptx::elect_one()) ptx::mma_f8_pair(tmem_base, adesc, bdesc, idesc, accumulate);
          } else {
            if (ptx::elect_one()) ptx::mma_f16_pair(tmem_base, adesc, bdesc, idesc, accumulate);
          }
          // a stage is released after the first MMA of the next k-block has been issued
          if (ks == 0 && have_prev) {
            if (ptx::elect_one()) ptx::tc_commit_pair(empty0 + 8 * prev_stage);
            if (ptx::elect_one()) ptx::tc_commit_pair(peer_empty0 + 8 * prev_stage);
          }
        }
        prev_stage = stage;
        have_prev = true;
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
      if (ok) {
        if (ptx::elect_one()) ptx::tc_commit_pair(acc_full0);
        if (ptx::elect_one()) ptx::tc_commit_pair(peer_acc_full0);
      } else if (ptx::elect_one()) {
        ptx::st_shared_cluster_u32(peer_abort, 1);
      }
    }
    __syncwarp();
    ptx::cluster_arrive();   // cluster barrier 2
    ptx::cluster_wait();
  } else {
    // ------------------------------------------------------------- epilogue (every CTA)
    // A warp's 32 accumulator rows (its TMEM lanes) belong to one owner pair.  Warps whose rows
    // this pair owns keep them in tensor memory; the others send theirs, 16 bytes per store, to
    // the owner on the same side of its pair: image `source pair` (owner left out) of the
    // owner's region, [row of the share][column] fp32 at a pitch of tile_n + 4 floats (rows of
    // one quarter-warp then start in different banks).
    const uint32_t quarter = warp & 3u;  // TMEM lanes 32 * quarter .. + 31 belong to this warp
    const uint32_t sh = 31u - __clz(parts);
    const uint32_t share = 128u >> sh;   // rows of this side's 128 that each pair owns (64 or 32)
    const uint32_t share_sh = 31u - __clz(share);
    const uint32_t r_local = quarter * 32u + lane;
    const uint32_t owner = r_local >> share_sh, rr = r_local - owner * share;
    const bool keeper = owner == part;   // warp-uniform
    const uint32_t row_pitch = (tile_n + 4u) * 4u;
    const uint32_t img_bytes = share * row_pitch;
    const uint32_t t_row = tmem_base + ((quarter * 32u) << 16);
    const bool ok = bounded_wait(acc_full0, 0, abort_flag, status, kStatusEpilogueTimeout,
                                 p.epilogue_backoff_ns);
    if (ok && !keeper) {
      ptx::tc_fence_after();
      const uint32_t slot = part < owner ? part : part - 1u;
      const uint32_t dst = ptx::mapa(red_base + slot * img_bytes + rr * row_pitch, 2u * owner + side);
      for (uint32_t cc = 0; cc < tile_n; cc += 32) {
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(t_row + cc, v);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 8; ++i)
          ptx::st_shared_cluster_v4(dst + (cc + 4u * i) * 4u, v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
      }
      ptx::tc_fence_before();
    } else if (!ok && lane == 0) {
      ptx::st_shared_cluster_u32(peer_abort, 1);
    }
    __syncwarp();
    // Cluster barrier 2.  Every warp of every CTA of the cluster passes it exactly once, whatever
    // happened in its role, so a CTA that gave up cannot strand the others.  After it every
    // partial has reached its owner and nobody writes another CTA's shared memory again.
    ptx::cluster_arrive();
    ptx::cluster_wait();
    if (ok && keeper && !*abort_flag) {
      ptx::tc_fence_after();
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
      const uint32_t row = tr * 256u + side * 128u + r_local;
      const uint32_t mine = red_base + rr * row_pitch;
      for (uint32_t cc = 0; cc < tile_n; cc += 32) {
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(t_row + cc, v);
        ptx::tmem_ld_wait();
        // own partial first, then the other pairs' images in pair order
        for (uint32_t slot = 0; slot + 1u < parts; ++slot) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 x = ptx::ld_shared_f32x4(mine + slot * img_bytes + (cc + 4u * i) * 4u);
            v[4 * i] = __float_as_uint(__uint_as_float(v[4 * i]) + x.x);
            v[4 * i + 1] = __float_as_uint(__uint_as_float(v[4 * i + 1]) + x.y);
            v[4 * i + 2] = __float_as_uint(__uint_as_float(v[4 * i + 2]) + x.z);
            v[4 * i + 3] = __float_as_uint(__uint_as_float(v[4 * i + 3]) + x.w);
          }
        }
        epilogue_store<TC, 32>(ep, row, tc * tile_n + cc, v);
      }
      ptx::tc_fence_before();
    }
  }

  // ---------------------------------------------------------------- tear-down
  // No CTA may exit (or free tensor memory) while another can still signal its barriers.
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_arrive();   // cluster barrier 3
  ptx::cluster_wait();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, tmem_cols);
  }
}

}  // namespace frisk
