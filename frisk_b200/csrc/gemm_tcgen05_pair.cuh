// The GEMM of gemm_tcgen05.cuh run by PAIRS of CTAs (a cluster of two, one CTA per SM of a TPC)
// with two-SM MMAs (tcgen05.mma.cta_group::2).  A pair owns a 256 x tile_n output tile: each CTA
// holds the accumulator of 128 of its rows in its own tensor memory, loads its own 128 rows of A
// and only HALF of B's tile_n columns; the hardware shares the B halves between the two SMs.
// Against the one-CTA kernel this cuts, per output element, the bytes each SM pulls from L2 by a
// third and the shared-memory traffic (TMA writes + operand reads) from about 192 to 128 bytes
// per clock, which is what the one-CTA kernel is bound by.
//
// Roles per CTA (224 threads) as in the one-CTA kernel: warps 0 and 6 produce, warp 1 issues MMAs
// (in the leader CTA only), warps 2-5 run the epilogue.  Barriers:
//   full[s]      in the leader: both CTAs' producers arrive (with their byte counts) and both
//                CTAs' TMA loads report their bytes there;
//   empty[s]     in each CTA: the leader's MMA warp commits to both;
//   acc_full[b]  in each CTA: the leader commits to both after the last k-block of a tile;
//   acc_empty[b] in the leader: the four epilogue warps of both CTAs arrive.
// No load is shared between the CTAs: each fetches its own boxes with ordinary TMA.
#pragma once
#include "gemm_tcgen05.cuh"

namespace frisk {

// Work items of the pair kernel.  Items [0, narrow_from) are whole 256 x tile_n tiles.  When the
// tiles do not fill the last wave of pairs at least half, each tile of that wave is cut into two
// 256 x tile_n/2 items instead, so that the wave takes about half as long: items narrow_from,
// narrow_from + 1, ... are the left and right halves of tiles narrow_from, narrow_from + 1, ...
//
// K planes (k_parts > 1; no narrow items then): item i is part i / tiles of tile i % tiles, covers
// k-blocks [kb0, kb1) and leaves as fp32 into plane `part` (GemmParams::k_parts).
struct PairItem {
  uint32_t tile, narrow, half, part, kb0, kb1;
};
__device__ __forceinline__ PairItem pair_item(uint32_t i, uint32_t narrow_from, const GemmParams& p) {
  PairItem it;
  const uint32_t j = i - narrow_from;   // meaningful when i >= narrow_from
  it.narrow = i >= narrow_from ? 1u : 0u;
  it.tile = it.narrow ? narrow_from + (j >> 1) : i;
  it.half = it.narrow ? (j & 1u) : 0u;
  it.part = 0;
  it.kb0 = 0;
  it.kb1 = p.num_kb;
  if (p.k_parts > 1u) {
    const uint32_t tiles = p.tiles_r * p.tiles_c;
    it.part = i / tiles;
    it.tile = i - it.part * tiles;
    it.kb0 = it.part * p.kb_per;
    it.kb1 = min(p.num_kb, it.kb0 + p.kb_per);
  }
  return it;
}

// kTf32 (C fp32 only) issues kind::tf32 MMAs on fp32 operand tiles: the 3xTF32 plan of fp32 GEMMs.
template <typename TC, bool kTf32 = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmap_a,
                         const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ GemmParams p,
                         const __grid_constant__ CStoreMaps c_maps) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kMaxStages];
  __shared__ __align__(8) uint64_t bar_empty[kMaxStages];
  __shared__ __align__(8) uint64_t bar_acc_full[2];
  __shared__ __align__(8) uint64_t bar_acc_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ uint32_t abort_word;

  const uint32_t warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0);
  const uint32_t lane = threadIdx.x & 31;
  // values that come out of inline PTX or shared memory are broadcast so that the compiler can
  // treat them (and the branches on them) as warp-uniform
  const uint32_t rank = __shfl_sync(0xffffffffu, ptx::cluster_ctarank(), 0);  // 0 = leader
  const uint32_t pair = blockIdx.x >> 1;
  const uint32_t num_pairs = gridDim.x >> 1;
  volatile uint32_t* abort_flag = &abort_word;

  const uint32_t tiles_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t full0 = ptx::smem_u32(&bar_full[0]);
  const uint32_t empty0 = ptx::smem_u32(&bar_empty[0]);
  const uint32_t acc_full0 = ptx::smem_u32(&bar_acc_full[0]);
  const uint32_t acc_empty0 = ptx::smem_u32(&bar_acc_empty[0]);
  // the same locations in the leader / in the other CTA (cluster-window addresses)
  const uint32_t leader_full0 = __shfl_sync(0xffffffffu, ptx::mapa(full0, 0), 0);
  const uint32_t leader_acc_empty0 = __shfl_sync(0xffffffffu, ptx::mapa(acc_empty0, 0), 0);
  const uint32_t peer_empty0 = __shfl_sync(0xffffffffu, ptx::mapa(empty0, rank ^ 1u), 0);
  const uint32_t peer_acc_full0 = __shfl_sync(0xffffffffu, ptx::mapa(acc_full0, rank ^ 1u), 0);
  const uint32_t peer_abort = __shfl_sync(0xffffffffu, ptx::mapa(ptx::smem_u32(&abort_word), rank ^ 1u), 0);

  const uint32_t stages = p.stages;
  const uint32_t stage_bytes = p.stage_bytes;  // per CTA
  const uint32_t tile_n = p.tile_n;
  const uint32_t tmem_cols = p.tmem_cols;
  const uint32_t tiles_r = p.tiles_r, tiles_c = p.tiles_c, group_r = p.group_r, group_c = p.group_c;
  const uint32_t n_items = p.n_items, narrow_from = p.narrow_from;
  int32_t* const status = p.status;
  const uint32_t debug_mode = kMeasureBuild ? p.debug_mode : 0u;

  if (threadIdx.x == 0) {
    abort_word = 0;
    for (uint32_t s = 0; s < stages; ++s) {
      ptx::mbar_init(full0 + 8 * s, 2);  // one producer arrival per CTA
      ptx::mbar_init(empty0 + 8 * s, 1);
    }
    for (uint32_t i = 0; i < 2; ++i) {
      ptx::mbar_init(acc_full0 + 8 * i, 1);
      ptx::mbar_init(acc_empty0 + 8 * i, 8);  // four epilogue warps in each CTA
    }
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
  // both CTAs' barriers must be initialised before either signals the other
  ptx::cluster_arrive();
  ptx::cluster_wait();
  ptx::tc_fence_after();
  const uint32_t tmem_base = __shfl_sync(0xffffffffu, tmem_base_slot, 0);
  // the set-up above may overlap the tail of the previous kernel in the stream; global memory is
  // touched only after that kernel has completed
  ptx::griddep_launch_dependents();
  ptx::griddep_wait();

  if (warp == 0 || warp == 6) {
    // ------------------------------------------------------------- TMA producers (both CTAs)
    const uint32_t a_boxes = p.a.num_boxes, a_box_bytes = p.a.box_bytes, a_box_mn = p.a.box_mn;
    const uint32_t b_boxes = p.b.num_boxes, b_box_bytes = p.b.box_bytes, b_box_mn = p.b.box_mn;
    const uint32_t a_mn_major = p.a.mn_major, b_mn_major = p.b.mn_major;
    const uint32_t a_stage_bytes = p.a.stage_bytes;
    const uint32_t bk_elems = p.bk_elems;
    const uint32_t my_turn = warp == 0 ? 0u : 1u;
    const uint32_t l2_hints = p.l2_hints;
    const uint64_t pol_a = ptx::l2_policy_evict_first(), pol_b = ptx::l2_policy_evict_last();
    uint32_t stage = 0, phase = 0, turn = 0;
    bool ok = true;
    for (uint32_t i = pair; ok && i < n_items; i += num_pairs) {
      const PairItem it = pair_item(i, narrow_from, p);
      uint32_t tr, tc;
      tile_coords(group_r, tiles_r, tiles_c, it.tile, tr, tc, group_c);
      const int32_t r0 = (int32_t)(tr * 256u + rank * 128u);
      // a narrow item covers columns [half * tile_n/2, +tile_n/2) of the tile; each CTA stages half
      const uint32_t cols_item = it.narrow ? (tile_n >> 1) : tile_n;
      const int32_t c0 = (int32_t)(tc * tile_n + it.half * (tile_n >> 1) + rank * (cols_item >> 1));
      const uint32_t b_boxes_item = it.narrow ? (b_boxes >> 1) : b_boxes;
      const uint32_t bytes_item = it.narrow ? a_stage_bytes + ((stage_bytes - a_stage_bytes) >> 1) : stage_bytes;
      for (uint32_t kb = it.kb0; kb < it.kb1; ++kb) {
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
        const uint32_t full = leader_full0 + 8 * stage;
        if (debug_mode & 1u) {
          if (ptx::elect_one()) ptx::mbar_arrive_cluster(full);
          if (++stage == stages) {
            stage = 0;
            phase ^= 1;
          }
          continue;
        }
        if (ptx::elect_one()) ptx::mbar_arrive_expect_tx_cluster(full, bytes_item);
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
          if (l2_hints & 1u) {
            if (ptx::elect_one()) ptx::tma_load_2d_pair_hint(a_dst + bx * a_box_bytes, &tmap_a, full, x, y, pol_a);
          } else {
            if (ptx::elect_one()) ptx::tma_load_2d_pair(a_dst + bx * a_box_bytes, &tmap_a, full, x, y);
          }
        }
        for (uint32_t bx = 0; bx < b_boxes_item; ++bx) {
          const int32_t mn = c0 + (int32_t)(bx * b_box_mn);
          const int32_t x = b_mn_major ? mn : k0b, y = b_mn_major ? k0b : mn;
          if (l2_hints & 2u) {
            if (ptx::elect_one()) ptx::tma_load_2d_pair_hint(b_dst + bx * b_box_bytes, &tmap_b, full, x, y, pol_b);
          } else {
            if (ptx::elect_one()) ptx::tma_load_2d_pair(b_dst + bx * b_box_bytes, &tmap_b, full, x, y);
          }
        }
        __syncwarp();  // reconverge after the elected-lane issues (see the one-CTA kernel)
        if (++stage == stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    if (!ok) {
      // tell the other CTA, then give copies in flight time to land (a copy takes a few
      // microseconds at most; this waits about 50)
      if (ptx::elect_one()) ptx::st_shared_cluster_u32(peer_abort, 1);
      const long long t0 = clock64();
      while (clock64() - t0 < 100000ll) {
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer (leader only)
    if (rank == 0) {
      const uint64_t a_desc_base = p.a.desc_base, b_desc_base = p.b.desc_base;
      const uint32_t a_k_step = p.a.k_step_bytes, b_k_step = p.b.k_step_bytes;
      const uint32_t a_stage_bytes = p.a.stage_bytes;
      const uint32_t idesc_wide = p.idesc, idesc_narrow = p.idesc_narrow;
      const uint32_t kind_f8 = p.kind_f8;
      uint32_t stage = 0, phase = 0, item = 0;
      bool ok = true;
      for (uint32_t i = pair; ok && i < n_items; i += num_pairs) {
        const uint32_t idesc = i >= narrow_from ? idesc_narrow : idesc_wide;
        const PairItem it = pair_item(i, narrow_from, p);
        const uint32_t acc = item & 1u;
        const uint32_t acc_phase = (item >> 1) & 1u;
        ok = bounded_wait(acc_empty0 + 8 * acc, acc_phase ^ 1, abort_flag, status,
                          kStatusMmaTimeout);
        if (!ok) break;
        ptx::tc_fence_after();
        const uint32_t d_base = tmem_base + acc * tile_n;
        // as in the one-CTA kernel: a stage is released after the first MMA of the next k-block,
        // and the next barrier is polled before the last MMA of the current one
        uint32_t prev_stage = 0;
        bool have_prev = false;
        uint32_t ready = __all_sync(0xffffffffu, ptx::mbar_try_wait(full0 + 8 * stage, phase));
        for (uint32_t kb = it.kb0; kb < it.kb1; ++kb) {
          if (!ready) {
            ok = bounded_wait_slow(full0 + 8 * stage, phase, abort_flag, status, kStatusMmaTimeout,
                                   0);
            if (!ok) break;
          }
          ptx::tc_fence_after();
          const uint32_t a_addr = tiles_base + stage * stage_bytes;
          const uint32_t b_addr = a_addr + a_stage_bytes;
          const uint64_t adesc0 = a_desc_base | (uint64_t)((a_addr & 0x3FFFFu) >> 4);
          const uint64_t bdesc0 = b_desc_base | (uint64_t)((b_addr & 0x3FFFFu) >> 4);
          const uint32_t first = kb > it.kb0 ? 1u : 0u;
          uint32_t next_stage = stage + 1, next_phase = phase;
          if (next_stage == stages) {
            next_stage = 0;
            next_phase ^= 1;
          }
          if (debug_mode & 2u) {
            if (ptx::elect_one()) ptx::mbar_arrive_cluster(empty0 + 8 * stage);
            if (ptx::elect_one()) ptx::mbar_arrive_cluster(peer_empty0 + 8 * stage);
            ready = __all_sync(0xffffffffu, ptx::mbar_test_wait(full0 + 8 * next_stage, next_phase));
            stage = next_stage;
            phase = next_phase;
            continue;
          }
#pragma unroll
          for (uint32_t ks = 0; ks < 4; ++ks) {
            const uint64_t bdesc = bdesc0 + (uint64_t)((ks * b_k_step) >> 4);
            const uint64_t adesc = adesc0 + (uint64_t)((ks * a_k_step) >> 4);
            const uint32_t accumulate = first | (ks > 0 ? 1u : 0u);
            if (ks == 3)
              ready = __all_sync(0xffffffffu, ptx::mbar_test_wait(full0 + 8 * next_stage, next_phase));
            if (kTf32) {
              if (ptx::elect_one()) ptx::mma_tf32_pair(d_base, adesc, bdesc, idesc, accumulate);
            } else if (kind_f8) {
              if (ptx::elect_one()) ptx::mma_f8_pair(d_base, adesc, bdesc, idesc, accumulate);
            } else {
              if (ptx::elect_one()) ptx::mma_f16_pair(d_base, adesc, bdesc, idesc, accumulate);
            }
            if (ks == 0 && have_prev) {
              if (ptx::elect_one()) ptx::tc_commit_pair(empty0 + 8 * prev_stage);
              if (ptx::elect_one()) ptx::tc_commit_pair(peer_empty0 + 8 * prev_stage);
            }
          }
          prev_stage = stage;
          have_prev = true;
          stage = next_stage;
          phase = next_phase;
        }
        if (!ok) break;
        if (have_prev) {
          if (ptx::elect_one()) ptx::tc_commit_pair(empty0 + 8 * prev_stage);
          if (ptx::elect_one()) ptx::tc_commit_pair(peer_empty0 + 8 * prev_stage);
        }
        if (ptx::elect_one()) ptx::tc_commit_pair(acc_full0 + 8 * acc);
        if (ptx::elect_one()) ptx::tc_commit_pair(peer_acc_full0 + 8 * acc);
        ++item;
      }
      if (!ok && ptx::elect_one()) ptx::st_shared_cluster_u32(peer_abort, 1);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------- epilogue (both CTAs)
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
    ex.c_maps = c_maps.m;
    RowFold rf;
    rf.kind = p.rr_kind;
    rf.nslots = 2u * tiles_c;
    rf.partials = p.rr_partials;
    const uint32_t quarter = warp & 3u;
    // the staging area of the epilogue sits behind the pipeline stages
    // (two buffers per warp when the rows leave through TMA stores)
    const uint32_t stage_area = tiles_base + stages * stage_bytes +
                                quarter * kEpiStageBytesPerWarp * (ex.staged == 3u ? 2u : 1u);
    uint32_t item = 0;
    bool ok = true;
    for (uint32_t i = pair; ok && i < n_items; i += num_pairs) {
      const PairItem it = pair_item(i, narrow_from, p);
      const uint32_t acc = item & 1u;
      const uint32_t acc_phase = (item >> 1) & 1u;
      uint32_t tr, tc;
      tile_coords(group_r, tiles_r, tiles_c, it.tile, tr, tc, group_c);
      const uint32_t cols_item = it.narrow ? (tile_n >> 1) : tile_n;
      const uint32_t col0 = tc * tile_n + it.half * (tile_n >> 1);
      ok = bounded_wait(acc_full0 + 8 * acc, acc_phase, abort_flag, status, kStatusEpilogueTimeout,
                        p.epilogue_backoff_ns);
      if (!ok) break;
      ptx::tc_fence_after();
      if (p.k_parts > 1u) ep.C = reinterpret_cast<TC*>(p.C) + (size_t)it.part * p.plane_elems;
      const uint32_t warp_row0 = tr * 256u + rank * 128u + quarter * 32u;
      const uint32_t t_row = tmem_base + ((quarter * 32u) << 16) + acc * tile_n;
      float red = fold_identity(rf.kind);
      epilogue_item<TC>(ep, ex, stage_area, lane, warp_row0, col0, cols_item, t_row, red);
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive_cluster(leader_acc_empty0 + 8 * acc);
      if (rf.kind) row_fold_store(rf, warp_row0 + lane, ep.rows, 2u * tc + it.half, it.narrow ? 1u : 2u, red);
      ++item;
    }
    if (!ok && lane == 0) ptx::st_shared_cluster_u32(peer_abort, 1);
    // shared memory must outlive the reads of the tensor stores still in flight
    if (ex.staged == 3u && lane == 0) ptx::bulk_wait_group_read<0>();
    __syncwarp();
  }

  // ---------------------------------------------------------------- tear-down
  // Neither CTA may exit (or free tensor memory) while the other can still signal its barriers.
  ptx::tc_fence_before();
  __syncthreads();
  ptx::cluster_arrive();
  ptx::cluster_wait();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc_pair(tmem_base, tmem_cols);
  }
}

}  // namespace frisk
