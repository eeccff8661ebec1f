// Host-only part of libfrisk_b200.so: the mapping from the reference's shared-memory layouts to
// TMA / UMMA descriptor fields, and its bank-conflict cost model carried over to those swizzles.
//
// Reference facts this file restates (lib/Dialect/Frisk/IR/FriskOps.cpp):
//   * buildHopperSharedLayout (589-618) picks, for a row-major tile whose contiguous extent is
//     `cont` elements and vec = 128 / elementBits:  cont % (8 vec) == 0 -> full-bank swizzle,
//     % (4 vec) -> half-bank, % (2 vec) -> quarter-bank, % vec -> linear, else no layout.
//   * makeFull/Half/QuarterBankSwizzle (500-558) map (i, j) to (column atom, row atom, offset in
//     an 8-row atom) and XOR the 16-byte chunk index with the row: in byte addresses that is
//     bits[4,7) ^= bits[7,10) for 128-byte rows, bits[4,6) ^= bits[7,9) for 64-byte rows and
//     bit 4 ^= bit 7 for 32-byte rows -- the 128B / 64B / 32B swizzles of TMA and of the UMMA
//     shared-memory descriptor.
#include "../../include/frisk_b200.h"

#include <algorithm>
#include <cstring>
#include <set>
#include <vector>

namespace {

// XOR pattern of a swizzle mode applied to a byte offset inside one swizzle span.
int64_t apply_swizzle(int64_t off, int mode) {
  switch (mode) {
    case 128: return off ^ (((off >> 7) & 7) << 4);
    case 64: return off ^ (((off >> 7) & 3) << 4);
    case 32: return off ^ (((off >> 7) & 1) << 4);
    case FRISK_SWIZZLE_128B_ATOM_32B: return off ^ (((off >> 7) & 3) << 5);  // 32-byte chunks
    case FRISK_SWIZZLE_128B_ATOM_64B: return off ^ (((off >> 7) & 1) << 6);  // 64-byte chunks
    default: return off;
  }
}

int span_bytes(int mode) {
  if (mode == FRISK_SWIZZLE_128B_ATOM_32B || mode == FRISK_SWIZZLE_128B_ATOM_64B) return 128;
  return mode;
}

bool valid_mode(int mode) {
  return mode == 0 || mode == 32 || mode == 64 || mode == 128 ||
         mode == FRISK_SWIZZLE_128B_ATOM_32B || mode == FRISK_SWIZZLE_128B_ATOM_64B;
}

}  // namespace

extern "C" {

int frisk_b200_layout_to_tma(const frisk_layout_desc* l, frisk_tma_params* out) {
  if (!l || !out) return FRISK_ERR_INVALID_ARGUMENT;
  if (l->rows <= 0 || l->cols <= 0) return FRISK_ERR_INVALID_ARGUMENT;
  if (l->elem_bits != 8 && l->elem_bits != 16 && l->elem_bits != 32)
    return FRISK_ERR_UNSUPPORTED;  // the reference's f64 layouts have no tcgen05 operand type
  memset(out, 0, sizeof *out);
  const int es = l->elem_bits / 8;
  const int64_t vec = 128 / l->elem_bits;  // elements per 16 bytes
  const int64_t cont = l->cols;
  int sw;
  const char* name;
  if (cont % (vec * 8) == 0) { sw = 128; name = "full_bank"; }
  else if (cont % (vec * 4) == 0) { sw = 64; name = "half_bank"; }
  else if (cont % (vec * 2) == 0) { sw = 32; name = "quarter_bank"; }
  else if (cont % vec == 0) { sw = 0; name = "linear"; }
  else return FRISK_ERR_MISALIGNED;  // the reference returns no layout here either
  strncpy(out->reference_layout, name, sizeof out->reference_layout - 1);
  out->swizzle_bytes = sw;
  out->umma_layout_type = sw == 128 ? 2 : sw == 64 ? 4 : sw == 32 ? 6 : 0;
  out->umma_major = l->k_inner ? 0 : 1;
  const int span = sw ? sw : 16;                 // bytes of one box row
  out->box_inner = span / es;
  out->num_boxes = (int32_t)(cont * es / span);  // column atoms side by side
  if (l->rows > 256) return FRISK_ERR_TOO_LARGE; // a TMA box has at most 256 rows
  out->box_outer = (int32_t)l->rows;
  const int32_t atom = 8 * span;                        // 8 rows of one column atom
  const int32_t column_atom = (int32_t)l->rows * span;  // one box
  if (l->k_inner) {
    // K-major: rows are M/N.  8-row groups follow each other at SBO; with a swizzle the K extent
    // of one instruction stays inside the span, so LBO is not used (encoded as 16 bytes).
    out->stride_byte_offset = atom;
    out->leading_byte_offset = sw ? 16 : column_atom;
    out->k_step_bytes = 32;
  } else {
    // MN-major: rows are K.  8 K rows per atom (SBO apart); the next `span` bytes of M/N are in
    // the next box (LBO apart).  One K step of 32 bytes is 32/es rows.
    out->stride_byte_offset = atom;
    out->leading_byte_offset = column_atom;
    out->k_step_bytes = (32 / es) * span;
  }
  return FRISK_OK;
}

int64_t frisk_b200_swizzled_offset(int64_t row, int64_t col, int64_t rows, int64_t cols,
                                   int32_t elem_bits, int32_t mode) {
  if (row < 0 || col < 0 || row >= rows || col >= cols || elem_bits <= 0 || elem_bits % 8 ||
      !valid_mode(mode))
    return -1;
  const int64_t es = elem_bits / 8;
  if (mode == 0) return (row * cols + col) * es;
  const int64_t span = span_bytes(mode);
  if ((cols * es) % span) return -1;
  const int64_t cb = col * es;
  const int64_t col_atom = cb / span;
  const int64_t in_row = cb % span;
  // one box per column atom: `rows` rows of `span` bytes, swizzled inside the box
  return col_atom * rows * span + apply_swizzle(row * span + in_row, mode);
}

int frisk_b200_bank_conflicts(int64_t rows, int64_t cols, int32_t elem_bits, int32_t mode,
                              int32_t lane_vector, int32_t distinct_words_only,
                              frisk_bank_stats* out) {
  if (!out || rows <= 0 || cols <= 0 || elem_bits <= 0 || elem_bits % 8 || !valid_mode(mode))
    return FRISK_ERR_INVALID_ARGUMENT;
  const int64_t es = elem_bits / 8;
  const int64_t span = span_bytes(mode);
  if (mode && (cols * es) % span) return FRISK_ERR_MISALIGNED;
  const int64_t lv = std::max<int32_t>(1, lane_vector);
  const int64_t window = 32 * lv;
  const int64_t total = rows * cols;
  out->avg_max_conflict = 0;
  out->max_conflict = 0;
  out->samples = 0;
  for (int64_t chunk = 0; chunk < total; chunk += window) {
    int64_t hist[32] = {0};
    std::set<int64_t> words[32];
    bool any = false;
    for (int64_t lane = 0; lane < 32; ++lane) {
      for (int64_t v = 0; v < lv; ++v) {
        const int64_t linear = chunk + lane * lv + v;
        if (linear >= total) break;
        any = true;
        const int64_t row = linear / cols, col = linear % cols;
        int64_t byte;
        if (mode == 0) {
          byte = linear * es;
        } else if (!distinct_words_only) {
          // the reference model looks at the offset inside the 8-row atom only
          // (exp/layout/gemm_layout_tool.cpp:169 takes the last map result)
          byte = apply_swizzle((row % 8) * span + (col * es) % span, mode);
        } else {
          const int64_t col_atom = col * es / span;
          byte = col_atom * rows * span + apply_swizzle(row * span + (col * es) % span, mode);
        }
        const int64_t bank = (byte / 4) % 32;
        if (distinct_words_only) words[bank].insert(byte / 4);
        else hist[bank]++;
      }
    }
    if (!any) continue;
    int64_t local = 0;
    for (int b = 0; b < 32; ++b)
      local = std::max<int64_t>(local, distinct_words_only ? (int64_t)words[b].size() : hist[b]);
    out->samples++;
    out->max_conflict = std::max<int32_t>(out->max_conflict, (int32_t)local);
    out->avg_max_conflict += (double)local;
  }
  if (out->samples) out->avg_max_conflict /= out->samples;
  return FRISK_OK;
}

int frisk_b200_bank_conflicts_access(int64_t rows, int64_t cols, int32_t elem_bits, int32_t mode,
                                     int32_t access, frisk_access_stats* out) {
  if (!out || rows <= 0 || cols <= 0 || elem_bits <= 0 || elem_bits % 8 || !valid_mode(mode))
    return FRISK_ERR_INVALID_ARGUMENT;
  if (access != FRISK_ACCESS_CHUNK_COLUMN && access != FRISK_ACCESS_ROW_PIECES)
    return FRISK_ERR_INVALID_ARGUMENT;
  const int64_t es = elem_bits / 8;
  const int64_t row_bytes = cols * es;
  if (row_bytes % 16) return FRISK_ERR_MISALIGNED;
  const int64_t span = mode ? span_bytes(mode) : row_bytes;
  if (row_bytes % span) return FRISK_ERR_MISALIGNED;
  const int64_t chunks_per_row = row_bytes / 16;
  memset(out, 0, sizeof *out);
  // byte address of 16-byte chunk `c` of row `r`: one box per column atom, as TMA lays a tile out
  auto chunk_addr = [&](int64_t r, int64_t c) -> int64_t {
    const int64_t cb = c * 16;
    if (mode == 0) return r * row_bytes + cb;
    return (cb / span) * rows * span + apply_swizzle(r * span + cb % span, mode);
  };
  // One warp request of 32 x 16 bytes.  The hardware serves 16-byte accesses a quarter warp (8
  // lanes, 128 bytes) at a time; within a quarter every distinct 4-byte word that shares a bank
  // with another costs one more pass over the banks (a wavefront).
  auto request = [&](const int64_t (&addr)[32], int lanes) {
    int wavefronts = 0;
    for (int q = 0; q < lanes; q += 8) {
      std::set<int64_t> words[32];
      for (int l = q; l < std::min(lanes, q + 8); ++l)
        for (int w = 0; w < 4; ++w) {
          const int64_t word = addr[l] / 4 + w;
          words[word % 32].insert(word);
        }
      size_t worst = 0;
      for (int b = 0; b < 32; ++b) worst = std::max(worst, words[b].size());
      wavefronts += (int)worst;
    }
    const int ideal = (lanes + 7) / 8;
    out->requests++;
    out->wavefronts += wavefronts;
    out->ideal_wavefronts += ideal;
    out->max_wavefronts_per_request = std::max<int32_t>(out->max_wavefronts_per_request, wavefronts);
  };
  int64_t addr[32];
  if (access == FRISK_ACCESS_CHUNK_COLUMN) {
    // lane = row, every lane the same chunk column: 32 consecutive rows x one 16-byte chunk
    for (int64_t r0 = 0; r0 < rows; r0 += 32)
      for (int64_t c = 0; c < chunks_per_row; ++c) {
        const int lanes = (int)std::min<int64_t>(32, rows - r0);
        for (int l = 0; l < lanes; ++l) addr[l] = chunk_addr(r0 + l, c);
        request(addr, lanes);
      }
  } else {
    // consecutive lanes walk the chunks of a row, then the next row
    const int64_t total = rows * chunks_per_row;
    for (int64_t i0 = 0; i0 < total; i0 += 32) {
      const int lanes = (int)std::min<int64_t>(32, total - i0);
      for (int l = 0; l < lanes; ++l) addr[l] = chunk_addr((i0 + l) / chunks_per_row, (i0 + l) % chunks_per_row);
      request(addr, lanes);
    }
  }
  out->conflict_degree = out->ideal_wavefronts ? (double)out->wavefronts / (double)out->ideal_wavefronts : 0.0;
  // what the mode costs outside shared memory: boxes TMA has to issue for the tile and the
  // length of the contiguous global segment behind each box row
  out->tma_boxes = (int32_t)(mode ? row_bytes / span * ((rows + 255) / 256) : 0);
  out->global_segment_bytes = (int32_t)(mode ? span : row_bytes);
  return FRISK_OK;
}

}  // extern "C"
