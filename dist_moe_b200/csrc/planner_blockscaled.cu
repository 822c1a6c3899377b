// Device-side activation-arena planner for the block-scaled (MXFP8 / NVFP4) paths.
//
// Same arena and state tensors as the BF16 planner (activation slots filled front to back with saved tensors, shared
// scratch carved back to front), but what is placed are *bundles*: quantised data immediately followed by its scale
// factors, row-quantised for the forward / input-gradient GEMMs and column-quantised for the weight-gradient GEMMs.
// One thread does the arithmetic; values, state updates and the two offset tables follow the reference kernels
// (dist_moe/_activation_buffer_planner_kernel.py:293-647 forward, 651-1065 backward, helpers 82-289).  Where the
// reference asserts on the device, this kernel sets a status word and carries on.
#include "common.cuh"
#include "../../include/dist_moe_b200.h"

namespace dm {

struct BsGeometry {
  int64_t element_size;          // dense activations (bf16 = 2)
  int64_t operand_element_size;  // bytes per quantised storage element
  int64_t values_per_element;    // logical values per storage element (2 for FP4)
  int64_t scale_element_size;
  int64_t row_scale_multiple;    // row-scale storage is over-allocated by this factor (blocked layout padding)
  int64_t row_global_scale_size;  // per-row payload after the row scales (4 for NVFP4)
  int64_t sf_vec;
};

__device__ __forceinline__ int64_t bs_align(int64_t v) { return (v + 127) / 128 * 128; }
__device__ __forceinline__ int64_t bs_cdiv(int64_t a, int64_t b) { return (a + b - 1) / b; }

struct BsPair {
  int64_t q, scale;
  __device__ int64_t total() const { return q + scale; }
};

__device__ BsPair row_quant_sizes(int64_t rows, int64_t dim, const BsGeometry& g) {
  const int64_t packed = bs_cdiv(dim, g.values_per_element);
  const int64_t scale_cols = bs_cdiv(dim, g.sf_vec);
  return {bs_align(rows * packed * g.operand_element_size),
          bs_align(rows * g.row_scale_multiple * scale_cols * g.scale_element_size + rows * g.row_global_scale_size)};
}

__device__ BsPair col_quant_sizes(int64_t rows, int64_t dim, const BsGeometry& g) {
  const int64_t packed_rows = bs_cdiv(rows, g.values_per_element);
  const int64_t scale_rows = bs_cdiv(rows, g.sf_vec);
  return {bs_align(dim * packed_rows * g.operand_element_size), bs_align(dim * scale_rows * g.scale_element_size)};
}

// Bytes of `rows` packed dispatch rows [q | scales | global scale], each padded to 16 bytes.
__device__ int64_t packed_dispatch_size(int64_t rows, int64_t dim, const BsGeometry& g) {
  const int64_t row_bytes = bs_cdiv(dim, g.values_per_element) * g.operand_element_size +
                            bs_cdiv(dim, g.sf_vec) * g.scale_element_size + g.row_global_scale_size;
  return bs_align(rows * ((row_bytes + 15) / 16 * 16));
}

// What one rank's rows cost in the slot when the layer is saved instead of recomputed.
__device__ int64_t no_recompute_alloc(int64_t rank_rows, int64_t h3_mem, int64_t D, int64_t F, const BsGeometry& g,
                                      bool native_backward) {
  const BsPair x = native_backward ? row_quant_sizes(rank_rows, D, g) : col_quant_sizes(rank_rows, D, g);
  const BsPair h2 = native_backward ? row_quant_sizes(rank_rows, F, g) : col_quant_sizes(rank_rows, F, g);
  return x.total() + bs_align(rank_rows * 2 * F * g.element_size) + h2.total() + h3_mem;
}

// One group of the offset tables: [a_q, b_q, c, a_scale, b_scale, source_x, source_y, col_q, col_scale].
__device__ void store_group(int64_t* table, int group, int64_t a_q, int64_t b_q, int64_t c, int64_t a_scale,
                            int64_t b_scale, int64_t source_x, int64_t source_y, int64_t col_q, int64_t col_scale) {
  int64_t* t = table + group * 9;
  t[0] = a_q;
  t[1] = b_q;
  t[2] = c;
  t[3] = a_scale;
  t[4] = b_scale;
  t[5] = source_x;
  t[6] = source_y;
  t[7] = col_q;
  t[8] = col_scale;
}

struct BsPlanCommon {
  const int32_t* recv_rows;
  const int32_t* per_rank;
  int64_t* saved;
  int64_t* buffer_offsets;
  int64_t* peak;
  int64_t* moe_layer_id;
  BsGeometry g;
  int ep, K, num_slots;
  int64_t T, D, F, capacity_rows, slot_bytes;
  int mega, native_backward;
  int* status;
};

struct BsPlanFwdParams {
  BsPlanCommon c;
  int32_t* per_rank_snapshot;
  uint8_t* need_recompute;
  int32_t* recompute_cond;
  int64_t* fwd_offsets;   // [x, x_gathered, h1, h2, h3, x_row, x_col, h2_row, h2_col, slot selector]
  int64_t* fwd_table;     // 2 groups: dispatch (W13), combine (W2)
  const int64_t* slot_selector;
  int num_layers, inference_mode, scratch_only, interleaved_fc13;
};

__global__ void plan_fwd_blockscaled_kernel(BsPlanFwdParams p) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const BsPlanCommon& c = p.c;
  const BsGeometry& g = c.g;
  const int N = c.num_slots;
  if (p.per_rank_snapshot)
    for (int r = 0; r < c.ep; ++r) p.per_rank_snapshot[r] = c.per_rank[r];
  const int64_t rows = c.recv_rows[0];
  if (rows > c.capacity_rows) set_status(c.status, kCapacityExceeded, 3);
  const int64_t h1_size = bs_align(rows * 2 * c.F * g.element_size);
  const BsPair x_row = row_quant_sizes(rows, c.D, g), h2_row = row_quant_sizes(rows, c.F, g);
  const BsPair x_col = col_quant_sizes(rows, c.D, g), h2_col = col_quant_sizes(rows, c.F, g);
  const int64_t scratch_end = c.buffer_offsets[N];
  int64_t x_row_off = scratch_end - x_row.total();
  int64_t h2_row_off, row_slot_size;
  if (c.mega) {  // one launch reads both row bundles: they may not alias
    h2_row_off = x_row_off - h2_row.total();
    row_slot_size = x_row.total() + h2_row.total();
  } else {  // staged launches run one after the other and share one slot
    h2_row_off = scratch_end - h2_row.total();
    row_slot_size = x_row.total() > h2_row.total() ? x_row.total() : h2_row.total();
  }
  const int64_t row_slot_off = scratch_end - row_slot_size;

  int64_t x_off = 0, h1_off = 0, h3_off = 0, x_col_off = 0, h2_col_off = 0, h2_staging_off = 0, scratch_bottom = 0;
  const int64_t scratch_base = p.inference_mode ? 0 : static_cast<int64_t>(N) * c.slot_bytes;
  const int64_t selector = p.slot_selector ? p.slot_selector[0] : 0;
  bool need = true;
  if (p.inference_mode || p.scratch_only) {
    if (p.interleaved_fc13) {
      h2_staging_off = row_slot_off;
      if (g.row_global_scale_size > 0) h2_staging_off = row_slot_off - bs_align(rows * c.F * g.element_size);
      scratch_bottom = h2_staging_off;
    } else {
      h1_off = row_slot_off - h1_size;
      scratch_bottom = h1_off;
    }
  } else {
    const int64_t m = selector % N;
    const int64_t free_start = c.buffer_offsets[m];
    const int64_t slot_end = (m + 1) * c.slot_bytes;
    const int64_t x_mem = c.native_backward ? packed_dispatch_size(c.T, c.D, g) : bs_align(c.T * c.D * g.element_size);
    const int64_t h3_mem = bs_align(c.T * c.K * c.D * g.element_size);
    const int64_t layer = c.moe_layer_id[m];
    const int64_t layers_after = (p.num_layers - 1) - layer;
    int64_t worst = INT64_MIN;
    for (int r = 0; r < c.ep; ++r) {
      const int64_t v = c.saved[m * c.ep + r] + no_recompute_alloc(c.per_rank[r], h3_mem, c.D, c.F, g, c.native_backward);
      worst = v > worst ? v : worst;
    }
    need = worst + layers_after * x_mem > c.slot_bytes;
    int64_t new_free;
    if (need && c.native_backward) {
      x_off = free_start;  // the packed dispatch input
      new_free = x_off + x_mem;
      h1_off = row_slot_off - h1_size;
      scratch_bottom = h1_off;
    } else if (need) {
      x_off = free_start;  // dense x; everything else is transient, descending below the row slot
      new_free = x_off + x_mem;
      x_col_off = row_slot_off - x_col.total();
      h1_off = x_col_off - h1_size;
      h2_col_off = h1_off - h2_col.total();
      scratch_bottom = h2_col_off;
    } else if (c.native_backward) {
      x_row_off = free_start;  // the row bundles the forward GEMMs read are what the backward needs
      h1_off = x_row_off + x_row.total();
      h2_row_off = h1_off + h1_size;
      h3_off = h2_row_off + h2_row.total();
      new_free = h3_off + h3_mem;
      scratch_bottom = scratch_end;
    } else {
      x_col_off = free_start;  // saved, ascending: x_col, h1, h2_col, h3
      h1_off = x_col_off + x_col.total();
      h2_col_off = h1_off + h1_size;
      h3_off = h2_col_off + h2_col.total();
      new_free = h3_off + h3_mem;
      scratch_bottom = row_slot_off;
    }
    if (new_free > slot_end) set_status(c.status, kArenaOverflow, 1, static_cast<int>(m));
    const int64_t slot_free = slot_end - new_free;
    if (slot_free < c.peak[m]) c.peak[m] = slot_free;
    c.buffer_offsets[m] = new_free;
    c.moe_layer_id[m] = layer + 1;
    for (int r = 0; r < c.ep; ++r)
      c.saved[m * c.ep + r] += need ? x_mem : no_recompute_alloc(c.per_rank[r], h3_mem, c.D, c.F, g, c.native_backward);
  }
  if (scratch_bottom < scratch_base) set_status(c.status, kArenaOverflow, 0);
  const int64_t scratch_free = scratch_bottom - scratch_base;
  if (scratch_free < c.peak[N]) c.peak[N] = scratch_free;

  if (c.native_backward) {
    x_col_off = x_row_off;
    h2_col_off = h2_row_off;
  }
  p.need_recompute[0] = need ? 1 : 0;
  if (p.recompute_cond) p.recompute_cond[0] = need ? 1 : 0;
  int64_t* o = p.fwd_offsets;
  o[0] = x_off;
  o[1] = 0;  // dense x_gathered and h2 do not exist on this path
  o[2] = h1_off;
  o[3] = 0;
  o[4] = h3_off;
  o[5] = x_row_off;
  o[6] = x_col_off;
  o[7] = h2_row_off;
  o[8] = h2_col_off;
  o[9] = selector;

  const int64_t missing = -1;
  int64_t d_col_q, d_col_s, c_col_q, c_col_s;
  if (c.native_backward) {  // no column bundle is produced: keep the entries addressable by aliasing the row bundle
    d_col_q = x_row_off;
    d_col_s = x_row_off + x_row.q;
    c_col_q = h2_row_off;
    c_col_s = h2_row_off + h2_row.q;
  } else {
    d_col_q = x_col_off;
    d_col_s = x_col_off + x_col.q;
    c_col_q = h2_col_off;
    c_col_s = h2_col_off + h2_col.q;
  }
  int64_t dispatch_c = h1_off, src_x = h1_off, src_y = h1_off + c.F * g.element_size;
  if (p.interleaved_fc13) {
    dispatch_c = missing;
    src_x = src_y = g.row_global_scale_size > 0 ? h2_staging_off : missing;
  }
  store_group(p.fwd_table, 0, x_row_off, missing, dispatch_c, x_row_off + x_row.q, missing, missing, missing, d_col_q,
              d_col_s);
  store_group(p.fwd_table, 1, h2_row_off, missing, missing, h2_row_off + h2_row.q, missing, src_x, src_y, c_col_q,
              c_col_s);
}

struct BsPlanBwdParams {
  BsPlanCommon c;
  const uint8_t* need_recompute;
  const int64_t* fwd_offsets;
  int64_t* bwd_offsets;  // 16 entries, see the header
  int64_t* bwd_table;    // 6 groups
};

__global__ void plan_bwd_blockscaled_kernel(BsPlanBwdParams p) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const BsPlanCommon& c = p.c;
  const BsGeometry& g = c.g;
  const int N = c.num_slots;
  const int64_t rows = c.recv_rows[0];
  if (rows > c.capacity_rows) set_status(c.status, kCapacityExceeded, 4);
  const bool need = p.need_recompute[0] != 0;
  // the slot the forward recorded, so that a later change of the selector cannot redirect this backward
  const int64_t m = p.fwd_offsets[9] % N;
  const int64_t scratch_end = c.buffer_offsets[N];
  const int64_t free_start = c.buffer_offsets[m];
  const int64_t slot_end = (m + 1) * c.slot_bytes;
  const int64_t fwd_x = p.fwd_offsets[0], fwd_h1 = p.fwd_offsets[2], fwd_x_row = p.fwd_offsets[5],
                fwd_x_col = p.fwd_offsets[6], fwd_h2_row = p.fwd_offsets[7], fwd_h2_col = p.fwd_offsets[8];

  const BsPair x_row = row_quant_sizes(rows, c.D, g), h2_row = row_quant_sizes(rows, c.F, g),
               dxy_row = row_quant_sizes(rows, 2 * c.F, g);
  auto max2 = [](int64_t a, int64_t b) { return a > b ? a : b; };
  int64_t x_row_off = scratch_end - x_row.total();
  int64_t recompute_h2_row_off, recompute_row_slot;
  if (c.mega || c.native_backward) {
    recompute_h2_row_off = x_row_off - h2_row.total();
    recompute_row_slot = max2(x_row.total() + h2_row.total(), dxy_row.total());
  } else {
    recompute_h2_row_off = scratch_end - h2_row.total();
    recompute_row_slot = max2(max2(x_row.total(), h2_row.total()), dxy_row.total());
  }
  const int64_t dxy_row_off = scratch_end - dxy_row.total();
  int64_t h2_row_off = need ? recompute_h2_row_off : dxy_row_off;
  const int64_t row_slot_size = need ? recompute_row_slot : max2(x_row.total(), dxy_row.total());
  const int64_t row_slot_off = scratch_end - row_slot_size;
  const int64_t grad_h3_row_off = x_row_off;  // the input-gradient launches are serialised and reuse the x_row bytes

  const BsPair x_col = col_quant_sizes(rows, c.D, g), h2_col = col_quant_sizes(rows, c.F, g),
               dxy_col = col_quant_sizes(rows, 2 * c.F, g);
  const int64_t h1_size = bs_align(rows * 2 * c.F * g.element_size);
  const int64_t grad_h2_size = bs_align(rows * c.F * g.element_size);
  const int64_t x_gathered_size = bs_align(rows * c.D * g.element_size);
  int64_t x_gathered_off = 0, h2_off = 0, grad_h3_gathered_off = 0, grad_h1_off = 0;
  int64_t h1_off, x_col_off, h2_col_off, grad_h3_col_off, grad_h2_off, dxy_col_off, scratch_bottom;
  int64_t cursor = row_slot_off;
  if (c.native_backward) {  // dense backward: the row bundles are dequantised up front
    if (need) {
      h1_off = cursor - h1_size;
      cursor = h1_off;
      h2_row_off = recompute_h2_row_off;
    } else {
      h1_off = fwd_h1;
      x_row_off = fwd_x_row;
      h2_row_off = fwd_h2_row;
      cursor = scratch_end;
    }
    x_gathered_off = cursor - x_gathered_size;
    h2_off = x_gathered_off - grad_h2_size;
    grad_h3_gathered_off = h2_off - x_gathered_size;
    grad_h2_off = grad_h3_gathered_off - grad_h2_size;
    grad_h1_off = grad_h2_off - h1_size;
    x_col_off = x_row_off;
    h2_col_off = h2_row_off;
    grad_h3_col_off = grad_h3_row_off;
    dxy_col_off = dxy_row_off;
    scratch_bottom = grad_h1_off;
  } else {
    if (need) {  // rebuilt in scratch, above the gradients
      x_col_off = cursor - x_col.total();
      cursor = x_col_off;
      h1_off = cursor - h1_size;
      cursor = h1_off;
      h2_col_off = cursor - h2_col.total();
      cursor = h2_col_off;
    } else {
      x_col_off = fwd_x_col;
      h1_off = fwd_h1;
      h2_col_off = fwd_h2_col;
    }
    grad_h3_col_off = cursor - x_col.total();
    cursor = grad_h3_col_off;
    grad_h2_off = cursor - grad_h2_size;
    cursor = grad_h2_off;
    dxy_col_off = cursor - dxy_col.total();
    scratch_bottom = dxy_col_off;
  }
  const int64_t scratch_base = static_cast<int64_t>(N) * c.slot_bytes;
  if (scratch_bottom < scratch_base) set_status(c.status, kArenaOverflow, 2);
  const int64_t scratch_free = scratch_bottom - scratch_base;
  if (scratch_free < c.peak[N]) c.peak[N] = scratch_free;
  if (slot_end - free_start < c.peak[m]) c.peak[m] = slot_end - free_start;

  int64_t* o = p.bwd_offsets;
  o[0] = x_gathered_off;
  o[1] = h1_off;
  o[2] = h2_off;
  o[3] = grad_h2_off;
  o[4] = grad_h3_gathered_off;
  o[5] = grad_h1_off;
  o[6] = x_row_off;
  o[7] = x_col_off;
  o[8] = h2_row_off;
  o[9] = h2_col_off;
  o[10] = grad_h3_row_off;
  o[11] = grad_h3_col_off;
  o[12] = dxy_row_off;
  o[13] = dxy_col_off;
  // where the per-row global scales of the two row bundles start (behind their block scales)
  o[14] = x_row_off + x_row.q + rows * g.row_scale_multiple * bs_cdiv(c.D, g.sf_vec) * g.scale_element_size;
  o[15] = h2_row_off + h2_row.q + rows * g.row_scale_multiple * bs_cdiv(c.F, g.sf_vec) * g.scale_element_size;

  const int64_t missing = -1;
  int64_t x_col_s, h2_col_s, grad_h3_col_s, dxy_col_s;
  if (c.native_backward) {
    x_col_s = x_row_off + x_row.q;
    h2_col_s = h2_row_off + h2_row.q;
    grad_h3_col_s = grad_h3_row_off + x_row.q;
    dxy_col_s = dxy_row_off + dxy_row.q;
  } else {
    x_col_s = x_col_off + x_col.q;
    h2_col_s = h2_col_off + h2_col.q;
    grad_h3_col_s = grad_h3_col_off + x_col.q;
    dxy_col_s = dxy_col_off + dxy_col.q;
  }
  int64_t* t = p.bwd_table;
  store_group(t, 0, x_row_off, missing, h1_off, x_row_off + x_row.q, missing, missing, missing, x_col_off, x_col_s);
  store_group(t, 1, h2_row_off, missing, missing, h2_row_off + h2_row.q, missing, h1_off,
              h1_off + c.F * g.element_size, h2_col_off, h2_col_s);
  store_group(t, 2, grad_h3_row_off, missing, grad_h2_off, grad_h3_row_off + x_row.q, missing, missing, missing,
              grad_h3_col_off, grad_h3_col_s);
  store_group(t, 3, grad_h3_col_off, h2_col_off, missing, grad_h3_col_s, h2_col_s, missing, missing, missing, missing);
  store_group(t, 4, dxy_row_off, missing, missing, dxy_row_off + dxy_row.q, missing, grad_h2_off, h1_off, dxy_col_off,
              dxy_col_s);
  store_group(t, 5, dxy_col_off, x_col_off, missing, dxy_col_s, x_col_s, missing, missing, missing, missing);

  // rewind the slot to where the matching forward layer began, and undo its accounting
  const int64_t saved_base = c.native_backward ? fwd_x_row : x_col_off;
  c.buffer_offsets[m] = need ? fwd_x : saved_base;
  const int64_t x_mem = c.native_backward ? packed_dispatch_size(c.T, c.D, g) : bs_align(c.T * c.D * g.element_size);
  const int64_t h3_mem = bs_align(c.T * c.K * c.D * g.element_size);
  for (int r = 0; r < c.ep; ++r)
    c.saved[m * c.ep + r] -= need ? x_mem : no_recompute_alloc(c.per_rank[r], h3_mem, c.D, c.F, g, c.native_backward);
  c.moe_layer_id[m] -= 1;
}

static bool geometry_ok(const int* g) {
  return g && g[0] > 0 && g[1] > 0 && g[2] > 0 && g[3] > 0 && g[4] >= 0 && g[5] > 0;
}

static BsGeometry make_geometry(const int* g) { return BsGeometry{2, g[0], g[1], g[2], g[3], g[4], g[5]}; }

}  // namespace dm

using namespace dm;

extern "C" int dm_plan_fwd_blockscaled(const int32_t* recv_rows, const int32_t* per_rank, int32_t* per_rank_snapshot,
                                       int64_t* saved_bytes_per_rank, int64_t* buffer_offsets, int64_t* peak_min_free,
                                       uint8_t* need_recompute, int32_t* recompute_cond, int64_t* fwd_offsets,
                                       int64_t* fwd_activation_offsets, const int64_t* slot_selector,
                                       int64_t* moe_layer_id, int ep, int64_t num_tokens, int K, int64_t D, int64_t F,
                                       const int* storage, int64_t capacity_rows, int64_t slot_bytes, int num_slots,
                                       int num_moe_layers, int mega, int inference_mode, int scratch_only,
                                       int native_backward, int interleaved_fc13, int* status, void* stream) {
  if (!recv_rows || !per_rank || !buffer_offsets || !peak_min_free || !need_recompute || !fwd_offsets ||
      !fwd_activation_offsets || !geometry_ok(storage))
    return kRcBadArg;
  const bool uses_slots = !(inference_mode || scratch_only);
  if (uses_slots && (!saved_bytes_per_rank || !moe_layer_id || !slot_selector || num_slots <= 0)) return kRcBadArg;
  if (ep <= 0 || num_tokens <= 0 || K <= 0 || D <= 0 || F <= 0 || num_slots < 0 || capacity_rows < 0) return kRcBadArg;
  if (interleaved_fc13 && uses_slots) return kRcBadArg;  // the swizzled W13 epilogue keeps nothing for a backward
  BsPlanFwdParams p{};
  p.c = BsPlanCommon{recv_rows, per_rank, saved_bytes_per_rank, buffer_offsets, peak_min_free, moe_layer_id,
                     make_geometry(storage), ep, K, num_slots, num_tokens, D, F, capacity_rows, slot_bytes,
                     mega, native_backward, status};
  p.per_rank_snapshot = per_rank_snapshot;
  p.need_recompute = need_recompute;
  p.recompute_cond = recompute_cond;
  p.fwd_offsets = fwd_offsets;
  p.fwd_table = fwd_activation_offsets;
  p.slot_selector = slot_selector;
  p.num_layers = num_moe_layers;
  p.inference_mode = inference_mode;
  p.scratch_only = scratch_only;
  p.interleaved_fc13 = interleaved_fc13;
  plan_fwd_blockscaled_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_plan_bwd_blockscaled(const int32_t* recv_rows, const int32_t* per_rank, int64_t* saved_bytes_per_rank,
                                       int64_t* buffer_offsets, int64_t* peak_min_free, const uint8_t* need_recompute,
                                       const int64_t* fwd_offsets, int64_t* bwd_offsets,
                                       int64_t* bwd_activation_offsets, int64_t* moe_layer_id, int ep,
                                       int64_t num_tokens, int K, int64_t D, int64_t F, const int* storage,
                                       int64_t capacity_rows, int64_t slot_bytes, int num_slots, int mega,
                                       int native_backward, int* status, void* stream) {
  if (!recv_rows || !per_rank || !saved_bytes_per_rank || !buffer_offsets || !peak_min_free || !need_recompute ||
      !fwd_offsets || !bwd_offsets || !bwd_activation_offsets || !moe_layer_id || !geometry_ok(storage))
    return kRcBadArg;
  if (ep <= 0 || num_tokens <= 0 || K <= 0 || D <= 0 || F <= 0 || num_slots <= 0 || capacity_rows < 0) return kRcBadArg;
  BsPlanBwdParams p{};
  p.c = BsPlanCommon{recv_rows, per_rank, saved_bytes_per_rank, buffer_offsets, peak_min_free, moe_layer_id,
                     make_geometry(storage), ep, K, num_slots, num_tokens, D, F, capacity_rows, slot_bytes,
                     mega, native_backward, status};
  p.need_recompute = need_recompute;
  p.fwd_offsets = fwd_offsets;
  p.bwd_offsets = bwd_offsets;
  p.bwd_table = bwd_activation_offsets;
  plan_bwd_blockscaled_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return static_cast<int>(cudaGetLastError());
}
