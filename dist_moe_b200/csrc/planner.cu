// Device-side activation-arena planner for the BF16 path.
//
// The arena is one byte buffer: N activation slots (saved forward state, LIFO
// per slot) followed by shared scratch that is carved back to front.  Whether a
// layer saves its intermediates or recomputes them is decided here, on the
// device, from the routed row counts of *every* rank, so that all ranks take
// the same branch without a host read.  One thread does the arithmetic; the
// values and in-place state updates follow the reference kernels line by line
// (dist_moe/_activation_buffer_planner_kernel.py:1068-1275 forward, 1278-1477
// backward).
#include "common.cuh"
#include "../../include/dist_moe_b200.h"

namespace dm {

__device__ __forceinline__ int64_t align128(int64_t v) { return (v + 127) / 128 * 128; }

struct PlanFwdParams {
  const int32_t* recv_rows;
  const int32_t* per_rank;
  int64_t* saved;
  int64_t* buffer_offsets;
  int64_t* peak;
  uint8_t* need_recompute;
  int32_t* recompute_cond;
  int64_t* fwd_state;
  const int64_t* slot_selector;
  int64_t* moe_layer_id;
  int ep, K, num_slots, num_layers, scratch_only;
  int64_t T, D, F, slot_bytes;
  int* status;
};

__global__ void plan_fwd_bf16_kernel(PlanFwdParams p) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int64_t es = 2;
  const int64_t R = p.recv_rows[0];
  const int64_t xg_size = align128(R * p.D * es);
  const int64_t h1_size = align128(R * 2 * p.F * es);
  const int64_t h2_size = align128(R * p.F * es);
  const int N = p.num_slots;
  const int64_t scratch_end = p.buffer_offsets[N];
  const int64_t s_h2 = scratch_end - h2_size;
  const int64_t s_h1 = s_h2 - h1_size;
  const int64_t s_xg = s_h1 - xg_size;
  const int64_t selector = p.slot_selector[0];

  bool need = true;
  int64_t x_off = 0, xg_off = s_xg, h1_off = s_h1, h2_off = s_h2, h3_off = 0;
  int64_t m = 0, new_free = 0, slot_end = 0, layer = 0;
  const int64_t x_mem = align128(p.T * p.D * es);
  const int64_t h3_mem = align128(p.T * p.K * p.D * es);
  if (!p.scratch_only) {
    m = selector % N;
    const int64_t free_start = p.buffer_offsets[m];
    slot_end = (m + 1) * p.slot_bytes;
    layer = p.moe_layer_id[m];
    const int64_t layers_after = (p.num_layers - 1) - layer;
    int64_t worst = INT64_MIN;
    for (int r = 0; r < p.ep; ++r) {
      const int64_t rr = p.per_rank[r];
      const int64_t full = align128(rr * p.D * es) + align128(rr * 2 * p.F * es) + h3_mem;
      const int64_t v = p.saved[m * p.ep + r] + full;
      worst = v > worst ? v : worst;
    }
    need = worst + layers_after * x_mem > p.slot_bytes;
    if (need) {
      x_off = free_start;
      new_free = x_off + x_mem;
    } else {
      xg_off = free_start;
      h1_off = xg_off + xg_size;
      h3_off = h1_off + h1_size;
      new_free = h3_off + h3_mem;
      x_off = 0;
    }
  }
  p.need_recompute[0] = need ? 1 : 0;
  if (p.recompute_cond) p.recompute_cond[0] = need ? 1 : 0;
  p.fwd_state[0] = x_off;
  p.fwd_state[1] = xg_off;
  p.fwd_state[2] = h1_off;
  p.fwd_state[3] = h2_off;
  p.fwd_state[4] = h3_off;
  p.fwd_state[5] = selector;

  const int64_t scratch_bottom = need ? xg_off : h2_off;
  const int64_t scratch_base = static_cast<int64_t>(N) * p.slot_bytes;
  if (scratch_bottom < scratch_base) set_status(p.status, kArenaOverflow, 0);
  const int64_t scratch_free = scratch_bottom - scratch_base;
  if (scratch_free < p.peak[N]) p.peak[N] = scratch_free;

  if (!p.scratch_only) {
    if (new_free > slot_end) set_status(p.status, kArenaOverflow, 1, static_cast<int>(m));
    const int64_t slot_free = slot_end - new_free;
    if (slot_free < p.peak[m]) p.peak[m] = slot_free;
    p.buffer_offsets[m] = new_free;
    p.moe_layer_id[m] = layer + 1;
    for (int r = 0; r < p.ep; ++r) {
      const int64_t rr = p.per_rank[r];
      const int64_t full = align128(rr * p.D * es) + align128(rr * 2 * p.F * es) + h3_mem;
      p.saved[m * p.ep + r] += need ? x_mem : full;
    }
  }
}

struct PlanBwdParams {
  const int32_t* recv_rows;
  const int32_t* per_rank;
  int64_t* saved;
  int64_t* buffer_offsets;
  int64_t* peak;
  const uint8_t* need_recompute;
  const int64_t* fwd_state;
  int64_t* bwd_offsets;
  int64_t* moe_layer_id;
  int ep, K, num_slots;
  int64_t T, D, F, slot_bytes;
  int* status;
};

__global__ void plan_bwd_bf16_kernel(PlanBwdParams p) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  const int64_t es = 2;
  const int N = p.num_slots;
  const int64_t R = p.recv_rows[0];
  // The slot is the one the forward recorded, so that a later change of the
  // selector cannot redirect this backward.
  const int64_t m = p.fwd_state[5] % N;
  const int64_t free_start = p.buffer_offsets[m];
  const int64_t slot_end = (m + 1) * p.slot_bytes;
  const int64_t scratch_end = p.buffer_offsets[N];
  const bool need = p.need_recompute[0] != 0;
  const int64_t fwd_x = p.fwd_state[0], fwd_xg = p.fwd_state[1], fwd_h1 = p.fwd_state[2];

  const int64_t xg_size = align128(R * p.D * es);
  const int64_t h1_size = align128(R * 2 * p.F * es);
  const int64_t h2_size = align128(R * p.F * es);
  const int64_t g_h1 = scratch_end - h1_size;
  const int64_t g_h2 = g_h1 - h2_size;
  const int64_t h2_off = scratch_end - h2_size;
  const int64_t g_h3g = (p.D * es <= p.F * es) ? h2_off - xg_size : g_h2 - xg_size;
  const int64_t grad_bottom = g_h2 < g_h3g ? g_h2 : g_h3g;
  int64_t xg_off, h1_off, bottom;
  if (need) {
    h1_off = grad_bottom - h1_size;
    xg_off = h1_off - xg_size;
    bottom = xg_off;
  } else {
    xg_off = fwd_xg;
    h1_off = fwd_h1;
    bottom = grad_bottom;
  }
  const int64_t scratch_base = static_cast<int64_t>(N) * p.slot_bytes;
  if (bottom < scratch_base) set_status(p.status, kArenaOverflow, 2);
  const int64_t slot_free = slot_end - free_start;
  if (slot_free < p.peak[m]) p.peak[m] = slot_free;
  const int64_t scratch_free = bottom - scratch_base;
  if (scratch_free < p.peak[N]) p.peak[N] = scratch_free;

  p.bwd_offsets[0] = xg_off;
  p.bwd_offsets[1] = h1_off;
  p.bwd_offsets[2] = h2_off;
  p.bwd_offsets[3] = g_h2;
  p.bwd_offsets[4] = g_h3g;
  p.bwd_offsets[5] = g_h1;

  p.buffer_offsets[m] = need ? fwd_x : fwd_xg;
  const int64_t x_mem = align128(p.T * p.D * es);
  const int64_t h3_mem = align128(p.T * p.K * p.D * es);
  for (int r = 0; r < p.ep; ++r) {
    const int64_t rr = p.per_rank[r];
    const int64_t full = align128(rr * p.D * es) + align128(rr * 2 * p.F * es) + h3_mem;
    p.saved[m * p.ep + r] -= need ? x_mem : full;
  }
  p.moe_layer_id[m] -= 1;
}

}  // namespace dm

using namespace dm;

extern "C" int dm_plan_fwd_bf16(const int32_t* recv_rows, const int32_t* per_rank, int64_t* saved_bytes_per_rank,
                                int64_t* buffer_offsets, int64_t* peak_min_free, uint8_t* need_recompute,
                                int32_t* recompute_cond, int64_t* fwd_state, const int64_t* slot_selector,
                                int64_t* moe_layer_id, int ep, int64_t num_tokens, int K, int64_t D, int64_t F,
                                int64_t slot_bytes, int num_slots, int num_moe_layers, int scratch_only, int* status,
                                void* stream) {
  if (!recv_rows || !per_rank || !buffer_offsets || !peak_min_free || !need_recompute || !fwd_state || !slot_selector)
    return kRcBadArg;
  if (!scratch_only && (!saved_bytes_per_rank || !moe_layer_id || num_slots <= 0)) return kRcBadArg;
  if (ep <= 0 || num_tokens <= 0 || K <= 0 || D <= 0 || F <= 0 || num_slots < 0) return kRcBadArg;
  PlanFwdParams p{recv_rows, per_rank, saved_bytes_per_rank, buffer_offsets, peak_min_free, need_recompute,
                  recompute_cond, fwd_state, slot_selector, moe_layer_id, ep, K, num_slots, num_moe_layers,
                  scratch_only, num_tokens, D, F, slot_bytes, status};
  plan_fwd_bf16_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_plan_bwd_bf16(const int32_t* recv_rows, const int32_t* per_rank, int64_t* saved_bytes_per_rank,
                                int64_t* buffer_offsets, int64_t* peak_min_free, const uint8_t* need_recompute,
                                const int64_t* fwd_state, int64_t* bwd_offsets, int64_t* moe_layer_id, int ep,
                                int64_t num_tokens, int K, int64_t D, int64_t F, int64_t slot_bytes, int num_slots,
                                int* status, void* stream) {
  if (!recv_rows || !per_rank || !saved_bytes_per_rank || !buffer_offsets || !peak_min_free || !need_recompute ||
      !fwd_state || !bwd_offsets || !moe_layer_id)
    return kRcBadArg;
  if (ep <= 0 || num_tokens <= 0 || K <= 0 || D <= 0 || F <= 0 || num_slots <= 0) return kRcBadArg;
  PlanBwdParams p{recv_rows, per_rank, saved_bytes_per_rank, buffer_offsets, peak_min_free, need_recompute,
                  fwd_state, bwd_offsets, moe_layer_id, ep, K, num_slots, num_tokens, D, F, slot_bytes, status};
  plan_bwd_bf16_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return static_cast<int>(cudaGetLastError());
}
