// Swapped-operand block-scaled grouped GEMM for experts that received few rows (decode).
//
//   C[r, n] = sum_k  (X[r,k] * sfx[r, k/V]) * (W[e][n,k] * sfw[e][n, k/V])        V = 32 (MXFP8) or 16 (NVFP4)
//
// The 128 x 256 kernel puts an expert's rows on the 128-row M side of tcgen05.mma, so an expert that received 30
// rows still pays for 128: at decode sizes the tensor pipe, not HBM, bounds the layer.  Here the roles are exchanged:
// 128 weight rows are the M side, the expert's rows are the N side in steps of 32 (at most 64 per tile), and the
// accumulator holds C transposed (TMEM lane = weight row, column = routed row).  A K stage then costs four MMAs of
// N = 32 or 64 and eight scale-atom copies, and the weights stream through once.
//
//   * with MMAs this short the limit is how fast one thread can issue tcgen05 instructions (50 to 100 cycles
//     each, measured; several issuing threads of one SM do not slow each other down).  So the scale-atom copies
//     and the MMAs of a stage are issued by two different threads (the copier commits to a per-stage barrier the
//     MMA thread waits on), and two CTAs share an SM, each with 256 TMEM columns and three stages;
//   * a stage = 128 bytes of K: 16 KiB of weights (one TMA box), 4 or 8 KiB of routed rows (32-row boxes),
//     and the stage's scale atoms of both;
//   * the rows' scale atom covers 128 rows in four TMEM columns of 32 rows each, so a tile that starts at row
//     32 q of its 128-row group names column q as its scale address: no separate scale layout for short tiles;
//   * epilogue: every thread owns one weight row (an output column); the warp transposes 32 x 32 values through
//     shared memory and writes 16-byte pieces of the output rows.  SwiGLU pairs lane l with lane l ^ 8, because a
//     prepared W13 alternates 8 gate rows with the matching 8 up rows.
//
// Forward only (inference has no backward); rows of every expert start at a multiple of 128 as the routing step
// lays them out, and `expert_counts` tells how many of them are real.
#include "gemm_common.cuh"

namespace dm {

constexpr int kSwStages = 3;
constexpr int kSwCtasPerSm = 2;
constexpr int kSwThreads = 256;  // TMA warp, MMA warp, four epilogue warps, accumulator watcher, scale copier
constexpr int kSwTileRows = 64;  // routed rows per tile (the MMA's N), in steps of 32
constexpr uint32_t kSwWBytes = 128 * 128;            // 16 KiB of weights
constexpr uint32_t kSwXBytes = kSwTileRows * 128;    // up to 8 KiB of routed rows
constexpr uint32_t kSwSfBytes = 2048;                // up to 4 atoms per operand
constexpr uint32_t kSwStageBytes = kSwWBytes + kSwXBytes + 2 * kSwSfBytes;  // 28 KiB
constexpr uint32_t kSwTransposeBytes = 32 * 32 * 2;  // per epilogue warp
constexpr size_t kSwSmemBytes = kSwStages * kSwStageBytes + 4 * kSwTransposeBytes + 1024;
constexpr uint32_t kSwTmemCols = 256;
constexpr uint32_t kSwSfTmemBase = 2 * kSwTileRows;  // then 32 scale columns per stage slot
static_assert(kSwSfTmemBase + kSwStages * 32 <= kSwTmemCols, "scale columns do not fit");
constexpr int kSwMaxGroups = 256;

struct SwParams {
  CUtensorMap tm_x;  // routed rows: (128 bytes, 128-byte lines of a row, rows), boxes of 32 rows
  CUtensorMap tm_w;  // weights: [e_local * N rows, row bytes], boxes of 128 rows
  const int64_t* x_off;
  const int64_t* sfx_off;
  const int64_t* c_off;
  const int64_t* h2_off;
  const int64_t* row_inv_off;
  const uint8_t* sfx_base;
  const uint8_t* sfw;
  const uint8_t* row_inv_base;  // fp32 per row (NVFP4 token scale inverse) or null
  const float* expert_inv;      // fp32 per expert (NVFP4 weight global scale inverse) or null
  uint8_t* c_base;
  uint8_t* h2_base;
  const int64_t* scatter_ptrs;
  const int32_t* expert_offsets;
  const int32_t* expert_counts;
  const int* cond;
  int* status;
  int64_t sfw_group_bytes;
  int e_local, max_rows, N, k_iters, fp4, swiglu, x_col_atoms, w_col_atoms;
  ActParams act;
};

struct SwTile {
  int e, m_blk, row0, n_valid;
};

__device__ __forceinline__ SwTile sw_decode(int tile, int& e, const int* tile_start, const int* off, const int* cnt,
                                            int m_tiles) {
  while (tile >= tile_start[e + 1]) ++e;
  const int local = tile - tile_start[e];
  const int n_blk = local / m_tiles;
  SwTile t;
  t.e = e;
  t.m_blk = local - n_blk * m_tiles;
  t.row0 = off[e] + n_blk * kSwTileRows;
  const int left = cnt[e] - n_blk * kSwTileRows;
  t.n_valid = left < kSwTileRows ? left : kSwTileRows;
  return t;
}

__global__ void __launch_bounds__(kSwThreads, kSwCtasPerSm) blockscaled_swapped_kernel(const __grid_constant__ SwParams p) {
  if (p.cond != nullptr && *p.cond == 0) return;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  __shared__ uint64_t full_bar[kSwStages];
  __shared__ uint64_t empty_bar[kSwStages];
  __shared__ uint64_t sf_bar[kSwStages];  // the stage's scale atoms are in TMEM
  __shared__ uint64_t tmem_full_bar[2];
  __shared__ uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int s_off[kSwMaxGroups + 1];
  __shared__ int s_cnt[kSwMaxGroups];
  __shared__ int s_tile_start[kSwMaxGroups + 1];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int m_tiles = p.N >> 7;
  const int atoms = p.fp4 ? 4 : 1;  // scale atoms per stage and operand

  for (int i = threadIdx.x; i <= p.e_local; i += blockDim.x) {
    const int v = p.expert_offsets[i];
    s_off[i] = v < p.max_rows ? v : p.max_rows;
  }
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kSwStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
      mbar_init(&sf_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], 4);
    }
    mbar_fence_init();
  }
  __syncthreads();
  for (int i = threadIdx.x; i < p.e_local; i += blockDim.x) {
    const int room = s_off[i + 1] - s_off[i];
    int c = p.expert_counts ? p.expert_counts[i] : room;
    c = c < room ? c : room;
    s_cnt[i] = c > 0 ? c : 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < p.e_local; ++e) {
      s_tile_start[e] = acc;
      if (s_cnt[e] > 0 && (s_off[e] & 127) != 0) set_status(p.status, kCapacityExceeded, -1, e, s_off[e]);
      acc += ((s_cnt[e] + kSwTileRows - 1) / kSwTileRows) * m_tiles;
    }
    s_tile_start[p.e_local] = acc;
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, kSwTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&p.tm_x);
    tma_prefetch_desc(&p.tm_w);
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const int total_tiles = s_tile_start[p.e_local];

  if (warp == 0) {
    // ======================= producer =======================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int e = 0;
      const int x_line0 = static_cast<int>((p.x_off ? *p.x_off : 0) >> 7);
      const uint8_t* sfx = p.sfx_base + (p.sfx_off ? *p.sfx_off : 0);
      const uint32_t sf_bytes = atoms * 512;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const SwTile t = sw_decode(tile, e, s_tile_start, s_off, s_cnt, m_tiles);
        const int nq = (t.n_valid + 31) >> 5;
        const uint8_t* sfw_row = p.sfw + t.e * p.sfw_group_bytes + static_cast<int64_t>(t.m_blk) * p.w_col_atoms * 512;
        const uint8_t* sfx_row = sfx + static_cast<int64_t>(t.row0 >> 7) * p.x_col_atoms * 512;
        for (int kb = 0; kb < p.k_iters && ok; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, &abort_flag);
          if (!ok) break;
          uint8_t* sw = smem + stage * kSwStageBytes;
          uint8_t* sx = sw + kSwWBytes;
          uint8_t* ssw = sx + kSwXBytes;
          uint8_t* ssx = ssw + kSwSfBytes;
          mbar_arrive_expect_tx(&full_bar[stage], kSwWBytes + nq * 4096u + 2 * sf_bytes);
          tma_load_2d(sw, &p.tm_w, kb * 128, t.e * p.N + t.m_blk * 128, &full_bar[stage]);
          for (int q = 0; q < nq; ++q)
            tma_load_3d(sx + q * 4096, &p.tm_x, 0, x_line0 + kb, t.row0 + 32 * q, &full_bar[stage]);
          bulk_load(ssw, sfw_row + static_cast<int64_t>(kb) * sf_bytes, sf_bytes, &full_bar[stage]);
          bulk_load(ssx, sfx_row + static_cast<int64_t>(kb) * sf_bytes, sf_bytes, &full_bar[stage]);
          if (++stage == kSwStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ======================= MMA issuer =======================
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int e = 0, it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        const SwTile t = sw_decode(tile, e, s_tile_start, s_off, s_cnt, m_tiles);
        const int n_mma = ((t.n_valid + 31) >> 5) * 32;
        const uint32_t col_off = static_cast<uint32_t>((t.row0 & 127) >> 5);  // the tile's 32-row group inside its atom
        const uint32_t idesc4 = umma_idesc_blockscaled(n_mma, 1, 0, 0);
        uint32_t idesc8[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) idesc8[j] = umma_idesc_blockscaled(n_mma, 0, j, j);
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        ok = mbar_wait(&tmem_empty_bar[buf], acc_phase ^ 1u, &abort_flag);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + buf * kSwTileRows;
        for (int kb = 0; kb < p.k_iters; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, &abort_flag) && mbar_wait(&sf_bar[stage], phase, &abort_flag);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t w_addr = smem_u32(smem + stage * kSwStageBytes), x_addr = w_addr + kSwWBytes;
          const uint32_t sfw_t = tmem_base + kSwSfTmemBase + stage * 32u;
          const uint32_t sfx_t = sfw_t + 16u;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t dw = umma_smem_desc(w_addr + j * 32u, 16, 1024);
            const uint64_t dx = umma_smem_desc(x_addr + j * 32u, 16, 1024);
            const uint32_t acc = (kb > 0 || j > 0) ? 1u : 0u;
            if (p.fp4)
              umma_nvf4(d_tmem, dw, dx, idesc4, sfw_t + 4 * j, sfx_t + 4 * j + col_off, acc);
            else
              umma_mxf8(d_tmem, dw, dx, idesc8[j], sfw_t, sfx_t + col_off, acc);
          }
          tcgen05_commit(&empty_bar[stage]);
          if (++stage == kSwStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (p.k_iters > 0)
          tcgen05_commit(&tmem_full_bar[buf]);
        else
          mbar_arrive(&tmem_full_bar[buf]);
      }
    }
    __syncwarp();
  } else if (warp == 7) {
    // ======================= scale copier =======================
    // Moves every stage's scale atoms from shared memory to the stage slot's TMEM columns.  The slot's previous
    // MMAs are complete by then: the producer refilled the stage only after their commit released it.
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < p.k_iters; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, &abort_flag);
          if (!ok) break;
          const uint32_t ssw = smem_u32(smem + stage * kSwStageBytes) + kSwWBytes + kSwXBytes, ssx = ssw + kSwSfBytes;
          const uint32_t sfw_t = tmem_base + kSwSfTmemBase + stage * 32u;
          const uint32_t sfx_t = sfw_t + 16u;
          for (int a = 0; a < atoms; ++a) {
            tmem_cp_sf_atom(sfw_t + 4 * a, sf_smem_desc(ssw + a * 512));
            tmem_cp_sf_atom(sfx_t + 4 * a, sf_smem_desc(ssx + a * 512));
          }
          tcgen05_commit(&sf_bar[stage]);
          if (++stage == kSwStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 6) {
    // ======================= accumulator watcher =======================
    // Polls the accumulator-ready barriers for the epilogue warps and releases them through a hardware named
    // barrier; it arrives for every tile, also after a timeout, so that no epilogue warp is left blocked.
    bool ok = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      if (ok && lane == 0) ok = mbar_wait(&tmem_full_bar[buf], acc_phase, &abort_flag);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      asm volatile("bar.arrive %0, %1;" ::"r"(1 + buf), "r"(4 * 32 + 32) : "memory");
    }
  } else {
    // ======================= epilogue =======================
    const int quad = warp & 3;
    uint16_t* tp = reinterpret_cast<uint16_t*>(smem + kSwStages * kSwStageBytes + (warp - 2) * kSwTransposeBytes);
    int e = 0, it = 0;
    bool ok = true;
    const int64_t c_off = p.c_off ? *p.c_off : 0;
    const int64_t h2_off = p.h2_off ? *p.h2_off : 0;
    const float* row_inv =
        p.row_inv_base ? reinterpret_cast<const float*>(p.row_inv_base + (p.row_inv_off ? *p.row_inv_off : 0)) : nullptr;
    const bool scaled = row_inv != nullptr || p.expert_inv != nullptr;
    const int F = p.N / 2;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      const SwTile t = sw_decode(tile, e, s_tile_start, s_off, s_cnt, m_tiles);
      const int buf = it & 1;
      asm volatile("bar.sync %0, %1;" ::"r"(1 + buf), "r"(4 * 32 + 32) : "memory");  // released by the watcher
      ok = abort_flag == 0;
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * kSwTileRows;
      const float escale = p.expert_inv ? p.expert_inv[t.e] : 1.0f;
      const int col0 = t.m_blk * 128 + quad * 32;  // first output column of this warp
      for (int c0 = 0; c0 < t.n_valid; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_ld_wait();
        // lane i looks after routed row c0 + i: its scale and its destination
        const int row = t.row0 + c0 + lane;
        const bool row_ok = c0 + lane < t.n_valid;
        const float my_scale = (row_inv != nullptr && row_ok) ? row_inv[row] : 1.0f;
        uint64_t my_dst = 0;
        if (row_ok) {
          if (p.swiglu)
            my_dst = reinterpret_cast<uint64_t>(p.h2_base) + h2_off + static_cast<uint64_t>(row) * F * 2;
          else if (p.scatter_ptrs != nullptr)
            my_dst = static_cast<uint64_t>(p.scatter_ptrs[row]);
          else
            my_dst = reinterpret_cast<uint64_t>(p.c_base) + c_off + static_cast<uint64_t>(row) * p.N * 2;
        }
        if (p.swiglu) {
          // lanes 0-7 and 16-23 hold gate rows, lane ^ 8 the matching up row: 16 features per warp
          const bool is_gate = (lane & 8) == 0;
          const int fl = (lane >> 4) * 8 + (lane & 7);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float v = __uint_as_float(r[i]);
            if (scaled) v = (v * __shfl_sync(0xffffffffu, my_scale, i)) * escale;
            const float vb = __uint_as_float(pack_bf16x2(0.0f, v) & 0xffff0000u);  // bf16-rounded, as h1 would hold it
            const float other = __shfl_xor_sync(0xffffffffu, vb, 8);
            if (is_gate) tp[i * 16 + fl] = static_cast<uint16_t>(pack_bf16x2(swiglu_f32(vb, other, p.act), 0.0f) & 0xffffu);
          }
          __syncwarp();
          const int f0 = col0 >> 1;
#pragma unroll
          for (int trip = 0; trip < 2; ++trip) {
            const int n = trip * 16 + (lane >> 1), ch = lane & 1;
            const uint4 v = *reinterpret_cast<const uint4*>(tp + n * 16 + ch * 8);
            const uint64_t rp = __shfl_sync(0xffffffffu, my_dst, n);
            if (rp != 0) *reinterpret_cast<uint4*>(rp + static_cast<uint64_t>(f0 + 8 * ch) * 2) = v;
          }
          __syncwarp();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float v = __uint_as_float(r[i]);
            if (scaled) v = (v * __shfl_sync(0xffffffffu, my_scale, i)) * escale;
            tp[i * 32 + lane] = static_cast<uint16_t>(pack_bf16x2(v, 0.0f) & 0xffffu);
          }
          __syncwarp();
#pragma unroll
          for (int trip = 0; trip < 4; ++trip) {
            const int n = trip * 8 + (lane >> 2), ch = lane & 3;
            const uint4 v = *reinterpret_cast<const uint4*>(tp + n * 32 + ch * 8);
            const uint64_t rp = __shfl_sync(0xffffffffu, my_dst, n);
            if (rp != 0) *reinterpret_cast<uint4*>(rp + static_cast<uint64_t>(col0 + 8 * ch) * 2) = v;
          }
          __syncwarp();
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[buf]);
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) set_status(p.status, kPipelineTimeout, 4, blockIdx.x);
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kSwTmemCols);
  }
}

}  // namespace dm

using namespace dm;

// Same contract as dm_gemm_blockscaled (forward, K-major weights) plus `expert_counts`, the real number of rows of
// every expert inside its 128-padded group (null: the whole group).  Rows past the count are neither read into an
// output nor written.
extern "C" int dm_gemm_blockscaled_swapped(int format, dm_operand a, dm_operand sfa, const void* w, const void* sfb,
                                           dm_operand c, dm_operand h2, const int64_t* scatter_ptrs,
                                           dm_operand row_scale_inv, const float* expert_scale_inv,
                                           const int32_t* expert_offsets, const int32_t* expert_counts, int e_local,
                                           int64_t max_rows, int64_t N, int64_t Kd, int swiglu_interleaved, int clamped,
                                           float alpha, float limit, const int* cond, int num_sms, int* status,
                                           void* stream) {
  if (!a.base || !sfa.base || !w || !sfb || !expert_offsets || e_local <= 0 || max_rows < 0 || N <= 0 || Kd <= 0)
    return kRcBadArg;
  if (format != 0 && format != 1) return kRcBadArg;
  if (!swiglu_interleaved && !c.base && !scatter_ptrs) return kRcBadArg;
  if (swiglu_interleaved && (!h2.base || scatter_ptrs || c.base)) return kRcBadArg;
  if (e_local > kSwMaxGroups || max_rows > (1 << 30)) return kRcTooLarge;
  const int fp4 = format == 1;
  const int64_t row_bytes = fp4 ? Kd / 2 : Kd;
  if ((row_bytes % 128) != 0 || (N % 128) != 0 || (max_rows % 128) != 0) return kRcUnsupportedShape;
  if (max_rows == 0) return kRcOk;
  static PerDeviceOnce attr_set;
  int rc = once_per_device(attr_set, [] {
    return static_cast<int>(cudaFuncSetAttribute(blockscaled_swapped_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(kSwSmemBytes)));
  });
  if (rc != kRcOk) return rc;
  SwParams p{};
  rc = encode_arena_u8(&p.tm_x, a, row_bytes, max_rows + 256, 32);
  if (rc != kRcOk) return rc;
  rc = encode_2d_u8(&p.tm_w, w, static_cast<int64_t>(e_local) * N, row_bytes, 128);
  if (rc != kRcOk) return rc;
  const int64_t scale_cols = Kd / (fp4 ? 16 : 32);
  p.x_col_atoms = static_cast<int>((scale_cols + 3) / 4);
  p.w_col_atoms = p.x_col_atoms;
  p.sfw_group_bytes = (N + 127) / 128 * 128 * static_cast<int64_t>(p.w_col_atoms) * 4;
  p.x_off = a.offset;
  p.sfx_off = sfa.offset;
  p.sfx_base = static_cast<const uint8_t*>(sfa.base);
  p.sfw = static_cast<const uint8_t*>(sfb);
  p.c_off = c.offset;
  p.h2_off = h2.offset;
  p.c_base = static_cast<uint8_t*>(c.base);
  p.h2_base = static_cast<uint8_t*>(h2.base);
  p.row_inv_base = static_cast<const uint8_t*>(row_scale_inv.base);
  p.row_inv_off = row_scale_inv.offset;
  p.expert_inv = expert_scale_inv;
  p.scatter_ptrs = scatter_ptrs;
  p.expert_offsets = expert_offsets;
  p.expert_counts = expert_counts;
  p.cond = cond;
  p.status = status;
  p.e_local = e_local;
  p.max_rows = static_cast<int>(max_rows);
  p.N = static_cast<int>(N);
  p.k_iters = static_cast<int>(row_bytes / 128);
  p.fp4 = fp4;
  p.swiglu = swiglu_interleaved ? 1 : 0;
  p.act = ActParams{clamped, alpha, limit};
  blockscaled_swapped_kernel<<<kSwCtasPerSm * persistent_grid(num_sms), kSwThreads, kSwSmemBytes, static_cast<cudaStream_t>(stream)>>>(p);
  return static_cast<int>(cudaGetLastError());
}
