// Persistent grouped block-scaled GEMMs (MXFP8 E4M3 / NVFP4) on tcgen05 with scale factors in TMEM.
//
//   C[r, n] = sum_k  (A[r,k] * sfa[r, k/V]) * (W[e][n,k] * sfb[e][n, k/V])        V = 32 (MXFP8) or 16 (NVFP4)
//
// Same warp-specialised skeleton as the BF16 kernel (TMA producer warp, one MMA-issuing lane, eight
// epilogue warps, one 128 x 256 fp32 accumulator in TMEM).  Differences:
//   * a pipeline stage is 128 bytes of K per row: 128 E4M3 or 256 packed E2M1 elements;
//   * next to the A/B tiles the producer bulk-copies the stage's scale atoms.  Scales are
//     stored in 128-row x 4-column atoms of 512 bytes (row r, column c at (r%32)*16 + (r/32)*4 + c),
//     which is exactly the 32-row x 16-byte source shape of tcgen05.cp ... 32x128b.warpx4, so an atom
//     goes to TMEM with one instruction and no shuffling;
//   * per K step the MMA names the TMEM scale columns (NVFP4: one atom per K=64 step) or the
//     scale byte inside them (MXFP8: a_sf_id / b_sf_id = K=32 step index);
//   * rows of every expert are padded to 128 by the routing step, so tiles and scale atoms align.
//
// Epilogues: plain bf16 rows (optionally scaled by the per-token and per-expert NVFP4 inverse
// scales, optionally scattered to per-row destinations), or SwiGLU over a W13 whose rows were
// interleaved in groups of 8 gate / 8 up rows at preparation time, producing bf16 h2 (and h1).
#include "gemm_common.cuh"
#include "quant_common.cuh"

namespace dm {

constexpr int kBsBM = 128;
constexpr int kBsBN = 128;
constexpr uint32_t kBsABytes = kBsBM * 128;  // 16 KiB
constexpr uint32_t kBsTmemCols = 512;
constexpr int kBsMaxGroups = 256;

struct BsParams {
  CUtensorMap tm_a;
  CUtensorMap tm_b;
  CUtensorMap tm_c;  // weight gradient: dW as [e_local][rows][cols], boxes of 16 rows x 128 bytes
  const int64_t* a_off;
  const int64_t* sfa_off;
  const int64_t* c_off;
  const int64_t* h2_off;
  const int64_t* row_inv_off;
  const uint8_t* sfa_base;
  const uint8_t* sfb;
  const uint8_t* row_inv_base;  // fp32 per row (NVFP4 token scale inverse) or null
  const float* expert_inv;      // fp32 per expert (NVFP4 weight global scale inverse) or null
  uint8_t* c_base;
  uint8_t* h2_base;
  const int64_t* scatter_ptrs;
  const int32_t* expert_offsets;
  const int* cond;
  int* status;
  int64_t sfb_group_bytes;
  int e_local, max_rows, N, k_iters, fp4, swiglu, a_col_atoms, b_col_atoms, compact_cols;
  int mode;       // 0 fprop (A, W K-major), 1 dgrad (W N-major), 2 wgrad (both operands MN-major, K = expert rows)
  int Kw;         // dgrad: rows of one expert's W (the contraction extent); wgrad: dW columns
  int out_fp32, accumulate;
  // SwiGLU epilogue of the 128 x 256 kernel writing h2 as MXFP8 rows (E4M3 bytes + blocked E8M0 scales) instead of bf16
  uint8_t* hq_base;
  const int64_t* hq_off;
  uint8_t* hsf_base;
  const int64_t* hsf_off;
  int h_atoms;
  int direct_store;  // NVFP4 SwiGLU forward without staging tiles (four stages)
  const int64_t* b_off;
  const int64_t* sfb_off;
  ActParams act;
};

struct BsTile {
  int e, m_blk, n_blk, row0, row_end, k_iters;
};

__device__ __forceinline__ BsTile bs_decode(int tile, int& e, const int* tile_start, const int* off, int mode,
                                            int n_tiles, int k_iters) {
  while (tile >= tile_start[e + 1]) ++e;
  const int local = tile - tile_start[e];
  const int rows = off[e + 1] - off[e];
  BsTile t;
  t.e = e;
  if (mode == 2) {
    t.n_blk = local % n_tiles;
    t.m_blk = local / n_tiles;
    t.row0 = off[e];
    t.row_end = off[e + 1];
    t.k_iters = (rows + 127) / 128;
    return t;
  }
  const int m_tiles = (rows + kBsBM - 1) / kBsBM;
  t.m_blk = local % m_tiles;
  t.n_blk = local / m_tiles;
  t.row0 = off[e] + t.m_blk * kBsBM;
  t.row_end = off[e + 1];
  t.k_iters = k_iters;
  return t;
}

// ---------------------------------------------------------------------------------------------------------
// 128 x 256 output tiles.  Per 128 bytes of K the tile moves 48 KiB of operands and needs, for NVFP4, twelve
// scale-atom copies (about 47 cycles each, they serialise with the MMAs) per four 132-cycle MMAs; a 128 x 128
// tile would spend more tensor-pipe time on its eight copies than on its four 69-cycle MMAs.  TMEM holds one
// 256-column accumulator plus two buffers of scale columns, so the epilogue (eight warps, a few thousand
// cycles) does not overlap the next tile's MMAs; tiles here are tens of thousands of cycles long.  Experts
// with few rows take the swapped-operand kernel instead (gemm_blockscaled_swapped.cu).
// ---------------------------------------------------------------------------------------------------------
constexpr int kWdBN = 256;
constexpr int kWdThreads = 384;  // TMA warp, MMA warp, eight epilogue warps, accumulator watcher, scale copier
constexpr uint32_t kWdBBytes = kWdBN * 128;                                   // 32 KiB
constexpr uint32_t kWdStageFp4 = kBsABytes + kWdBBytes + 2048 + 4096;         // 54 KiB: 4 + 8 scale atoms
constexpr uint32_t kWdStageFp8 = kBsABytes + kWdBBytes + 2048;                // 50 KiB: 1 + 2 scale atoms, padded
constexpr int kWdStagesFp4 = 3;
constexpr int kWdStagesFp8 = 4;
constexpr int kWdMaxStages = 4;
constexpr uint32_t kWdSfTmemBase = kWdBN;  // scale columns: 64 per stage slot after the accumulator
static_assert(kWdSfTmemBase + kWdMaxStages * 64 <= kBsTmemCols, "scale columns do not fit");
constexpr size_t kWdSmemFp4 = kWdStagesFp4 * kWdStageFp4 + 8 * kStaging64Bytes + 1024;
// NVFP4 forward with the SwiGLU epilogue and no h1 output: every lane stores its own 64 bytes of h2 per block
// straight from registers, the staging tiles go, and a fourth stage fits.  Three 54 KiB stages do not cover the load
// latency plus the scale-copy phase; the stores of this form are less coalesced but run while the next tile's MMAs do.
constexpr int kWdStagesFp4Direct = 4;
constexpr size_t kWdSmemFp4Direct = kWdStagesFp4Direct * kWdStageFp4 + 1024;
constexpr size_t kWdSmemFp8 = kWdStagesFp8 * kWdStageFp8 + 8 * kStaging64Bytes + 1024;

__global__ void __launch_bounds__(kWdThreads, 1) blockscaled_wide_kernel(const __grid_constant__ BsParams p) {
  if (p.cond != nullptr && *p.cond == 0) return;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  __shared__ uint64_t full_bar[kWdMaxStages];
  __shared__ uint64_t empty_bar[kWdMaxStages];
  __shared__ uint64_t sf_bar[kWdMaxStages];  // the stage's scale atoms are in TMEM
  __shared__ uint64_t tmem_full_bar;
  __shared__ uint64_t tmem_empty_bar;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int s_off[kBsMaxGroups + 1];
  __shared__ int s_tile_start[kBsMaxGroups + 1];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_tiles = p.mode == 2 ? (p.Kw + kWdBN - 1) / kWdBN : (p.N + kWdBN - 1) / kWdBN;
  const int wgrad_m_tiles = (p.N + kBsBM - 1) / kBsBM;
  const int atoms = p.fp4 ? 4 : 1;  // scale atoms per stage and 128 rows
  const int stages = p.fp4 ? (p.direct_store ? kWdStagesFp4Direct : kWdStagesFp4) : kWdStagesFp8;
  const uint32_t stage_bytes = p.fp4 ? kWdStageFp4 : kWdStageFp8;

  for (int i = threadIdx.x; i <= p.e_local; i += blockDim.x) {
    const int v = p.expert_offsets[i];
    s_off[i] = v < p.max_rows ? v : p.max_rows;
  }
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kWdMaxStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
      mbar_init(&sf_bar[s], p.fp4 ? 2 : 1);  // NVFP4: two copier threads share the stage's atoms
    }
    mbar_init(&tmem_full_bar, 1);
    mbar_init(&tmem_empty_bar, 8);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < p.e_local; ++e) {
      s_tile_start[e] = acc;
      const int rows = s_off[e + 1] - s_off[e];
      if ((s_off[e] & 127) != 0) set_status(p.status, kCapacityExceeded, -1, e, s_off[e]);  // rows must be 128-padded
      acc += p.mode == 2 ? wgrad_m_tiles * n_tiles : ((rows + kBsBM - 1) / kBsBM) * n_tiles;
    }
    s_tile_start[p.e_local] = acc;
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, kBsTmemCols);
    tmem_relinquish();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&p.tm_a);
    tma_prefetch_desc(&p.tm_b);
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
      const int a_line0 = static_cast<int>((p.a_off ? *p.a_off : 0) >> 7);
      const int b_line0 = static_cast<int>((p.b_off ? *p.b_off : 0) >> 7);
      const uint8_t* sfa = p.sfa_base + (p.sfa_off ? *p.sfa_off : 0);
      const uint8_t* sfb_dyn = p.sfb + (p.sfb_off ? *p.sfb_off : 0);
      const uint32_t sf_bytes = atoms * 512;
      const int row_blocks = ((p.mode == 2 ? p.Kw : p.N) + 127) >> 7;  // 128-wide blocks of the B side
      int a_col_atoms = p.a_col_atoms, b_col_atoms = p.b_col_atoms;
      // column bundles sized by the device row count: their scale layout has rows/128 column atoms
      if (p.mode == 2 && p.compact_cols) a_col_atoms = b_col_atoms = ((s_off[p.e_local] + 31) / 32 + 3) / 4;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const BsTile t = bs_decode(tile, e, s_tile_start, s_off, p.mode, n_tiles, p.k_iters);
        const uint8_t* sfa_row;
        const uint8_t* sfb_row0;
        if (p.mode == 2) {
          // scales of the column-quantised operands: rows = features, columns = 32-row blocks of the packed rows
          sfa_row = sfa + (static_cast<int64_t>(t.m_blk) * a_col_atoms + (t.row0 >> 7)) * 512;
          sfb_row0 = sfb_dyn + (static_cast<int64_t>(t.n_blk * 2) * b_col_atoms + (t.row0 >> 7)) * 512;
        } else {
          sfa_row = sfa + static_cast<int64_t>(t.row0 >> 7) * a_col_atoms * 512;
          sfb_row0 = p.sfb + t.e * p.sfb_group_bytes + static_cast<int64_t>(t.n_blk * 2) * b_col_atoms * 512;
        }
        const uint8_t* sfb_row1 = sfb_row0 + static_cast<int64_t>(b_col_atoms) * 512;
        const bool second = t.n_blk * 2 + 1 < row_blocks;  // the tile's upper 128 columns exist
        for (int kb = 0; kb < t.k_iters && ok; ++kb) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, &abort_flag);
          if (!ok) break;
          uint8_t* sa = smem + stage * stage_bytes;
          uint8_t* sb = sa + kBsABytes;
          uint8_t* ssa = sb + kWdBBytes;
          uint8_t* ssb = ssa + sf_bytes;
          if (p.mode == 0) {
            mbar_arrive_expect_tx(&full_bar[stage], kBsABytes + kWdBBytes + (second ? 3 : 2) * sf_bytes);
            tma_load_3d(sa, &p.tm_a, 0, a_line0 + kb, t.row0, &full_bar[stage]);
            tma_load_2d(sb, &p.tm_b, kb * 128, t.e * p.N + t.n_blk * kWdBN, &full_bar[stage]);
          } else {
            // B arrives as two 128-byte-wide boxes of 128 K rows (MN-major); the upper one only where it exists
            mbar_arrive_expect_tx(&full_bar[stage], kBsABytes + (second ? kWdBBytes + 3 * sf_bytes : kWdBBytes / 2 + 2 * sf_bytes));
            if (p.mode == 1) {
              tma_load_3d(sa, &p.tm_a, 0, a_line0 + kb, t.row0, &full_bar[stage]);
              tma_load_2d(sb, &p.tm_b, t.n_blk * kWdBN, t.e * p.Kw + kb * 128, &full_bar[stage]);
              if (second) tma_load_2d(sb + kWdBBytes / 2, &p.tm_b, t.n_blk * kWdBN + 128, t.e * p.Kw + kb * 128, &full_bar[stage]);
            } else {
              tma_load_3d(sa, &p.tm_a, 0, a_line0 + t.m_blk, t.row0 + kb * 128, &full_bar[stage]);
              tma_load_3d(sb, &p.tm_b, 0, b_line0 + t.n_blk * 2, t.row0 + kb * 128, &full_bar[stage]);
              if (second) tma_load_3d(sb + kWdBBytes / 2, &p.tm_b, 0, b_line0 + t.n_blk * 2 + 1, t.row0 + kb * 128, &full_bar[stage]);
            }
          }
          bulk_load(ssa, sfa_row + static_cast<int64_t>(kb) * sf_bytes, sf_bytes, &full_bar[stage]);
          bulk_load(ssb, sfb_row0 + static_cast<int64_t>(kb) * sf_bytes, sf_bytes, &full_bar[stage]);
          if (second) bulk_load(ssb + sf_bytes, sfb_row1 + static_cast<int64_t>(kb) * sf_bytes, sf_bytes, &full_bar[stage]);
          if (++stage == stages) {
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
      const int a_mn = p.mode == 2, b_mn = p.mode != 0;
      const uint32_t a_step = a_mn ? 4096u : 32u, b_step = b_mn ? 4096u : 32u;
      const uint32_t b_lbo = b_mn ? kWdBBytes / 2 : 16u;  // MN-major: the two 128-byte-wide halves are 16 KiB apart
      const uint32_t idesc4 = umma_idesc_blockscaled(kWdBN, 1, 0, 0);
      uint32_t idesc8[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) idesc8[j] = umma_idesc_blockscaled(kWdBN, 0, j, j, a_mn, b_mn);
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
        const BsTile t = bs_decode(tile, e, s_tile_start, s_off, p.mode, n_tiles, p.k_iters);
        ok = mbar_wait(&tmem_empty_bar, (it & 1u) ^ 1u, &abort_flag);  // the epilogue has drained the accumulator
        if (!ok) break;
        tcgen05_fence_after();
        for (int kb = 0; kb < t.k_iters; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, &abort_flag) && mbar_wait(&sf_bar[stage], phase, &abort_flag);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * stage_bytes), b_addr = a_addr + kBsABytes;
          const uint32_t sfa_t = tmem_base + kWdSfTmemBase + stage * 64u;
          const uint32_t sfb_t = sfa_t + 16u;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint64_t da = umma_smem_desc(a_addr + j * a_step, 16, 1024);
            const uint64_t db = umma_smem_desc(b_addr + j * b_step, b_lbo, 1024);
            const uint32_t acc = (kb > 0 || j > 0) ? 1u : 0u;
            if (p.fp4)
              umma_nvf4(tmem_base, da, db, idesc4, sfa_t + 4 * j, sfb_t + 8 * j, acc);
            else
              umma_mxf8(tmem_base, da, db, idesc8[j], sfa_t, sfb_t, acc);
          }
          tcgen05_commit(&empty_bar[stage]);
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (t.k_iters > 0)
          tcgen05_commit(&tmem_full_bar);
        else
          mbar_arrive(&tmem_full_bar);
      }
    }
    __syncwarp();
  } else if (warp == 11 || warp == 10) {
    // ======================= scale copiers (the second one is also the accumulator watcher) =======================
    // A thread issues a tcgen05 instruction every 50 to 100 cycles, and an NVFP4 stage needs twelve scale-atom
    // copies next to its four MMAs; issued by one thread they cost more than the tensor pipe needs to run them.
    // These two threads move every stage's atoms to the stage slot's TMEM columns and commit to a per-stage
    // barrier the MMA thread waits on.  Columns: A atom a (K step a) at +4a; B atoms of the tile's lower and
    // upper 128 columns side by side, 8 columns per K step.  The slot's previous MMAs are complete by then: the
    // producer refilled the stage only after their commit released it.  NVFP4 has four atoms per stage and
    // operand and each thread takes two; MXFP8 has one, taken by warp 11.
    //
    // Warp 10 then polls the accumulator-ready barrier for the epilogue warps and releases them through a hardware
    // named barrier; it arrives for every tile, also after a timeout, so that no epilogue warp is left blocked.
    const bool watcher = warp == 10;
    const int a_lo = watcher ? 2 : 0, a_hi = p.fp4 ? a_lo + 2 : (watcher ? 0 : 1);
    int stage = 0;
    uint32_t phase = 0;
    int e = 0, it = 0;
    bool ok = true;
    const uint32_t sf_bytes = atoms * 512;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      if (lane == 0 && a_hi > a_lo && ok) {
        const BsTile t = bs_decode(tile, e, s_tile_start, s_off, p.mode, n_tiles, p.k_iters);
        for (int kb = 0; kb < t.k_iters; ++kb) {
          ok = mbar_wait(&full_bar[stage], phase, &abort_flag);
          if (!ok) break;
          const uint32_t ssa = smem_u32(smem + stage * stage_bytes) + kBsABytes + kWdBBytes, ssb = ssa + sf_bytes;
          const uint32_t sfa_t = tmem_base + kWdSfTmemBase + stage * 64u;
          const uint32_t sfb_t = sfa_t + 16u;
          for (int a = a_lo; a < a_hi; ++a) {
            tmem_cp_sf_atom(sfa_t + 4 * a, sf_smem_desc(ssa + a * 512));
            tmem_cp_sf_atom(sfb_t + 8 * a, sf_smem_desc(ssb + a * 512));
            tmem_cp_sf_atom(sfb_t + 8 * a + 4, sf_smem_desc(ssb + sf_bytes + a * 512));
          }
          tcgen05_commit(&sf_bar[stage]);
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
      if (watcher) {
        if (ok && lane == 0) ok = mbar_wait(&tmem_full_bar, it & 1u, &abort_flag);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        asm volatile("bar.arrive %0, %1;" ::"r"(1 + (it & 1)), "r"(8 * 32 + 32) : "memory");
      }
    }
    __syncwarp();
  } else {
    // ======================= epilogue =======================
    // Eight warps: two per TMEM lane quadrant, each owning 128 of the tile's 256 columns.  A lane reads its own
    // accumulator row; the warp transposes 32 x 32 blocks through its staging tile and stores 64-byte row segments.
    const int ew = warp - 2;
    const int quad = warp & 3;
    const int half = ew >> 2;
    const int row_in_tile = quad * 32 + lane;
    uint8_t* stg = smem + stages * stage_bytes + ew * kStaging64Bytes;
    int e = 0, it = 0;
    bool ok = true;
    const int64_t c_off = p.c_off ? *p.c_off : 0;
    const int64_t h2_off = p.h2_off ? *p.h2_off : 0;
    const float* row_inv =
        p.row_inv_base ? reinterpret_cast<const float*>(p.row_inv_base + (p.row_inv_off ? *p.row_inv_off : 0)) : nullptr;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      const BsTile t = bs_decode(tile, e, s_tile_start, s_off, p.mode, n_tiles, p.k_iters);
      asm volatile("bar.sync %0, %1;" ::"r"(1 + (it & 1)), "r"(8 * 32 + 32) : "memory");  // released by the watcher
      ok = abort_flag == 0;
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
      if (p.mode == 2) {
        // weight gradient: dW[e][m][n], overwrite or accumulate (fp32 or bf16 destination)
        uint32_t ra[32], rb[32], rc[32], rd[32];
        if (t.k_iters > 0) {
          tmem_ld_32x32(taddr + half * (kWdBN / 2), ra);
          tmem_ld_32x32(taddr + half * (kWdBN / 2) + 32, rb);
          tmem_ld_32x32(taddr + half * (kWdBN / 2) + 64, rc);
          tmem_ld_32x32(taddr + half * (kWdBN / 2) + 96, rd);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) ra[j] = rb[j] = rc[j] = rd[j] = 0u;
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty_bar);  // accumulator handed back before the stores
        // 128 bytes of output columns per trip (64 bf16 or 32 fp32).  The staging tile is laid out as a 16-row x
        // 128-byte box in the 128-byte swizzle, so the warp's 32 rows go in two passes; one thread hands each box
        // to the copy engine, which stores it or adds it to dW in L2 in whole 128-byte lines and clips rows and
        // columns past the matrix.
        const int col0 = t.n_blk * kWdBN + half * (kWdBN / 2);
        auto send = [&](int cc, int pass) {
          fence_proxy_async_smem();
          __syncwarp();
          const int box_row = t.m_blk * kBsBM + quad * 32 + pass * 16;
          if (lane == 0 && box_row < p.N && cc < p.Kw) {
            if (p.accumulate)
              tma_reduce_add_3d(&p.tm_c, stg, cc, box_row, t.e);
            else
              tma_store_3d(&p.tm_c, stg, cc, box_row, t.e);
            bulk_commit();
          }
        };
        if (p.out_fp32) {
#pragma unroll
          for (int trip = 0; trip < 4; ++trip) {
            uint32_t (&r)[32] = trip == 0 ? ra : (trip == 1 ? rb : (trip == 2 ? rc : rd));
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
              if (lane == 0) bulk_wait_read();  // the engine has read the previous box out of the staging tile
              __syncwarp();
              if ((lane >> 4) == pass) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  stage_put(stg, lane & 15, j, make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]));
              }
              send(col0 + 32 * trip, pass);
            }
          }
        } else {
#pragma unroll
          for (int trip = 0; trip < 2; ++trip) {
            uint32_t (&r0)[32] = trip == 0 ? ra : rc;
            uint32_t (&r1)[32] = trip == 0 ? rb : rd;
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
              if (lane == 0) bulk_wait_read();
              __syncwarp();
              if ((lane >> 4) == pass) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  stage_put(stg, lane & 15, j, pack8_bf16(r0 + 8 * j));
                  stage_put(stg, lane & 15, j + 4, pack8_bf16(r1 + 8 * j));
                }
              }
              send(col0 + 64 * trip, pass);
            }
          }
        }
        continue;
      }
      const int row = t.row0 + row_in_tile;
      const bool row_ok = row < t.row_end;
      float scale = 1.0f;
      bool scaled = false;
      if (row_inv != nullptr && row_ok) {
        scale = row_inv[row];
        scaled = true;
      }
      const float escale = p.expert_inv ? p.expert_inv[t.e] : 1.0f;
      scaled = scaled || p.expert_inv != nullptr;
      if (p.swiglu) {
        // Columns come in groups of 16: 8 gate features then the matching 8 up features.
        const int F = p.N / 2;
        const uint64_t my_h2 =
            row_ok ? reinterpret_cast<uint64_t>(p.h2_base) + h2_off + static_cast<uint64_t>(row) * F * 2 : 0ull;
        const uint64_t my_h1 = (row_ok && p.c_base)
                                   ? reinterpret_cast<uint64_t>(p.c_base) + c_off + static_cast<uint64_t>(row) * p.N * 2
                                   : 0ull;
        // Drain this warp's 128 columns into registers and hand the accumulator back at once: the SwiGLU
        // arithmetic and the stores below then run while the next tile's MMAs fill the accumulator again.
        uint32_t ra[32], rb[32], rc[32], rd[32];
        tmem_ld_32x32(taddr + half * (kWdBN / 2), ra);
        tmem_ld_32x32(taddr + half * (kWdBN / 2) + 32, rb);
        tmem_ld_32x32(taddr + half * (kWdBN / 2) + 64, rc);
        tmem_ld_32x32(taddr + half * (kWdBN / 2) + 96, rd);
        tmem_ld_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty_bar);
#pragma unroll
        for (int blk = 0; blk < 2; ++blk) {
          const int c0 = half * (kWdBN / 2) + 64 * blk;
          uint32_t (&r0)[32] = blk == 0 ? ra : rc;
          uint32_t (&r1)[32] = blk == 0 ? rb : rd;
          uint4 zv[4], gv[4], uv[4];
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint32_t gw[4], uw[4], zw[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int b = 16 * (g & 1) + 2 * q;
              float g0 = __uint_as_float(g < 2 ? r0[b] : r1[b]), g1 = __uint_as_float(g < 2 ? r0[b + 1] : r1[b + 1]);
              float u0 = __uint_as_float(g < 2 ? r0[b + 8] : r1[b + 8]), u1 = __uint_as_float(g < 2 ? r0[b + 9] : r1[b + 9]);
              if (scaled) {
                g0 = (g0 * scale) * escale; g1 = (g1 * scale) * escale;
                u0 = (u0 * scale) * escale; u1 = (u1 * scale) * escale;
              }
              gw[q] = pack_bf16x2(g0, g1);
              uw[q] = pack_bf16x2(u0, u1);
              const float z0 = swiglu_f32(__uint_as_float(gw[q] << 16), __uint_as_float(uw[q] << 16), p.act);
              const float z1 =
                  swiglu_f32(__uint_as_float(gw[q] & 0xffff0000u), __uint_as_float(uw[q] & 0xffff0000u), p.act);
              zw[q] = pack_bf16x2(z0, z1);
            }
            zv[g] = make_uint4(zw[0], zw[1], zw[2], zw[3]);
            gv[g] = make_uint4(gw[0], gw[1], gw[2], gw[3]);
            uv[g] = make_uint4(uw[0], uw[1], uw[2], uw[3]);
          }
          const int f0 = t.n_blk * (kWdBN / 2) + c0 / 2;  // first of the 32 features of this block
          if (p.hq_base != nullptr) {
            // The lane holds one whole 1 x 32 block of its h2 row (already rounded to bf16): quantise it here, as
            // the row quantiser would from the stored bf16 values, and store 32 E4M3 bytes and the block's scale.
            if (row_ok && f0 + 32 <= F) {
              const uint32_t zw[16] = {zv[0].x, zv[0].y, zv[0].z, zv[0].w, zv[1].x, zv[1].y, zv[1].z, zv[1].w,
                                       zv[2].x, zv[2].y, zv[2].z, zv[2].w, zv[3].x, zv[3].y, zv[3].z, zv[3].w};
              uint32_t m = 0;
#pragma unroll
              for (int j = 0; j < 16; ++j) m = __vmaxu2(m, zw[j] & 0x7fff7fffu);
              const uint32_t top = (m >> 16) > (m & 0xffffu) ? (m >> 16) : (m & 0xffffu);
              float recip;
              const uint8_t byte = mxfp8_scale(amax_from_bf16_bits(top), recip);
              uint32_t o[8];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                o[j] = e4m3x4(__uint_as_float(zw[2 * j] << 16) * recip, __uint_as_float(zw[2 * j] & 0xffff0000u) * recip,
                              __uint_as_float(zw[2 * j + 1] << 16) * recip,
                              __uint_as_float(zw[2 * j + 1] & 0xffff0000u) * recip);
              uint4* dst = reinterpret_cast<uint4*>(p.hq_base + (p.hq_off ? *p.hq_off : 0) +
                                                    static_cast<int64_t>(row) * F + f0);
              dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
              dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
              (p.hsf_base + (p.hsf_off ? *p.hsf_off : 0))[blocked_offset(row, f0 >> 5, p.h_atoms)] = byte;
            }
            continue;
          }
          if (p.direct_store) {
            if (my_h2 != 0) {
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (f0 + 8 * j + 8 <= F) *reinterpret_cast<uint4*>(my_h2 + static_cast<uint64_t>(f0 + 8 * j) * 2) = zv[j];
            }
            continue;
          }
#pragma unroll
          for (int which = 0; which < 3; ++which) {
            if (which > 0 && p.c_base == nullptr) break;
#pragma unroll
            for (int j = 0; j < 4; ++j) stage64_put(stg, lane, j, which == 0 ? zv[j] : (which == 1 ? gv[j] : uv[j]));
            __syncwarp();
            const uint64_t base = which == 0 ? my_h2 : my_h1;
            const int col_out = which == 2 ? F + f0 : f0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int rr = i * 8 + (lane >> 2), j = lane & 3;
              const uint4 v = stage64_get(stg, rr, j);
              const uint64_t rp = __shfl_sync(0xffffffffu, base, rr);
              if (rp != 0 && f0 + 8 * j + 8 <= F)
                *reinterpret_cast<uint4*>(rp + static_cast<uint64_t>(col_out + 8 * j) * 2) = v;
            }
            __syncwarp();
          }
        }
      } else {
        uint64_t my_row = 0;
        if (row_ok) {
          if (p.scatter_ptrs != nullptr)
            my_row = static_cast<uint64_t>(p.scatter_ptrs[row]);
          else
            my_row = reinterpret_cast<uint64_t>(p.c_base) + c_off + static_cast<uint64_t>(row) * p.N * 2;
        }
        uint32_t ra[32], rb[32], rc[32], rd[32];
        tmem_ld_32x32(taddr + half * (kWdBN / 2), ra);
        tmem_ld_32x32(taddr + half * (kWdBN / 2) + 32, rb);
        tmem_ld_32x32(taddr + half * (kWdBN / 2) + 64, rc);
        tmem_ld_32x32(taddr + half * (kWdBN / 2) + 96, rd);
        tmem_ld_wait();
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty_bar);  // accumulator handed back, see above
#pragma unroll
        for (int blk = 0; blk < 4; ++blk) {
          const int c0 = half * (kWdBN / 2) + 32 * blk;
          uint32_t (&r)[32] = blk == 0 ? ra : (blk == 1 ? rb : (blk == 2 ? rc : rd));
          if (scaled) {
#pragma unroll
            for (int j = 0; j < 32; ++j) r[j] = __float_as_uint((__uint_as_float(r[j]) * scale) * escale);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) stage64_put(stg, lane, j, pack8_bf16(r + 8 * j));
          __syncwarp();
          const int col = t.n_blk * kWdBN + c0;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int rr = i * 8 + (lane >> 2), j = lane & 3;
            const uint4 v = stage64_get(stg, rr, j);
            const uint64_t rp = __shfl_sync(0xffffffffu, my_row, rr);
            if (rp != 0 && col + 8 * j + 8 <= p.N)
              *reinterpret_cast<uint4*>(rp + static_cast<uint64_t>(col + 8 * j) * 2) = v;
          }
          __syncwarp();
        }
      }
    }
  }

  tcgen05_fence_before();
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) set_status(p.status, kPipelineTimeout, 4, blockIdx.x);
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kBsTmemCols);
  }
}

}  // namespace dm

using namespace dm;

// Launches the 128 x 256 kernel.
static int bs_launch(const BsParams& p, int num_sms, cudaStream_t st) {
  const int grid = persistent_grid(num_sms);
  static PerDeviceOnce wide_attr_set;
  const int rc = once_per_device(wide_attr_set, [] {
    return static_cast<int>(cudaFuncSetAttribute(blockscaled_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(kWdSmemFp4Direct)));
  });
  if (rc != 0) return rc;
  static_assert(kWdSmemFp4Direct >= kWdSmemFp4 && kWdSmemFp4Direct >= kWdSmemFp8, "largest shared-memory request");
  const size_t smem = p.fp4 ? (p.direct_store ? kWdSmemFp4Direct : kWdSmemFp4) : kWdSmemFp8;
  blockscaled_wide_kernel<<<grid, kWdThreads, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_gemm_blockscaled(int format, dm_operand a, dm_operand sfa, const void* w, const void* sfb,
                                   dm_operand c, dm_operand h2, const int64_t* scatter_ptrs, dm_operand row_scale_inv,
                                   const float* expert_scale_inv, const int32_t* expert_offsets, int e_local,
                                   int64_t max_rows, int64_t N, int64_t Kd, int swiglu_interleaved, int clamped,
                                   float alpha, float limit, const int* cond, int num_sms, int* status, void* stream) {
  if (!a.base || !sfa.base || !w || !sfb || !expert_offsets || e_local <= 0 || max_rows < 0 || N <= 0 || Kd <= 0)
    return kRcBadArg;
  if (format != 0 && format != 1) return kRcBadArg;
  if (!swiglu_interleaved && !c.base && !scatter_ptrs) return kRcBadArg;
  if (swiglu_interleaved && (!h2.base || scatter_ptrs)) return kRcBadArg;
  if (e_local > kBsMaxGroups || max_rows > (1 << 30)) return kRcTooLarge;
  const int fp4 = format == 1;
  const int64_t row_bytes = fp4 ? Kd / 2 : Kd;
  if ((row_bytes % 128) != 0 || (N % 128) != 0 || (max_rows % 128) != 0) return kRcUnsupportedShape;
  if (max_rows == 0) return kRcOk;
  BsParams p{};
  int rc = encode_arena_u8(&p.tm_a, a, row_bytes, max_rows + 256, kBsBM);
  if (rc != kRcOk) return rc;
  rc = encode_2d_u8(&p.tm_b, w, static_cast<int64_t>(e_local) * N, row_bytes, kWdBN);
  if (rc != kRcOk) return rc;
  const int64_t scale_cols = Kd / (fp4 ? 16 : 32);
  p.a_col_atoms = static_cast<int>((scale_cols + 3) / 4);
  p.b_col_atoms = p.a_col_atoms;
  p.sfb_group_bytes = (N + 127) / 128 * 128 * static_cast<int64_t>(p.b_col_atoms) * 4;
  p.a_off = a.offset;
  p.sfa_off = sfa.offset;
  p.sfa_base = static_cast<const uint8_t*>(sfa.base);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.c_off = c.offset;
  p.h2_off = h2.offset;
  p.c_base = static_cast<uint8_t*>(c.base);
  p.h2_base = static_cast<uint8_t*>(h2.base);
  p.row_inv_base = static_cast<const uint8_t*>(row_scale_inv.base);
  p.row_inv_off = row_scale_inv.offset;
  p.expert_inv = expert_scale_inv;
  p.scatter_ptrs = scatter_ptrs;
  p.expert_offsets = expert_offsets;
  p.cond = cond;
  p.status = status;
  p.e_local = e_local;
  p.max_rows = static_cast<int>(max_rows);
  p.N = static_cast<int>(N);
  p.k_iters = static_cast<int>(row_bytes / 128);
  p.fp4 = fp4;
  p.swiglu = swiglu_interleaved ? 1 : 0;
  p.direct_store = (fp4 && swiglu_interleaved && !c.base) ? 1 : 0;
  p.act = ActParams{clamped, alpha, limit};
  return bs_launch(p, num_sms, static_cast<cudaStream_t>(stream));
}

// MXFP8 forward W13 GEMM whose SwiGLU epilogue writes h2 already row-quantised (the operand of the W2 GEMM).
extern "C" int dm_gemm_blockscaled_swiglu_mxfp8(dm_operand a, dm_operand sfa, const void* w, const void* sfb,
                                                dm_operand h2_q, dm_operand h2_sf, const int32_t* expert_offsets,
                                                int e_local, int64_t max_rows, int64_t N, int64_t Kd, int clamped,
                                                float alpha, float limit, const int* cond, int num_sms, int* status,
                                                void* stream) {
  if (!a.base || !sfa.base || !w || !sfb || !h2_q.base || !h2_sf.base || !expert_offsets || e_local <= 0 ||
      max_rows < 0 || N <= 0 || Kd <= 0)
    return kRcBadArg;
  if (e_local > kBsMaxGroups || max_rows > (1 << 30)) return kRcTooLarge;
  if ((Kd % 128) != 0 || (N % 128) != 0 || (max_rows % 128) != 0 || ((N / 2) % 32) != 0) return kRcUnsupportedShape;
  if (max_rows == 0) return kRcOk;
  BsParams p{};
  int rc = encode_arena_u8(&p.tm_a, a, Kd, max_rows + 256, kBsBM);
  if (rc != kRcOk) return rc;
  rc = encode_2d_u8(&p.tm_b, w, static_cast<int64_t>(e_local) * N, Kd, kWdBN);
  if (rc != kRcOk) return rc;
  p.a_col_atoms = static_cast<int>((Kd / 32 + 3) / 4);
  p.b_col_atoms = p.a_col_atoms;
  p.sfb_group_bytes = (N + 127) / 128 * 128 * static_cast<int64_t>(p.b_col_atoms) * 4;
  p.a_off = a.offset;
  p.sfa_off = sfa.offset;
  p.sfa_base = static_cast<const uint8_t*>(sfa.base);
  p.sfb = static_cast<const uint8_t*>(sfb);
  p.hq_base = static_cast<uint8_t*>(h2_q.base);
  p.hq_off = h2_q.offset;
  p.hsf_base = static_cast<uint8_t*>(h2_sf.base);
  p.hsf_off = h2_sf.offset;
  p.h_atoms = static_cast<int>((N / 2 / 32 + 3) / 4);
  p.h2_base = p.hq_base;  // the SwiGLU branch keys on a non-null h2
  p.expert_offsets = expert_offsets;
  p.cond = cond;
  p.status = status;
  p.e_local = e_local;
  p.max_rows = static_cast<int>(max_rows);
  p.N = static_cast<int>(N);
  p.k_iters = static_cast<int>(Kd / 128);
  p.swiglu = 1;
  p.act = ActParams{clamped, alpha, limit};
  return bs_launch(p, num_sms, static_cast<cudaStream_t>(stream));
}

// Input gradient: C[r, n] = sum_k dY[r, k] * W[e][k, n].  W is the same E4M3 qdata as in the forward
// ([E, Kd, N] bytes, 32x32-tile quantised) read N-major, with the scales of the transposed orientation
// ([N rows, Kd/32 columns] per expert, blocked).
extern "C" int dm_gemm_blockscaled_dgrad(dm_operand dy, dm_operand sf_dy, const void* w, const void* sfb_dgrad,
                                         dm_operand c, const int64_t* scatter_ptrs, const int32_t* expert_offsets,
                                         int e_local, int64_t max_rows, int64_t N, int64_t Kd, const int* cond,
                                         int num_sms, int* status, void* stream) {
  if (!dy.base || !sf_dy.base || !w || !sfb_dgrad || !expert_offsets || e_local <= 0 || max_rows < 0 || N <= 0 ||
      Kd <= 0)
    return kRcBadArg;
  if (!c.base && !scatter_ptrs) return kRcBadArg;
  if (e_local > kBsMaxGroups || max_rows > (1 << 30)) return kRcTooLarge;
  if ((Kd % 128) != 0 || (N % 128) != 0 || (max_rows % 128) != 0) return kRcUnsupportedShape;
  if (max_rows == 0) return kRcOk;
  BsParams p{};
  int rc = encode_arena_u8(&p.tm_a, dy, Kd, max_rows + 256, kBsBM);
  if (rc != kRcOk) return rc;
  rc = encode_2d_u8(&p.tm_b, w, static_cast<int64_t>(e_local) * Kd, N, kBsBN);
  if (rc != kRcOk) return rc;
  p.a_col_atoms = static_cast<int>((Kd / 32 + 3) / 4);
  p.b_col_atoms = p.a_col_atoms;
  p.sfb_group_bytes = (N + 127) / 128 * 128 * static_cast<int64_t>(p.b_col_atoms) * 4;
  p.a_off = dy.offset;
  p.sfa_off = sf_dy.offset;
  p.sfa_base = static_cast<const uint8_t*>(sf_dy.base);
  p.sfb = static_cast<const uint8_t*>(sfb_dgrad);
  p.c_off = c.offset;
  p.c_base = static_cast<uint8_t*>(c.base);
  p.scatter_ptrs = scatter_ptrs;
  p.expert_offsets = expert_offsets;
  p.cond = cond;
  p.status = status;
  p.e_local = e_local;
  p.max_rows = static_cast<int>(max_rows);
  p.N = static_cast<int>(N);
  p.Kw = static_cast<int>(Kd);
  p.k_iters = static_cast<int>(Kd / 128);
  p.mode = 1;
  p.act = ActParams{0, 1.0f, 0.0f};
  return bs_launch(p, num_sms, static_cast<cudaStream_t>(stream));
}

// Weight gradient: dW[e][m, n] (+)= sum_{r in expert e} dY[r, m] * X[r, n].  Both operands are quantised
// along the row dimension (32 rows share a scale, per column); their scales are blocked with the
// feature as the row index and the 32-row block as the column index.
static int blockscaled_wgrad(dm_operand dy_col, dm_operand sf_dy_col, dm_operand x_col, dm_operand sf_x_col, void* dw,
                             int dw_is_fp32, int accumulate, const int32_t* expert_offsets, int e_local,
                             int64_t max_rows, int64_t M, int64_t N, const int* cond, int num_sms, int* status,
                             void* stream, int compact_cols) {
  if (!dy_col.base || !sf_dy_col.base || !x_col.base || !sf_x_col.base || !dw || !expert_offsets || e_local <= 0 ||
      max_rows < 0 || M <= 0 || N <= 0)
    return kRcBadArg;
  if (e_local > kBsMaxGroups || max_rows > (1 << 30)) return kRcTooLarge;
  if ((M % 128) != 0 || (N % 128) != 0 || (max_rows % 128) != 0) return kRcUnsupportedShape;
  BsParams p{};
  int rc = kRcOk;
  // with no rows at all the kernel still runs so that a non-accumulating call zero-fills dW
  const int64_t rows_extent = max_rows > 0 ? max_rows : 128;
  rc = encode_arena_u8(&p.tm_a, dy_col, M, rows_extent, 128);
  if (rc != kRcOk) return rc;
  rc = encode_arena_u8(&p.tm_b, x_col, N, rows_extent, 128);
  if (rc != kRcOk) return rc;
  p.a_col_atoms = static_cast<int>(((max_rows + 31) / 32 + 3) / 4);
  p.b_col_atoms = p.a_col_atoms;
  p.a_off = dy_col.offset;
  p.b_off = x_col.offset;
  p.sfa_off = sf_dy_col.offset;
  p.sfb_off = sf_x_col.offset;
  p.sfa_base = static_cast<const uint8_t*>(sf_dy_col.base);
  p.sfb = static_cast<const uint8_t*>(sf_x_col.base);
  p.c_base = static_cast<uint8_t*>(dw);
  rc = encode_out_3d(&p.tm_c, dw, e_local, M, N, dw_is_fp32 != 0);
  if (rc != kRcOk) return rc;
  p.expert_offsets = expert_offsets;
  p.cond = cond;
  p.status = status;
  p.e_local = e_local;
  p.max_rows = static_cast<int>(max_rows);
  p.N = static_cast<int>(M);
  p.Kw = static_cast<int>(N);
  p.mode = 2;
  p.compact_cols = compact_cols;
  p.out_fp32 = dw_is_fp32 ? 1 : 0;
  p.accumulate = accumulate ? 1 : 0;
  p.act = ActParams{0, 1.0f, 0.0f};
  return bs_launch(p, num_sms, static_cast<cudaStream_t>(stream));
}

extern "C" int dm_gemm_blockscaled_wgrad(dm_operand dy_col, dm_operand sf_dy_col, dm_operand x_col, dm_operand sf_x_col,
                                         void* dw, int dw_is_fp32, int accumulate, const int32_t* expert_offsets,
                                         int e_local, int64_t max_rows, int64_t M, int64_t N, const int* cond,
                                         int num_sms, int* status, void* stream) {
  return blockscaled_wgrad(dy_col, sf_dy_col, x_col, sf_x_col, dw, dw_is_fp32, accumulate, expert_offsets, e_local,
                           max_rows, M, N, cond, num_sms, status, stream, 0);
}

// The same product for column bundles whose scale layout was sized by the device row count
// (expert_offsets[e_local] rows, as the *_at quantisers write them) instead of by max_rows.
extern "C" int dm_gemm_blockscaled_wgrad_compact(dm_operand dy_col, dm_operand sf_dy_col, dm_operand x_col,
                                                 dm_operand sf_x_col, void* dw, int dw_is_fp32, int accumulate,
                                                 const int32_t* expert_offsets, int e_local, int64_t max_rows,
                                                 int64_t M, int64_t N, const int* cond, int num_sms, int* status,
                                                 void* stream) {
  return blockscaled_wgrad(dy_col, sf_dy_col, x_col, sf_x_col, dw, dw_is_fp32, accumulate, expert_offsets, e_local,
                           max_rows, M, N, cond, num_sms, status, stream, 1);
}
