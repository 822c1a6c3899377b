// Grouped BF16 forward / input-gradient GEMMs on CTA pairs (tcgen05.mma.cta_group::2), operands swapped.
//
// The expert weights are the M side of the MMA and the routed rows the N side:
//
//   fprop  Ct[n, r] = sum_k W[e][n][k]  X[r, k]        A = W rows (K-major),    B = routed rows (K-major)
//   dgrad  Ct[n, r] = sum_k W[e][k][n] dY[r, k]        A = W columns (M-major), B = routed rows (K-major)
//
// Why swapped: M is fixed by the hardware (128 accumulator lanes per CTA) while N may be any multiple of
// 16 up to 256.  With the rows of an expert on the N side a ragged expert costs at most 31 padding rows per
// chunk instead of up to 127 per tile, and the weight side (always a multiple of 64 features) fills M.
//
// Why pairs: one MMA covers 256 features x n rows; each CTA stages its own 128 features of A and HALF of the
// routed rows of B, so a stage moves (16 KiB + n/2 x 128 B) per CTA for 128 x n x 64 MACs - about two thirds
// of the shared-memory traffic per FLOP of a single-CTA 128 x 256 tile.
//
// Per CTA (480 threads): warps 0 and 14 TMA producers (weights / routed rows), warp 1 owns TMEM (the even
// CTA's lane 0 issues every MMA of the pair), warps 2-9 epilogue, warps 10-13 gather (fused dispatch).  Pipeline: loads of both CTAs signal
// the even CTA's "full" barrier; MMA completion is committed to the "empty" barrier of both CTAs; the
// accumulator-ready barrier likewise; epilogue warps of both CTAs release an accumulator on the even CTA's
// barrier.  Every wait is bounded; a timeout sets a status word and the kernel drains.
//
// Accumulator layout: TMEM lane = feature (128 per CTA), column = routed row of the chunk.  The epilogue
// transposes 32 x 32 blocks through shared memory and stores 64-byte row segments (plain rows, per-row
// scatter pointers, or fused SwiGLU where a CTA holds 64 gate features in lanes 0-63 and the matching 64 up
// features in lanes 64-127).
#include "gemm_common.cuh"

namespace dm {

constexpr int kPStages = 3;   // stages of K = 128 (two 64-element slabs per operand)
constexpr int kPThreads = 480;
constexpr int kPGatherWarps = 4;
constexpr int kPMaxGroups = 256;
constexpr uint32_t kPABytes = 128 * 128;  // 128 features x 64 bf16
constexpr uint32_t kPBBytes = 128 * 128;  // up to 128 routed rows x 64 bf16 per CTA
constexpr uint32_t kPSlabBytes = kPABytes + kPBBytes;   // one K = 64 slab: A tile then B tile
constexpr uint32_t kPStageBytes = 2 * kPSlabBytes;
constexpr uint32_t kPStagingBytes = 32 * 64;
constexpr uint32_t kPTmemCols = 512;
constexpr size_t kPSmemBytes = kPStages * kPStageBytes + 8 * kPStagingBytes + 1024;

struct PairParams {
  CUtensorMap tm_a;     // weights, 64 x 64 boxes
  CUtensorMap tm_a128;  // weights, 128 rows x 64 (forward without SwiGLU pairing)
  CUtensorMap tm_b128;  // routed rows, 128 / 64 / 32 / 16-row boxes
  CUtensorMap tm_b64;
  CUtensorMap tm_b32;
  CUtensorMap tm_b16;
  const int64_t* b_off;
  const int64_t* c_off;
  const int64_t* h2_off;
  uint8_t* c_base;
  uint8_t* h2_base;
  const int64_t* scatter_ptrs;
  const int64_t* gather_ptrs;
  int* gather_flags;
  uint8_t* b_base;
  const int32_t* expert_offsets;
  const int* cond;
  int* status;
  int e_local;
  int max_rows;
  int N;      // output features
  int Kd;     // contraction
  int fused;  // fprop only: N = 2F, gate/up pairing + SwiGLU
  int dgrad;
  ActParams act;
};

struct Unit {
  int e, fb, tok0, valid, n_mma;
};

// Loads / MMAs taking precomputed shared-memory addresses and descriptor words.
__device__ __forceinline__ void tma_load_2d_pair_a(uint32_t smem_dst, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_dst), "l"(tmap), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair_a(uint32_t smem_dst, const void* tmap, int x, int y, int z,
                                                   uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_dst), "l"(tmap), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
__device__ __forceinline__ void umma_bf16_pair_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                                  uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Bounded spin on a shared-memory sequence flag written by another warp of the CTA.
__device__ __forceinline__ bool flag_wait(const volatile int* flag, int want, volatile int* abort_flag) {
  if (*flag >= want) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (*flag < want) {
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > 2000000000ull) {
        *abort_flag = 1;
        return false;
      }
    }
  }
  return true;
}

__device__ __forceinline__ Unit decode_unit(int unit, int& e, const int* unit_start, const int* off, const int* nt,
                                            int fbs) {
  while (unit >= unit_start[e + 1]) ++e;
  const int local = unit - unit_start[e];
  Unit u;
  u.e = e;
  u.fb = local % fbs;
  const int tc = local / fbs;
  const int rows = off[e + 1] - off[e];
  u.tok0 = off[e] + tc * nt[e];
  const int left = rows - tc * nt[e];
  u.valid = left < nt[e] ? left : nt[e];
  u.n_mma = (u.valid + 31) & ~31;
  return u;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPThreads, 1)
    paired_gemm_kernel(const __grid_constant__ PairParams p) {
  if (p.cond != nullptr && *p.cond == 0) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  __shared__ uint64_t full_bar[kPStages];
  __shared__ uint64_t empty_bar[kPStages];
  __shared__ uint64_t tmem_full_bar[2];
  __shared__ uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int s_off[kPMaxGroups + 1];
  __shared__ int s_unit_start[kPMaxGroups + 1];
  __shared__ int s_nt[kPMaxGroups];
  __shared__ volatile int s_ready[8];  // fused epilogue: block sequence number whose staging tile is written
  __shared__ volatile int s_done[8];   //                 block sequence number the warp has finished reading

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  // feature blocks of one expert: 256 features per pair, or (fused) 128 gate + the matching 128 up features
  const int fbs = p.fused ? (p.N / 2) / 128 : (p.N + 255) / 256;

  for (int i = threadIdx.x; i <= p.e_local; i += blockDim.x) {
    const int v = p.expert_offsets[i];
    s_off[i] = v < p.max_rows ? v : p.max_rows;
  }
  if (threadIdx.x < 8) {
    s_ready[threadIdx.x] = 0;
    s_done[threadIdx.x] = 0;
  }
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kPStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], 16);  // eight epilogue warps of each CTA
    }
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < p.e_local; ++e) {
      s_unit_start[e] = acc;
      const int rows = s_off[e + 1] - s_off[e];
      const int chunks = (rows + 255) / 256;
      s_nt[e] = chunks > 0 ? (((rows + chunks - 1) / chunks + 31) & ~31) : 0;
      acc += chunks * fbs;
    }
    s_unit_start[p.e_local] = acc;
  }
  // the peer CTA must be resident before TMEM of the pair is allocated and before remote barriers are used
  cluster_sync_all();
  if (warp == 1) {
    tmem_alloc_pair(&tmem_base_slot, kPTmemCols);
    tmem_relinquish_pair();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&p.tm_a);
    tma_prefetch_desc(&p.tm_a128);
    tma_prefetch_desc(&p.tm_b128);
    tma_prefetch_desc(&p.tm_b64);
    tma_prefetch_desc(&p.tm_b32);
    tma_prefetch_desc(&p.tm_b16);
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_base_slot;
  const int total_units = s_unit_start[p.e_local];
  const int k_iters = p.Kd / 128;
  const int64_t b_off = p.b_off ? *p.b_off : 0;

  if (warp == 0 || warp == 14) {
    // ======================= TMA producers (both CTAs) =======================
    // Two single-thread producers share the ring: warp 0 loads the weight tile (and, in the even CTA, arms
    // the stage's barrier with the byte count of the whole pair), warp 14 loads the routed rows.  The
    // loops are kept to a few dozen instructions per stage: a single thread issues them one after another.
    if (lane == 0) {
      const bool is_a = warp == 0;
      int stage = 0;
      uint32_t phase = 0;
      int e = 0;
      const int b_line0 = static_cast<int>(b_off >> 7);
      bool ok = true;
      const int total_rows = s_off[p.e_local];
      const int nblocks = (total_rows + 127) >> 7;
      const uint32_t smem_base = smem_u32(smem);
      const uint32_t full0 = mapa_shared(smem_u32(&full_bar[0]), 0);  // the even CTA's barriers
      const uint32_t empty0 = smem_u32(&empty_bar[0]);
      for (int unit = pair; unit < total_units && ok; unit += num_pairs) {
        const Unit u = decode_unit(unit, e, s_unit_start, s_off, s_nt, fbs);
        const int h = u.n_mma >> 1;  // routed rows staged by this CTA
        const int my_row0 = u.tok0 + static_cast<int>(rank) * h;
        if (!is_a && p.gather_flags != nullptr) {
          // rows are pulled by gather warps of some CTA: wait (bounded) for the 128-row blocks this CTA loads
          int first = my_row0 >> 7, last = (my_row0 + h - 1) >> 7;
          if (last > nblocks - 1) last = nblocks - 1;
          const uint64_t t0 = globaltimer_ns();
          for (int b = first; b <= last && ok; ++b) {
            uint32_t spins = 0;
            while (ld_acquire_gpu(p.gather_flags + b) < kPGatherWarps) {
              if ((++spins & 0xff) == 0 && (abort_flag || globaltimer_ns() - t0 > 2000000000ull)) {
                abort_flag = 1;
                ok = false;
                break;
              }
            }
          }
          fence_proxy_async_all();
          if (!ok) break;
        }
        if (is_a) {
          int a_r0, a_r1;  // fprop: first row of the 64-row boxes; dgrad: first column of the 64-column boxes
          if (p.dgrad) {
            a_r0 = u.fb * 256 + static_cast<int>(rank) * 128;
            a_r1 = a_r0 + 64;
          } else if (p.fused) {
            a_r0 = u.e * p.N + u.fb * 128 + static_cast<int>(rank) * 64;
            a_r1 = a_r0 + p.N / 2;
          } else {
            a_r0 = u.e * p.N + u.fb * 256 + static_cast<int>(rank) * 128;
            a_r1 = a_r0 + 64;
          }
          const uint32_t tx = 2 * (2 * kPABytes + static_cast<uint32_t>(u.n_mma) * 128);
          const int k_row0 = u.e * p.Kd;
          const int mode = p.dgrad ? 2 : (p.fused ? 1 : 0);
          for (int kb = 0; kb < k_iters; ++kb) {
            ok = mbar_wait_lean(empty0 + stage * 8, &empty_bar[stage], phase ^ 1u, &abort_flag);
            if (!ok) break;
            const uint32_t sa = smem_base + stage * kPStageBytes;
            const uint32_t bar = full0 + stage * 8;
            if (rank == 0) mbar_arrive_expect_tx(&full_bar[stage], tx);
#pragma unroll
            for (int sl = 0; sl < 2; ++sl) {
              const int k0 = kb * 128 + sl * 64;
              const uint32_t dst = sa + sl * kPSlabBytes;
              if (mode == 0) {
                tma_load_2d_pair_a(dst, &p.tm_a128, k0, a_r0, bar);
              } else if (mode == 1) {
                tma_load_2d_pair_a(dst, &p.tm_a, k0, a_r0, bar);
                tma_load_2d_pair_a(dst + 8192, &p.tm_a, k0, a_r1, bar);
              } else {
                tma_load_2d_pair_a(dst, &p.tm_a, a_r0, k_row0 + k0, bar);
                tma_load_2d_pair_a(dst + 8192, &p.tm_a, a_r1, k_row0 + k0, bar);
              }
            }
            if (++stage == kPStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        } else {
          for (int kb = 0; kb < k_iters; ++kb) {
            ok = mbar_wait_lean(empty0 + stage * 8, &empty_bar[stage], phase ^ 1u, &abort_flag);
            if (!ok) break;
            const uint32_t bar = full0 + stage * 8;
#pragma unroll
            for (int sl = 0; sl < 2; ++sl) {
              const uint32_t sb = smem_base + stage * kPStageBytes + sl * kPSlabBytes + kPABytes;
              const int line = b_line0 + kb * 2 + sl;
              // h is a multiple of 16: at most one box of each size
              int r = 0;
              if (h & 128) {
                tma_load_3d_pair_a(sb, &p.tm_b128, 0, line, my_row0, bar);
                r = 128;
              }
              if (h & 64) {
                tma_load_3d_pair_a(sb + r * 128, &p.tm_b64, 0, line, my_row0 + r, bar);
                r += 64;
              }
              if (h & 32) {
                tma_load_3d_pair_a(sb + r * 128, &p.tm_b32, 0, line, my_row0 + r, bar);
                r += 32;
              }
              if (h & 16) tma_load_3d_pair_a(sb + r * 128, &p.tm_b16, 0, line, my_row0 + r, bar);
            }
            if (++stage == kPStages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ======================= MMA issuer (one thread of the even CTA) =======================
    if (rank == 0 && lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int e = 0, it = 0;
      bool ok = true;
      // Shared-memory descriptors: the upper word is constant, the lower word is (address >> 4) | (LBO >> 4) << 16.
      constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version 1, 128-byte swizzle
      const uint32_t a_lbo = p.dgrad ? (8192u >> 4) << 16 : (16u >> 4) << 16;
      const uint32_t a_step = p.dgrad ? (2048u >> 4) : (32u >> 4);  // per K = 16 step
      const uint32_t a_lo0 = ((smem_u32(smem) & 0x3ffffu) >> 4) | a_lbo;
      const uint32_t b_lo0 = (((smem_u32(smem) + kPABytes) & 0x3ffffu) >> 4) | ((16u >> 4) << 16);
      const uint32_t full0 = smem_u32(&full_bar[0]);
      const uint32_t tempty0 = smem_u32(&tmem_empty_bar[0]);
      const uint32_t idesc_base = umma_idesc_bf16(256, 0, p.dgrad ? 1 : 0, 0);
      for (int unit = pair; unit < total_units && ok; unit += num_pairs, ++it) {
        const Unit u = decode_unit(unit, e, s_unit_start, s_off, s_nt, fbs);
        const int buf = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        ok = mbar_wait_lean(tempty0 + buf * 8, &tmem_empty_bar[buf], acc_phase ^ 1u, &abort_flag);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + buf * 256;
        const uint32_t idesc = idesc_base | (static_cast<uint32_t>(u.n_mma >> 3) << 17);
        uint32_t acc = 0;
        for (int kb = 0; kb < k_iters; ++kb) {
          ok = mbar_wait_lean(full0 + stage * 8, &full_bar[stage], phase, &abort_flag);
          if (!ok) break;
          const uint32_t a_lo = a_lo0 + stage * (kPStageBytes >> 4);
          const uint32_t b_lo = b_lo0 + stage * (kPStageBytes >> 4);
          umma_bf16_pair_lo(d_tmem, a_lo, b_lo, kDescHi, idesc, acc);
          umma_bf16_pair_lo(d_tmem, a_lo + a_step, b_lo + 2, kDescHi, idesc, 1u);
          umma_bf16_pair_lo(d_tmem, a_lo + 2 * a_step, b_lo + 4, kDescHi, idesc, 1u);
          umma_bf16_pair_lo(d_tmem, a_lo + 3 * a_step, b_lo + 6, kDescHi, idesc, 1u);
          constexpr uint32_t kSlab = kPSlabBytes >> 4;
          umma_bf16_pair_lo(d_tmem, a_lo + kSlab, b_lo + kSlab, kDescHi, idesc, 1u);
          umma_bf16_pair_lo(d_tmem, a_lo + kSlab + a_step, b_lo + kSlab + 2, kDescHi, idesc, 1u);
          umma_bf16_pair_lo(d_tmem, a_lo + kSlab + 2 * a_step, b_lo + kSlab + 4, kDescHi, idesc, 1u);
          umma_bf16_pair_lo(d_tmem, a_lo + kSlab + 3 * a_step, b_lo + kSlab + 6, kDescHi, idesc, 1u);
          acc = 1u;
          tcgen05_commit_pair(&empty_bar[stage]);  // releases the stage in both CTAs
          if (++stage == kPStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        tcgen05_commit_pair(&tmem_full_bar[buf]);
      }
    }
    __syncwarp();
  } else if (warp >= 10 && warp < 14) {
    // ======================= gather (fused dispatch) =======================
    if (p.gather_flags != nullptr) {
      const int gw = warp - 10;
      const int total_rows = s_off[p.e_local];
      const int nblocks = (total_rows + 127) >> 7;
      const int vec_per_row = p.Kd / 8;
      uint4* dst_base = reinterpret_cast<uint4*>(p.b_base + b_off);
      for (int u = gw * gridDim.x + blockIdx.x; u < nblocks * 4; u += kPGatherWarps * gridDim.x) {
        const int blk = u >> 2;
        const int r_begin = blk * 128 + (u & 3) * 32;
        for (int rr = 0; rr < 32; rr += 2) {
          const int r0 = r_begin + rr, r1 = r0 + 1;
          if (r0 >= total_rows) break;
          const uint4* src0 = reinterpret_cast<const uint4*>(p.gather_ptrs[r0]);
          const uint4* src1 = r1 < total_rows ? reinterpret_cast<const uint4*>(p.gather_ptrs[r1]) : nullptr;
          uint4* dst0 = dst_base + static_cast<int64_t>(r0) * vec_per_row;
          uint4* dst1 = dst_base + static_cast<int64_t>(r1) * vec_per_row;
          for (int v0 = 0; v0 < vec_per_row; v0 += 256) {
            uint4 b0[8], b1[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int v = v0 + j * 32 + lane;
              b0[j] = (src0 != nullptr && v < vec_per_row) ? __ldcg(src0 + v) : make_uint4(0, 0, 0, 0);
              b1[j] = (src1 != nullptr && v < vec_per_row) ? __ldcg(src1 + v) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const int v = v0 + j * 32 + lane;
              if (v < vec_per_row) {
                dst0[v] = b0[j];
                if (r1 < total_rows) dst1[v] = b1[j];
              }
            }
          }
        }
        __threadfence();
        __syncwarp();
        if (lane == 0) red_release_gpu_add(p.gather_flags + blk, 1);
      }
    }
  } else {
    // ======================= epilogue (both CTAs) =======================
    const int ew = warp - 2;    // 0..7
    const int quad = warp & 3;  // TMEM lanes [32*quad, 32*quad + 32)
    const int half = ew >> 2;   // which 32-column blocks of the chunk: even or odd
    uint8_t* stg = smem + kPStages * kPStageBytes + ew * kPStagingBytes;
    uint8_t* stg_peer = smem + kPStages * kPStageBytes + (ew ^ 2) * kPStagingBytes;  // fused: warp holding the other of gate / up
    const uint32_t empty_remote0 = mapa_shared(smem_u32(&tmem_empty_bar[0]), 0);
    const uint32_t empty_remote1 = mapa_shared(smem_u32(&tmem_empty_bar[1]), 0);
    int e = 0, it = 0, seq = 0;
    bool ok = true;
    const int64_t c_off = p.c_off ? *p.c_off : 0;
    const int64_t h2_off = p.h2_off ? *p.h2_off : 0;
    const int F = p.N / 2;
    for (int unit = pair; unit < total_units && ok; unit += num_pairs, ++it) {
      const Unit u = decode_unit(unit, e, s_unit_start, s_off, s_nt, fbs);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      if (lane == 0) ok = mbar_wait(&tmem_full_bar[buf], acc_phase, &abort_flag);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * 256;
      const int row_end = u.tok0 + u.valid;
      const int blocks = u.n_mma >> 5;
      if (p.fused) {
        // lanes 0-63: gate features f0 + lane; lanes 64-127: the matching up features
        const int f0 = u.fb * 128 + static_cast<int>(rank) * 64 + (quad & 1) * 32;
        const bool is_gate = quad < 2;
        const int peer = ew ^ 2;
        for (int cb = half; cb < blocks && ok; cb += 2) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + cb * 32, r);
          tmem_ld_wait();
          ++seq;
          // the partner must have finished reading this warp's previous staging tile
          if (lane == 0) ok = flag_wait(&s_done[peer], seq - 1, &abort_flag);
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
#pragma unroll
          for (int j = 0; j < 32; ++j)
            reinterpret_cast<__nv_bfloat16*>(stg + j * 64)[lane] = __float2bfloat16_rn(__uint_as_float(r[j]));
          __syncwarp();
          if (lane == 0) {
            __threadfence_block();
            s_ready[ew] = seq;
            ok = flag_wait(&s_ready[peer], seq, &abort_flag);
            __threadfence_block();
          }
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
          const uint8_t* sg = is_gate ? stg : stg_peer;
          const uint8_t* su = is_gate ? stg_peer : stg;
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int jj = (is_gate ? 0 : 16) + i * 8 + (lane >> 2), ch = lane & 3;
            const int row = u.tok0 + cb * 32 + jj;
            const uint4 g = *reinterpret_cast<const uint4*>(sg + jj * 64 + ch * 16);
            const uint4 v = *reinterpret_cast<const uint4*>(su + jj * 64 + ch * 16);
            if (row < row_end) {
              const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, uw[4] = {v.x, v.y, v.z, v.w};
              uint32_t zw[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const float z0 = swiglu_f32(__uint_as_float(gw[q] << 16), __uint_as_float(uw[q] << 16), p.act);
                const float z1 =
                    swiglu_f32(__uint_as_float(gw[q] & 0xffff0000u), __uint_as_float(uw[q] & 0xffff0000u), p.act);
                zw[q] = pack_bf16x2(z0, z1);
              }
              const int col = f0 + ch * 8;
              uint8_t* h1 = p.c_base + c_off + static_cast<int64_t>(row) * p.N * 2;
              *reinterpret_cast<uint4*>(h1 + static_cast<int64_t>(col) * 2) = g;
              *reinterpret_cast<uint4*>(h1 + static_cast<int64_t>(F + col) * 2) = v;
              *reinterpret_cast<uint4*>(p.h2_base + h2_off + (static_cast<int64_t>(row) * F + col) * 2) =
                  make_uint4(zw[0], zw[1], zw[2], zw[3]);
            }
          }
          __syncwarp();
          if (lane == 0) {
            __threadfence_block();
            s_done[ew] = seq;
          }
        }
        if (!ok) break;
      } else {
        const int feat0 = u.fb * 256 + static_cast<int>(rank) * 128 + quad * 32;
        for (int cb = half; cb < blocks; cb += 2) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + cb * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            reinterpret_cast<__nv_bfloat16*>(stg + j * 64)[lane] = __float2bfloat16_rn(__uint_as_float(r[j]));
          __syncwarp();
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int jj = i * 8 + (lane >> 2), ch = lane & 3;
            const int row = u.tok0 + cb * 32 + jj;
            const uint4 v = *reinterpret_cast<const uint4*>(stg + jj * 64 + ch * 16);
            const int col = feat0 + ch * 8;
            if (row < row_end && col + 8 <= p.N) {
              uint64_t dst;
              if (p.scatter_ptrs != nullptr)
                dst = static_cast<uint64_t>(p.scatter_ptrs[row]);
              else
                dst = reinterpret_cast<uint64_t>(p.c_base) + c_off + static_cast<uint64_t>(row) * p.N * 2;
              if (dst != 0) *reinterpret_cast<uint4*>(dst + static_cast<uint64_t>(col) * 2) = v;
            }
          }
          __syncwarp();
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(buf ? empty_remote1 : empty_remote0);
    }
  }

  // ---- teardown: neither CTA may leave while the peer can still touch its barriers or TMEM ----
  tcgen05_fence_before();
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) set_status(p.status, kPipelineTimeout, 4 + p.dgrad, blockIdx.x);
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, kPTmemCols);
  }
}

}  // namespace dm

using namespace dm;

// Shapes the paired kernel takes; everything else stays on the single-CTA kernel.
bool dm::dm_pair_supported(int64_t N, int64_t Kd, int fused, int dgrad) {
  if ((Kd % 128) != 0 || Kd < 128) return false;
  if (fused) return !dgrad && ((N / 2) % 128) == 0;
  return (N % 64) == 0;
}

int dm::dm_pair_launch(const dm_operand& b, const void* w, dm_operand c, dm_operand h2, const int64_t* scatter_ptrs,
                   const int64_t* gather_ptrs, int32_t* gather_flags, const int32_t* expert_offsets, int e_local,
                   int64_t max_rows, int64_t N, int64_t Kd, int fused, int dgrad, int clamped, float alpha, float limit,
                   const int* cond, int num_sms, int* status, cudaStream_t st) {
  static PerDeviceOnce attr_set;
  const int rc_attr = once_per_device(attr_set, [] {
    return static_cast<int>(cudaFuncSetAttribute(paired_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(kPSmemBytes)));
  });
  if (rc_attr != 0) return rc_attr;
  PairParams p{};
  int rc;
  if (dgrad)
    rc = encode_2d(&p.tm_a, w, static_cast<int64_t>(e_local) * Kd, N, 64);  // W = [e_local * Kd][N], box 64 k-rows x 64 features
  else
    rc = encode_2d(&p.tm_a, w, static_cast<int64_t>(e_local) * N, Kd, 64);  // W = [e_local * N][Kd], box 64 features x 64 k
  if (rc != kRcOk) return rc;
  if (!dgrad) {
    rc = encode_2d(&p.tm_a128, w, static_cast<int64_t>(e_local) * N, Kd, 128);
    if (rc != kRcOk) return rc;
  } else {
    p.tm_a128 = p.tm_a;
  }
  const int box_rows[4] = {128, 64, 32, 16};
  CUtensorMap* maps[4] = {&p.tm_b128, &p.tm_b64, &p.tm_b32, &p.tm_b16};
  for (int i = 0; i < 4; ++i) {
    rc = encode_arena(maps[i], b, Kd * 2, max_rows + 256, box_rows[i]);
    if (rc != kRcOk) return rc;
  }
  p.b_off = b.offset;
  p.c_off = c.offset;
  p.h2_off = h2.offset;
  p.c_base = static_cast<uint8_t*>(c.base);
  p.h2_base = static_cast<uint8_t*>(h2.base);
  p.scatter_ptrs = scatter_ptrs;
  p.expert_offsets = expert_offsets;
  p.cond = cond;
  p.status = status;
  p.e_local = e_local;
  p.max_rows = static_cast<int>(max_rows);
  p.N = static_cast<int>(N);
  p.Kd = static_cast<int>(Kd);
  p.fused = fused ? 1 : 0;
  p.dgrad = dgrad ? 1 : 0;
  p.act = ActParams{clamped, alpha, limit};
  if (gather_ptrs != nullptr) {
    p.gather_ptrs = gather_ptrs;
    p.gather_flags = gather_flags;
    p.b_base = static_cast<uint8_t*>(b.base);
    const cudaError_t e = cudaMemsetAsync(gather_flags, 0, sizeof(int32_t) * static_cast<size_t>((max_rows + 127) / 128 + 1), st);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  int grid = persistent_grid(num_sms);
  grid &= ~1;
  if (grid < 2) return kRcBadArg;
  paired_gemm_kernel<<<grid, kPThreads, kPSmemBytes, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}
