// Persistent grouped BF16 GEMMs on tcgen05 tensor cores (sm_100a).
//
// One CTA per SM, 320 threads, warp-specialised:
//   warp 0      TMA producer: fills a 4-stage shared-memory ring (A 128x64, B 256x64 bf16,
//               128-byte swizzle) with cp.async.bulk.tensor loads, no multicast.
//   warp 1      MMA issuer: owns the TMEM allocation (512 columns = two 128x256 fp32
//               accumulators), issues tcgen05.mma (M128 N256 K16) from one lane and
//               releases stages / publishes accumulators with tcgen05.commit.
//   warps 2..9  epilogue (two per TMEM lane quadrant): tcgen05.ld their 32 TMEM lanes, convert and store (plain rows,
//               fused SwiGLU, per-row scatter to peer memory, or weight-gradient
//               read-modify-write) while the next tile's main loop already runs.
//
// Groups are the local experts; their row ranges come from device memory
// (expert_offsets), so the tile list is built by every CTA at kernel start and no
// host read is needed.  Activation operands are addressed as (arena base, device
// byte offset): the tensor map views the whole arena as [row][128-byte line][64 bf16]
// with overlapping strides, so a planner-chosen offset only changes a coordinate.
//
// Three operand arrangements share the kernel:
//   fprop  C[r,n]  = sum_k A[r,k] W[e][n][k]     A, W K-major
//   dgrad  C[r,n]  = sum_k A[r,k] W[e][k][n]     A K-major, W N-major
//   wgrad  dW[e][n][k] (+)= sum_r dY[r,n] X[r,k] both operands MN-major; the ragged last
//          64-row chunk of an expert is zeroed in shared memory before the MMA reads it.
#include "gemm_common.cuh"

namespace dm {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBK = 64;
constexpr int kStages = 4;
constexpr int kGemmThreads = 480;  // TMA warp, MMA warp, eight epilogue warps, four gather warps, one accumulator watcher
constexpr int kGatherWarps = 4;
constexpr int kGatherUnitRows = 8;                      // rows one gather warp pulls before it reports
constexpr int kGatherUnitsPerBlock = 128 / kGatherUnitRows;  // reports that make a 128-row block ready
constexpr int kMaxGroups = 256;
constexpr uint32_t kABytes = kBM * kBK * 2;  // 16 KiB
constexpr uint32_t kBBytes = kBN * kBK * 2;  // 32 KiB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kTmemCols = 512;
constexpr size_t kGemmSmemBytes = kStages * kStageBytes + 8 * kStaging64Bytes + 1024;  // + slack for 1024-byte alignment

enum GemmMode : int { kFprop = 0, kDgrad = 1, kWgrad = 2 };

struct GemmParams {
  CUtensorMap tm_a;
  CUtensorMap tm_b;
  CUtensorMap tm_b256;  // forward without SwiGLU pairing: one 256-row box per stage
  CUtensorMap tm_c;     // wgrad: dW as [e_local][N][Kd], boxes of 16 rows x 128 bytes
  const int64_t* a_off;  // device byte offsets (may be null = 0)
  const int64_t* b_off;
  const int64_t* c_off;
  const int64_t* h2_off;
  uint8_t* c_base;
  uint8_t* h2_base;
  const int64_t* scatter_ptrs;
  const int64_t* gather_ptrs;  // fused dispatch: row r of A is pulled from gather_ptrs[r] (may be peer memory)
  int* gather_flags;           // one counter per 128-row block of A, zero before the launch
  uint8_t* a_base;             // where the pulled rows land (the A operand itself)
  const int32_t* expert_offsets;
  const int* cond;
  int* status;
  int e_local;
  int max_rows;
  int N;        // output columns (fprop/dgrad), dW rows (wgrad)
  int Kd;       // contraction (fprop/dgrad), dW columns (wgrad)
  int fused;    // fprop: W13 gate/up pairing + SwiGLU epilogue (N = 2F)
  int out_fp32; // wgrad
  int accumulate;
  ActParams act;
};

struct Tile {
  int e, m_blk, n_blk, row0, row_end, k_iters;
};

template <int kMode>
__device__ __forceinline__ Tile decode_tile(int tile, int& e, const int* tile_start, const int* off, int n_tiles,
                                            int Kd) {
  while (tile >= tile_start[e + 1]) ++e;
  const int local = tile - tile_start[e];
  Tile t;
  t.e = e;
  const int rows = off[e + 1] - off[e];
  if (kMode == kWgrad) {
    t.n_blk = local % n_tiles;
    t.m_blk = local / n_tiles;
    t.row0 = off[e];
    t.row_end = off[e + 1];
    t.k_iters = (rows + kBK - 1) / kBK;
  } else {
    const int m_tiles = (rows + kBM - 1) / kBM;
    t.m_blk = local % m_tiles;
    t.n_blk = local / m_tiles;
    t.row0 = off[e] + t.m_blk * kBM;
    t.row_end = off[e + 1];
    t.k_iters = (Kd + kBK - 1) / kBK;
  }
  return t;
}

template <int kMode>
__global__ void __launch_bounds__(kGemmThreads, 1) grouped_gemm_kernel(const __grid_constant__ GemmParams p) {
  if (p.cond != nullptr && *p.cond == 0) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));

  __shared__ uint64_t full_bar[kStages];
  __shared__ uint64_t empty_bar[kStages];
  __shared__ uint64_t tmem_full_bar[2];
  __shared__ uint64_t tmem_empty_bar[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;
  __shared__ int s_off[kMaxGroups + 1];
  __shared__ int s_tile_start[kMaxGroups + 1];

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- tile table -----------------------------------------------------------
  const int n_tiles = (kMode == kWgrad) ? (p.Kd + kBN - 1) / kBN
                                        : (p.fused ? (p.N / 2) / (kBN / 2) : (p.N + kBN - 1) / kBN);
  const int wgrad_m_tiles = (p.N + kBM - 1) / kBM;
  for (int i = threadIdx.x; i <= p.e_local; i += blockDim.x) {
    int v = p.expert_offsets[i];
    s_off[i] = v < p.max_rows ? v : p.max_rows;
  }
  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full_bar[b], 1);
      mbar_init(&tmem_empty_bar[b], 8);
    }
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < p.e_local; ++e) {
      s_tile_start[e] = acc;
      const int rows = s_off[e + 1] - s_off[e];
      acc += (kMode == kWgrad) ? wgrad_m_tiles * n_tiles : ((rows + kBM - 1) / kBM) * n_tiles;
    }
    s_tile_start[p.e_local] = acc;
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, kTmemCols);
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

  const int64_t a_off = p.a_off ? *p.a_off : 0;
  const int64_t b_off = p.b_off ? *p.b_off : 0;

  // Weight gradient: a stage is six 64 x 64 boxes, and one thread cannot issue six TMA loads in the time the
  // tensor cores need for the stage, so the (otherwise idle) warps 10 and 11 issue the boxes of the second
  // operand; warp 0 arms the stage's barrier and loads the first operand.
  const int wgrad_part = (kMode == kWgrad) ? (warp == 0 ? 0 : (warp == 10 ? 1 : (warp == 11 ? 2 : -1))) : -1;
  if (warp == 0 || wgrad_part > 0) {
    // ======================= TMA producer =======================
    int stage = 0;
    uint32_t phase = 0;
    int e = 0;
    const int a_line0 = static_cast<int>(a_off >> 7);
    const int b_line0 = static_cast<int>(b_off >> 7);
    bool ok = true;
    int ready_blocks = 0;  // row blocks [0, ready_blocks) are known to have landed
    const int total_rows = s_off[p.e_local];
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
      const Tile t = decode_tile<kMode>(tile, e, s_tile_start, s_off, n_tiles, p.Kd);
      if (kMode != kWgrad && p.gather_flags != nullptr && lane == 0) {
        // Rows of this tile are pulled by the gather warps of some CTA; wait (bounded) for their blocks.
        int last = (t.row0 + kBM - 1) >> 7;
        const int nblocks = (total_rows + 127) >> 7;
        if (last > nblocks - 1) last = nblocks - 1;
        if (last >= ready_blocks) {
          const uint64_t t0 = globaltimer_ns();
          for (int b = ready_blocks > (t.row0 >> 7) ? ready_blocks : (t.row0 >> 7); b <= last && ok; ++b) {
            uint32_t spins = 0;
            while (ld_acquire_gpu(p.gather_flags + b) < kGatherUnitsPerBlock) {
              if ((++spins & 0xff) == 0 && (abort_flag || globaltimer_ns() - t0 > 2000000000ull)) {
                abort_flag = 1;
                ok = false;
                break;
              }
            }
          }
          if (ok) ready_blocks = last + 1;
          fence_proxy_async_all();  // rows were written with ordinary stores, TMA reads them through the async proxy
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      for (int kb = 0; kb < t.k_iters; ++kb) {
        if (lane == 0) {
          ok = mbar_wait(&empty_bar[stage], phase ^ 1u, &abort_flag);
          if (ok) {
            uint8_t* sa = smem + stage * kStageBytes;
            uint8_t* sb = sa + kABytes;
            if (kMode != kWgrad || wgrad_part == 0) mbar_arrive_expect_tx(&full_bar[stage], kStageBytes);
            if (kMode == kWgrad) {
              const int row = t.row0 + kb * kBK;
              if (wgrad_part == 0) {
#pragma unroll
                for (int b = 0; b < kBM / 64; ++b)
                  tma_load_3d(sa + b * 8192, &p.tm_a, 0, a_line0 + t.m_blk * (kBM / 64) + b, row, &full_bar[stage]);
              } else {
                const int b0 = (wgrad_part - 1) * 2;
#pragma unroll
                for (int b = b0; b < b0 + 2; ++b)
                  tma_load_3d(sb + b * 8192, &p.tm_b, 0, b_line0 + t.n_blk * (kBN / 64) + b, row, &full_bar[stage]);
              }
            } else {
              tma_load_3d(sa, &p.tm_a, 0, a_line0 + kb, t.row0, &full_bar[stage]);
              if (kMode == kFprop) {
                int r0, r1;
                if (p.fused) {
                  const int F = p.N / 2;
                  r0 = t.e * p.N + t.n_blk * (kBN / 2);
                  r1 = r0 + F;
                } else {
                  r0 = t.e * p.N + t.n_blk * kBN;
                  r1 = r0 + kBN / 2;
                }
                if (p.fused) {
                  tma_load_2d(sb, &p.tm_b, kb * kBK, r0, &full_bar[stage]);
                  tma_load_2d(sb + kBBytes / 2, &p.tm_b, kb * kBK, r1, &full_bar[stage]);
                } else {
                  tma_load_2d(sb, &p.tm_b256, kb * kBK, r0, &full_bar[stage]);
                }
              } else {
#pragma unroll
                for (int b = 0; b < kBN / 64; ++b)
                  tma_load_2d(sb + b * 8192, &p.tm_b, t.n_blk * kBN + b * 64, t.e * p.Kd + kb * kBK,
                              &full_bar[stage]);
              }
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    // ======================= MMA issuer =======================
    // One thread runs the whole issue loop: a poll of the stage barrier, the K = 16 MMAs with descriptor words
    // derived by integer adds, one commit.  The other lanes join only where a weight-gradient tile ends in a
    // ragged chunk whose tail rows must be zeroed in shared memory.  (Per-stage warp synchronisation in this
    // loop costs about a quarter of the tensor time of a stage; tiles of the weight gradient are only a few
    // stages long, so it mattered most there.)
    constexpr uint32_t idesc = umma_idesc_bf16(kBM, kBN, kMode == kWgrad ? 1 : 0, kMode == kFprop ? 0 : 1);
    constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);  // SBO 1024, version 1, 128-byte swizzle
    constexpr uint32_t kLboK = (16u >> 4) << 16, kLboMN = (8192u >> 4) << 16;
    constexpr uint32_t a_step = kMode == kWgrad ? (2048u >> 4) : (32u >> 4);
    constexpr uint32_t b_step = kMode == kFprop ? (32u >> 4) : (2048u >> 4);
    const uint32_t a_lo0 = ((smem_u32(smem) & 0x3ffffu) >> 4) | (kMode == kWgrad ? kLboMN : kLboK);
    const uint32_t b_lo0 = (((smem_u32(smem) + kABytes) & 0x3ffffu) >> 4) | (kMode == kFprop ? kLboK : kLboMN);
    const uint32_t empty0 = smem_u32(&empty_bar[0]), tfull0 = smem_u32(&tmem_full_bar[0]);
    int stage = 0;
    uint32_t phase = 0;
    int e = 0;
    int it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      const Tile t = decode_tile<kMode>(tile, e, s_tile_start, s_off, n_tiles, p.Kd);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      const uint32_t d_tmem = tmem_base + buf * kBN;
      // weight gradient: rows of the last chunk that belong to the expert, and whether its tail needs zeroing
      const int valid_last = kMode == kWgrad ? (t.row_end - t.row0) - (t.k_iters - 1) * kBK : kBK;
      const bool ragged = kMode == kWgrad && t.k_iters > 0 && (valid_last & 15) != 0;
      if (ragged && t.k_iters <= 16) {
        // Short ragged tile: the lanes that must zero the tail stay in step with the issuing lane for the
        // whole tile (re-joining lanes that waited through a single-thread loop costs about a microsecond,
        // which only long tiles can afford).
        if (lane == 0) ok = mbar_wait(&tmem_empty_bar[buf], acc_phase ^ 1u, &abort_flag);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (!ok) break;
        tcgen05_fence_after();
        for (int kb = 0; kb < t.k_iters; ++kb) {
          if (lane == 0) ok = mbar_wait(&full_bar[stage], phase, &abort_flag);
          ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
          if (!ok) break;
          int ksteps = kBK / 16;
          if (kb == t.k_iters - 1) {
            uint8_t* sa = smem + stage * kStageBytes;
            ksteps = (valid_last + 15) >> 4;
            const int vec_per_box = (ksteps * 16 - valid_last) * 8;
            const int boxes = (kBM + kBN) / 64;
            for (int i = lane; i < boxes * vec_per_box; i += 32) {
              const int box = i / vec_per_box, v = i - box * vec_per_box;
              reinterpret_cast<uint4*>(sa + box * 8192 + valid_last * 128)[v] = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
            __syncwarp();
          }
          if (lane == 0) {
            const uint32_t a_lo = a_lo0 + stage * (kStageBytes >> 4), b_lo = b_lo0 + stage * (kStageBytes >> 4);
            umma_bf16_lo(d_tmem, a_lo, b_lo, kDescHi, idesc, kb > 0 ? 1u : 0u);
            if (ksteps > 1) umma_bf16_lo(d_tmem, a_lo + a_step, b_lo + b_step, kDescHi, idesc, 1u);
            if (ksteps > 2) umma_bf16_lo(d_tmem, a_lo + 2 * a_step, b_lo + 2 * b_step, kDescHi, idesc, 1u);
            if (ksteps > 3) umma_bf16_lo(d_tmem, a_lo + 3 * a_step, b_lo + 3 * b_step, kDescHi, idesc, 1u);
            tcgen05_commit_addr(empty0 + stage * 8);
          }
          __syncwarp();
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        if (lane == 0) tcgen05_commit_addr(tfull0 + buf * 8);
        __syncwarp();
        continue;
      }
      const int solo = ragged ? t.k_iters - 1 : t.k_iters;  // stages lane 0 handles alone
      if (lane == 0) {
        ok = mbar_wait(&tmem_empty_bar[buf], acc_phase ^ 1u, &abort_flag);
        tcgen05_fence_after();
        int st = stage;
        uint32_t ph = phase;
        for (int kb = 0; kb < solo && ok; ++kb) {
          ok = mbar_wait(&full_bar[st], ph, &abort_flag);
          if (!ok) break;
          const uint32_t a_lo = a_lo0 + st * (kStageBytes >> 4), b_lo = b_lo0 + st * (kStageBytes >> 4);
          const int ksteps = (kMode == kWgrad && kb == t.k_iters - 1) ? (valid_last + 15) >> 4 : kBK / 16;
          umma_bf16_lo(d_tmem, a_lo, b_lo, kDescHi, idesc, kb > 0 ? 1u : 0u);
          if (ksteps > 1) umma_bf16_lo(d_tmem, a_lo + a_step, b_lo + b_step, kDescHi, idesc, 1u);
          if (ksteps > 2) umma_bf16_lo(d_tmem, a_lo + 2 * a_step, b_lo + 2 * b_step, kDescHi, idesc, 1u);
          if (ksteps > 3) umma_bf16_lo(d_tmem, a_lo + 3 * a_step, b_lo + 3 * b_step, kDescHi, idesc, 1u);
          tcgen05_commit_addr(empty0 + st * 8);
          if (++st == kStages) {
            st = 0;
            ph ^= 1u;
          }
        }
      }
      {  // every lane tracks the ring position
        const int adv = stage + solo;
        phase ^= static_cast<uint32_t>(adv / kStages) & 1u;
        stage = adv % kStages;
      }
      if (ragged) {
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (ok && lane == 0) ok = mbar_wait(&full_bar[stage], phase, &abort_flag);
        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        if (ok) {
          // Ragged last chunk: only the K = 16 steps that hold rows of this expert are issued, and the rows
          // between the expert's end and the end of its last step (at most 15) are zeroed in shared memory.
          // Row r of every 64 x 64 box is one contiguous 128-byte line.
          uint8_t* sa = smem + stage * kStageBytes;
          const int ksteps = (valid_last + 15) >> 4;
          const int vec_per_box = (ksteps * 16 - valid_last) * 8;
          const int boxes = (kBM + kBN) / 64;
          for (int i = lane; i < boxes * vec_per_box; i += 32) {
            const int box = i / vec_per_box, v = i - box * vec_per_box;
            reinterpret_cast<uint4*>(sa + box * 8192 + valid_last * 128)[v] = make_uint4(0, 0, 0, 0);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            const uint32_t a_lo = a_lo0 + stage * (kStageBytes >> 4), b_lo = b_lo0 + stage * (kStageBytes >> 4);
            umma_bf16_lo(d_tmem, a_lo, b_lo, kDescHi, idesc, t.k_iters > 1 ? 1u : 0u);
            if (ksteps > 1) umma_bf16_lo(d_tmem, a_lo + a_step, b_lo + b_step, kDescHi, idesc, 1u);
            if (ksteps > 2) umma_bf16_lo(d_tmem, a_lo + 2 * a_step, b_lo + 2 * b_step, kDescHi, idesc, 1u);
            if (ksteps > 3) umma_bf16_lo(d_tmem, a_lo + 3 * a_step, b_lo + 3 * b_step, kDescHi, idesc, 1u);
            tcgen05_commit_addr(empty0 + stage * 8);
          }
        }
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (lane == 0) {
        if (t.k_iters > 0)
          tcgen05_commit_addr(tfull0 + buf * 8);
        else
          mbar_arrive(&tmem_full_bar[buf]);
      }
      __syncwarp();
    }
  } else if (warp == 14) {
    // ======================= accumulator watcher =======================
    // One warp polls the accumulator-ready barriers on behalf of the eight epilogue warps and releases them
    // through a hardware named barrier: the epilogue warps then sleep without taking issue slots from the
    // MMA-issuing and TMA-issuing threads that share their schedulers.  The watcher arrives for every tile,
    // also after a timeout, so that no epilogue warp is left blocked.
    bool ok = true;
    int it = 0;
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++it) {
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      if (ok && lane == 0) ok = mbar_wait(&tmem_full_bar[buf], acc_phase, &abort_flag);
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      asm volatile("bar.arrive %0, %1;" ::"r"(1 + buf), "r"(8 * 32 + 32) : "memory");
    }
  } else if (warp >= 10) {
    // ======================= gather (fused dispatch) =======================
    // Units of 8 rows are dealt round-robin over all gather warps of the grid in ascending row order, the order
    // in which the tiles consume them.  Each warp pulls its unit with 16-byte loads (peer memory allowed), two rows
    // x eight loads in flight per lane, and then bumps the counter of the unit's 128-row block; the TMA producer of
    // whichever CTA needs a block waits for sixteen reports.  Gather warps wait on nothing.  Small units matter at
    // the start of the launch: a warp keeps 8 KiB in flight, so over NVLink a 32-row unit took about 30 us before
    // the first tiles could begin, an 8-row unit a quarter of that, and later units are far ahead of the MMAs anyway.
    if (kMode != kWgrad && p.gather_flags != nullptr) {
      const int gw = warp - 10;
      const int total_rows = s_off[p.e_local];
      const int nblocks = (total_rows + 127) >> 7;
      const int vec_per_row = p.Kd / 8;
      uint4* dst_base = reinterpret_cast<uint4*>(p.a_base + a_off);
      for (int u = gw * gridDim.x + blockIdx.x; u < nblocks * kGatherUnitsPerBlock; u += kGatherWarps * gridDim.x) {
        const int blk = u / kGatherUnitsPerBlock;
        const int r_begin = blk * 128 + (u % kGatherUnitsPerBlock) * kGatherUnitRows;
        for (int rr = 0; rr < kGatherUnitRows; rr += 2) {
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
    // ======================= epilogue =======================
    // Eight warps: two per TMEM lane quadrant, each owning half of the tile's columns.  A lane reads
    // its own accumulator row from TMEM 32 columns at a time; the warp transposes the 32x32 block
    // through a private staging tile (32 rows x 64 bytes, 16-byte chunks XOR-swizzled so that both
    // directions are bank-conflict free) and stores 64-byte row segments: 4 lanes per row, 8 rows
    // per instruction.
    const int ew = warp - 2;            // 0..7
    const int quad = warp & 3;          // TMEM lanes [32*quad, 32*quad+32)
    const int half = ew >> 2;           // column half of the tile
    const int row_in_tile = quad * 32 + lane;
    uint8_t* stg = smem + kStages * kStageBytes + ew * kStaging64Bytes;
    int e = 0;
    int it = 0;
    bool ok = true;
    const int64_t c_off = p.c_off ? *p.c_off : 0;
    const int64_t h2_off = p.h2_off ? *p.h2_off : 0;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
      const Tile t = decode_tile<kMode>(tile, e, s_tile_start, s_off, n_tiles, p.Kd);
      const int buf = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      asm volatile("bar.sync %0, %1;" ::"r"(1 + buf), "r"(8 * 32 + 32) : "memory");  // released by the watcher
      (void)acc_phase;
      ok = abort_flag == 0;
      if (!ok) break;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + buf * kBN;
      if (kMode == kWgrad) {
        // 128 bytes of output columns per trip (64 bf16 or 32 fp32).  The staging tile is laid out as a 16-row x
        // 128-byte box in the 128-byte swizzle, so the warp's 32 rows go in two passes; one thread hands each
        // box to the copy engine, which stores it or adds it to dW in L2 (accumulation rounds the fp32
        // accumulator to the stored type first, then L2 adds whole 128-byte lines: no read round trip through
        // the SM) and clips rows and columns past the matrix.
        const int cols_per_trip = p.out_fp32 ? 32 : 64;
        for (int c0 = half * (kBN / 2); c0 < (half + 1) * (kBN / 2); c0 += cols_per_trip) {
          uint32_t r0[32], r1[32];
          if (t.k_iters > 0) {
            tmem_ld_32x32(taddr + c0, r0);
            if (!p.out_fp32) tmem_ld_32x32(taddr + c0 + 32, r1);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) r0[j] = r1[j] = 0u;
          }
          const int cc = t.n_blk * kBN + c0;
#pragma unroll
          for (int pass = 0; pass < 2; ++pass) {
            if (lane == 0) bulk_wait_read();  // the engine has read the previous box out of the staging tile
            __syncwarp();
            if ((lane >> 4) == pass) {
              const int rr = lane & 15;
              if (p.out_fp32) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                  stage_put(stg, rr, j, make_uint4(r0[4 * j], r0[4 * j + 1], r0[4 * j + 2], r0[4 * j + 3]));
              } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  stage_put(stg, rr, j, pack8_bf16(r0 + 8 * j));
                  stage_put(stg, rr, j + 4, pack8_bf16(r1 + 8 * j));
                }
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            const int box_row = t.m_blk * kBM + quad * 32 + pass * 16;
            if (lane == 0 && box_row < p.N && cc < p.Kd) {
              if (p.accumulate)
                tma_reduce_add_3d(&p.tm_c, stg, cc, box_row, t.e);
              else
                tma_store_3d(&p.tm_c, stg, cc, box_row, t.e);
              bulk_commit();
            }
          }
        }
      } else {
        const int row = t.row0 + row_in_tile;
        const bool row_ok = row < t.row_end;
        uint64_t my_row = 0;
        if (row_ok) {
          if (p.scatter_ptrs != nullptr)
            my_row = static_cast<uint64_t>(p.scatter_ptrs[row]);
          else
            my_row = reinterpret_cast<uint64_t>(p.c_base) + c_off + static_cast<uint64_t>(row) * p.N * 2;
        }
        if (kMode == kFprop && p.fused) {
          const int F = p.N / 2;
          const uint64_t my_h2 =
              row_ok ? reinterpret_cast<uint64_t>(p.h2_base) + h2_off + static_cast<uint64_t>(row) * F * 2 : 0ull;
          for (int c0 = half * (kBN / 4); c0 < (half + 1) * (kBN / 4); c0 += 32) {
            uint32_t g[32], u[32];
            tmem_ld_32x32(taddr + c0, g);
            tmem_ld_32x32(taddr + kBN / 2 + c0, u);
            tmem_ld_wait();
            uint4 gp[4], up[4], zp[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              uint32_t gw[4], uw[4], zw[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                gw[q] = pack_bf16x2(__uint_as_float(g[8 * j + 2 * q]), __uint_as_float(g[8 * j + 2 * q + 1]));
                uw[q] = pack_bf16x2(__uint_as_float(u[8 * j + 2 * q]), __uint_as_float(u[8 * j + 2 * q + 1]));
                const float z0 = swiglu_f32(__uint_as_float(gw[q] << 16), __uint_as_float(uw[q] << 16), p.act);
                const float z1 =
                    swiglu_f32(__uint_as_float(gw[q] & 0xffff0000u), __uint_as_float(uw[q] & 0xffff0000u), p.act);
                zw[q] = pack_bf16x2(z0, z1);
              }
              gp[j] = make_uint4(gw[0], gw[1], gw[2], gw[3]);
              up[j] = make_uint4(uw[0], uw[1], uw[2], uw[3]);
              zp[j] = make_uint4(zw[0], zw[1], zw[2], zw[3]);
            }
            const int col = t.n_blk * (kBN / 2) + c0;  // column inside the gate (and up) half
#pragma unroll
            for (int which = 0; which < 3; ++which) {
#pragma unroll
              for (int j = 0; j < 4; ++j) stage64_put(stg, lane, j, which == 0 ? gp[j] : (which == 1 ? up[j] : zp[j]));
              __syncwarp();
              const uint64_t base = which == 2 ? my_h2 : my_row;
              const int col_out = which == 1 ? F + col : col;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int rr = i * 8 + (lane >> 2), j = lane & 3;
                const uint4 v = stage64_get(stg, rr, j);
                const uint64_t rp = __shfl_sync(0xffffffffu, base, rr);
                if (rp != 0 && col + 8 * j + 8 <= F)
                  *reinterpret_cast<uint4*>(rp + static_cast<uint64_t>(col_out + 8 * j) * 2) = v;
              }
              __syncwarp();
            }
          }
        } else {
          // 64 columns per trip: a row segment is 128 contiguous bytes, the unit that peer (NVLink) and local
          // stores move best.  The staging tile holds 16 rows x 128 bytes, so the warp's 32 rows go in two passes.
          for (int c0 = half * (kBN / 2); c0 < (half + 1) * (kBN / 2); c0 += 64) {
            uint32_t r0[32], r1[32];
            tmem_ld_32x32(taddr + c0, r0);
            tmem_ld_32x32(taddr + c0 + 32, r1);
            tmem_ld_wait();
            const int col = t.n_blk * kBN + c0;
#pragma unroll
            for (int pass = 0; pass < 2; ++pass) {
              if ((lane >> 4) == pass) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  stage_put(stg, lane & 15, j, pack8_bf16(r0 + 8 * j));
                  stage_put(stg, lane & 15, j + 4, pack8_bf16(r1 + 8 * j));
                }
              }
              __syncwarp();
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int rr = i * 4 + (lane >> 3), j = lane & 7;
                const uint4 v = stage_get(stg, rr, j);
                const uint64_t rp = __shfl_sync(0xffffffffu, my_row, pass * 16 + rr);
                if (rp != 0 && col + 8 * j + 8 <= p.N)
                  *reinterpret_cast<uint4*>(rp + static_cast<uint64_t>(col + 8 * j) * 2) = v;
              }
              __syncwarp();
            }
          }
        }
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[buf]);
    }
    if (kMode == kWgrad && lane == 0) bulk_wait_all();  // staged boxes are out of shared memory and written
  }

  // ---- teardown ---------------------------------------------------------------
  tcgen05_fence_before();
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) set_status(p.status, kPipelineTimeout, kMode, blockIdx.x);
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

template <int kMode>
static int launch(const GemmParams& p, int num_sms, cudaStream_t st) {
  static PerDeviceOnce attr_set;
  const int rc = once_per_device(attr_set, [] {
    return static_cast<int>(cudaFuncSetAttribute(grouped_gemm_kernel<kMode>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(kGemmSmemBytes)));
  });
  if (rc != 0) return rc;
  const int grid = persistent_grid(num_sms);
  grouped_gemm_kernel<kMode><<<grid, kGemmThreads, kGemmSmemBytes, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace dm

using namespace dm;

static int setup_gather(GemmParams& p, const dm_operand& a, const int64_t* gather_ptrs, int32_t* gather_flags,
                        int64_t max_rows, cudaStream_t st) {
  if (gather_ptrs == nullptr) return kRcOk;
  if (gather_flags == nullptr) return kRcBadArg;
  p.gather_ptrs = gather_ptrs;
  p.gather_flags = gather_flags;
  p.a_base = static_cast<uint8_t*>(a.base);
  const cudaError_t e = cudaMemsetAsync(gather_flags, 0, sizeof(int32_t) * static_cast<size_t>((max_rows + 127) / 128 + 1), st);
  return static_cast<int>(e);
}

static int fprop_impl(dm_operand a, const void* w, dm_operand c, dm_operand h2, const int64_t* scatter_ptrs,
                      const int64_t* gather_ptrs, int32_t* gather_flags, const int32_t* expert_offsets, int e_local,
                      int64_t max_rows, int64_t N, int64_t Kd, int fuse_swiglu, int clamped, float alpha, float limit,
                      const int* cond, int num_sms, int* status, void* stream) {
  if (!a.base || !w || !expert_offsets || e_local <= 0 || max_rows < 0 || N <= 0 || Kd <= 0) return kRcBadArg;
  if (!c.base && !scatter_ptrs) return kRcBadArg;
  if (e_local > kMaxGroups || max_rows > (1 << 30)) return kRcTooLarge;
  if ((Kd % 64) != 0 || (N % 8) != 0) return kRcUnsupportedShape;
  if (fuse_swiglu && (((N / 2) % (kBN / 2)) != 0 || !h2.base || !c.base || scatter_ptrs)) return kRcUnsupportedShape;
  if (max_rows == 0) return kRcOk;
  if (gather_ptrs != nullptr && gather_flags == nullptr) return kRcBadArg;
  GemmParams p{};
  int rc = encode_arena(&p.tm_a, a, Kd * 2, max_rows + 256, kBM);
  if (rc != kRcOk) return rc;
  rc = encode_2d(&p.tm_b, w, static_cast<int64_t>(e_local) * N, Kd, kBN / 2);
  if (rc != kRcOk) return rc;
  rc = encode_2d(&p.tm_b256, w, static_cast<int64_t>(e_local) * N, Kd, kBN);
  if (rc != kRcOk) return rc;
  p.a_off = a.offset;
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
  p.fused = fuse_swiglu ? 1 : 0;
  p.act = ActParams{clamped, alpha, limit};
  rc = setup_gather(p, a, gather_ptrs, gather_flags, max_rows, static_cast<cudaStream_t>(stream));
  if (rc != kRcOk) return rc;
  return launch<kFprop>(p, num_sms, static_cast<cudaStream_t>(stream));
}

extern "C" int dm_gemm_fprop(dm_operand a, const void* w, dm_operand c, dm_operand h2, const int64_t* scatter_ptrs,
                             const int32_t* expert_offsets, int e_local, int64_t max_rows, int64_t N, int64_t Kd,
                             int fuse_swiglu, int clamped, float alpha, float limit, const int* cond, int num_sms,
                             int* status, void* stream) {
  return fprop_impl(a, w, c, h2, scatter_ptrs, nullptr, nullptr, expert_offsets, e_local, max_rows, N, Kd, fuse_swiglu,
                    clamped, alpha, limit, cond, num_sms, status, stream);
}

extern "C" int dm_gemm_fprop_dispatch(const int64_t* gather_ptrs, int32_t* gather_flags, dm_operand a, const void* w,
                                      dm_operand c, dm_operand h2, const int32_t* expert_offsets, int e_local,
                                      int64_t max_rows, int64_t N, int64_t Kd, int fuse_swiglu, int clamped,
                                      float alpha, float limit, const int* cond, int num_sms, int* status,
                                      void* stream) {
  if (!gather_ptrs || !gather_flags) return kRcBadArg;
  return fprop_impl(a, w, c, h2, nullptr, gather_ptrs, gather_flags, expert_offsets, e_local, max_rows, N, Kd,
                    fuse_swiglu, clamped, alpha, limit, cond, num_sms, status, stream);
}

static int dgrad_impl(dm_operand a, const void* w, dm_operand c, const int64_t* scatter_ptrs,
                      const int64_t* gather_ptrs, int32_t* gather_flags, const int32_t* expert_offsets, int e_local,
                      int64_t max_rows, int64_t N, int64_t Kd, const int* cond, int num_sms, int* status,
                      void* stream) {
  if (!a.base || !w || !expert_offsets || e_local <= 0 || max_rows < 0 || N <= 0 || Kd <= 0) return kRcBadArg;
  if (!c.base && !scatter_ptrs) return kRcBadArg;
  if (e_local > kMaxGroups || max_rows > (1 << 30)) return kRcTooLarge;
  if ((Kd % 64) != 0 || (N % 8) != 0) return kRcUnsupportedShape;
  if (max_rows == 0) return kRcOk;
  if (gather_ptrs != nullptr && gather_flags == nullptr) return kRcBadArg;
  GemmParams p{};
  int rc = encode_arena(&p.tm_a, a, Kd * 2, max_rows + 256, kBM);
  if (rc != kRcOk) return rc;
  // W = [e_local * Kd][N], N contiguous; box = 64 k-rows x 64 columns.
  rc = encode_2d(&p.tm_b, w, static_cast<int64_t>(e_local) * Kd, N, 64);
  if (rc != kRcOk) return rc;
  p.a_off = a.offset;
  p.c_off = c.offset;
  p.c_base = static_cast<uint8_t*>(c.base);
  p.scatter_ptrs = scatter_ptrs;
  p.expert_offsets = expert_offsets;
  p.cond = cond;
  p.status = status;
  p.e_local = e_local;
  p.max_rows = static_cast<int>(max_rows);
  p.N = static_cast<int>(N);
  p.Kd = static_cast<int>(Kd);
  rc = setup_gather(p, a, gather_ptrs, gather_flags, max_rows, static_cast<cudaStream_t>(stream));
  if (rc != kRcOk) return rc;
  return launch<kDgrad>(p, num_sms, static_cast<cudaStream_t>(stream));
}

extern "C" int dm_gemm_dgrad(dm_operand a, const void* w, dm_operand c, const int64_t* scatter_ptrs,
                             const int32_t* expert_offsets, int e_local, int64_t max_rows, int64_t N, int64_t Kd,
                             const int* cond, int num_sms, int* status, void* stream) {
  return dgrad_impl(a, w, c, scatter_ptrs, nullptr, nullptr, expert_offsets, e_local, max_rows, N, Kd, cond, num_sms,
                    status, stream);
}

extern "C" int dm_gemm_dgrad_dispatch(const int64_t* gather_ptrs, int32_t* gather_flags, dm_operand a, const void* w,
                                      dm_operand c, const int32_t* expert_offsets, int e_local, int64_t max_rows,
                                      int64_t N, int64_t Kd, const int* cond, int num_sms, int* status, void* stream) {
  if (!gather_ptrs || !gather_flags) return kRcBadArg;
  return dgrad_impl(a, w, c, nullptr, gather_ptrs, gather_flags, expert_offsets, e_local, max_rows, N, Kd, cond,
                    num_sms, status, stream);
}

extern "C" int dm_gemm_wgrad(dm_operand dy, dm_operand x, void* dw, int out_is_fp32, int accumulate,
                             const int32_t* expert_offsets, int e_local, int64_t max_rows, int64_t N, int64_t Kd,
                             int num_sms, int* status, void* stream) {
  if (!dy.base || !x.base || !dw || !expert_offsets || e_local <= 0 || max_rows < 0 || N <= 0 || Kd <= 0)
    return kRcBadArg;
  if (e_local > kMaxGroups || max_rows > (1 << 30)) return kRcTooLarge;
  if ((N % 64) != 0 || (Kd % 64) != 0) return kRcUnsupportedShape;
  if ((reinterpret_cast<uintptr_t>(dw) % 16) != 0) return kRcBadArg;
  GemmParams p{};
  int rc = encode_arena(&p.tm_a, dy, N * 2, max_rows + 256, kBK);
  if (rc != kRcOk) return rc;
  rc = encode_arena(&p.tm_b, x, Kd * 2, max_rows + 256, kBK);
  if (rc != kRcOk) return rc;
  p.a_off = dy.offset;
  p.b_off = x.offset;
  p.c_base = static_cast<uint8_t*>(dw);
  p.expert_offsets = expert_offsets;
  p.status = status;
  p.e_local = e_local;
  p.max_rows = static_cast<int>(max_rows);
  p.N = static_cast<int>(N);
  p.Kd = static_cast<int>(Kd);
  p.out_fp32 = out_is_fp32 ? 1 : 0;
  p.accumulate = accumulate ? 1 : 0;
  rc = encode_out_3d(&p.tm_c, dw, e_local, N, Kd, out_is_fp32 != 0);
  if (rc != kRcOk) return rc;
  return launch<kWgrad>(p, num_sms, static_cast<cudaStream_t>(stream));
}
