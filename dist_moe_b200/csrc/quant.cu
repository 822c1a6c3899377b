// Block-scaled quantisers: MXFP8 E4M3 (E8M0 scale per 32 elements) and NVFP4 (E2M1 data,
// E4M3 scale per 16 elements, fp32 per-token or per-expert scale).  All HBM bound:
// 16-byte loads, byte-exact hardware conversions (cvt.rp.ue8m0, cvt.rn.satfinite.e4m3x2,
// cvt.rn.satfinite.e2m1x2 through the cuda_fp8/cuda_fp4 intrinsics), no fast-math.
//
// Numerics follow the reference's quantisers step by step
// (dist_moe/kernels/blockscaled_quantization_common.py:120-257, 739-752;
//  dist_moe/kernels/triton_quantization/blockscaled_quantize.py:296-493):
//   MXFP8: s = amax * fl(1/448); byte = round-up-to-power-of-two(s); recip = 2^(127-byte);
//          q = e4m3_rn_satfinite(x * recip); a non-finite block gets byte 0xFF and NaN data.
//   NVFP4: raw = (amax * scale) * fl(1/6) clamped to [2^-9, 448]; byte = e4m3_rn(raw);
//          mult = div_rn(scale, f32(byte)); codes = e2m1_rn_satfinite(x * mult), even element
//          in the low nibble.
#include <cuda_fp4.h>

#include "quant_common.cuh"
#include "../../include/dist_moe_b200.h"

namespace dm {

// ---------------------------------------------------------------------------
// MXFP8 row mode: 1x32 blocks along the contiguous dimension.  8 elements per
// thread, 4 threads per block.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) mxfp8_row_kernel(const uint4* __restrict__ x, const int32_t* num_rows,
                                                        int64_t max_rows, int vec_per_row, uint8_t* __restrict__ q,
                                                        int64_t q_stride, uint8_t* __restrict__ scales,
                                                        int64_t s_stride, int blocked, int n_col_atoms) {
  int64_t rows = num_rows ? *num_rows : max_rows;
  if (rows > max_rows) rows = max_rows;
  const int64_t total = rows * vec_per_row;
  const int64_t start = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t step = static_cast<int64_t>(gridDim.x) * blockDim.x;
  // The bound is rounded up to a whole warp so that every lane takes part in the shuffles.
  for (int64_t i = start; i < (total + 31) / 32 * 32; i += step) {
    const bool live = i < total;
    float f[8];
    if (live) {
      unpack8f(x[i], f);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) amax = amax_nonfinite(amax, f[j]);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    float recip;
    const uint8_t byte = mxfp8_scale(amax, recip);
    if (!live) continue;
    const int64_t r = i / vec_per_row;
    const int v = static_cast<int>(i - r * vec_per_row);
    *reinterpret_cast<uint2*>(q + r * q_stride + v * 8) =
        make_uint2(e4m3x4(f[0] * recip, f[1] * recip, f[2] * recip, f[3] * recip),
                   e4m3x4(f[4] * recip, f[5] * recip, f[6] * recip, f[7] * recip));
    if ((v & 3) == 0) {
      const int blk = v >> 2;
      if (blocked)
        scales[blocked_offset(r, blk, n_col_atoms)] = byte;
      else
        scales[r * s_stride + blk] = byte;
    }
  }
}

// ---------------------------------------------------------------------------
// MXFP8 column mode (32x1 blocks along the rows) and 32x32 tile mode.
// One CTA handles a 32-row x 256-column slab staged in shared memory.
//   col mode : scale[c][r/32]           (natural: [C][ceil(R/32)], or blocked with rows = C)
//   tile mode: one scale per 32x32 tile, written for both GEMM orientations:
//              row_scales[n][k/32] (forward) and col_scales[k][n/32] (input gradient).
// ---------------------------------------------------------------------------
template <bool kTile>
__global__ void __launch_bounds__(256) mxfp8_slab_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* num_rows,
                                                         int64_t max_rows, int C, uint8_t* __restrict__ q,
                                                         uint8_t* __restrict__ s0, uint8_t* __restrict__ s1,
                                                         int blocked, int s0_col_atoms, int s1_col_atoms,
                                                         int64_t batch_rows, uint8_t* __restrict__ q_row = nullptr,
                                                         uint8_t* __restrict__ s_row = nullptr, int row_col_atoms = 0) {
  __shared__ float tile[32][257];
  __shared__ float col_amax[256];
  int64_t rows = num_rows ? *num_rows : max_rows;
  if (rows > max_rows) rows = max_rows;
  const int64_t row0 = static_cast<int64_t>(blockIdx.y) * 32;
  const int col0 = blockIdx.x * 256;
  if (row0 >= rows) return;
  const int t = threadIdx.x;
  for (int i = t; i < 32 * 256; i += 256) {
    const int r = i >> 8, c = i & 255;
    float v = 0.f;
    if (row0 + r < rows && col0 + c < C) v = __bfloat162float(x[(row0 + r) * C + col0 + c]);
    tile[r][c] = v;
  }
  __syncthreads();
  {
    float a = 0.f;
#pragma unroll 8
    for (int r = 0; r < 32; ++r) a = amax_nonfinite(a, tile[r][t]);
    col_amax[t] = a;
  }
  __syncthreads();
  float amax = col_amax[t];
  if (kTile) {
    const int g = t & ~31;
    amax = 0.f;
    for (int j = 0; j < 32; ++j) {
      const float v = col_amax[g + j];
      amax = (v != v || amax != amax) ? __int_as_float(0x7f800000) : fmaxf(amax, v);
    }
  }
  float recip;
  const uint8_t byte = mxfp8_scale(amax, recip);
  const int c = col0 + t;
  if (c < C) {
    if (kTile) {
      // batch_rows = rows of one expert: scale tensors are per-expert blocked groups.
      const int64_t e = row0 / batch_rows, rl = row0 - e * batch_rows;
      if ((t & 31) == 0) {
        // forward orientation: 32 rows share the byte for k-block c/32
        for (int r = 0; r < 32 && row0 + r < rows; ++r) {
          const int64_t rr = row0 + r;
          if (blocked) {
            const int64_t grp = (batch_rows + 127) / 128 * 128 * static_cast<int64_t>(s0_col_atoms) * 4;
            s0[e * grp + blocked_offset(rl + r, c >> 5, s0_col_atoms)] = byte;
          } else {
            s0[rr * ((C + 31) / 32) + (c >> 5)] = byte;
          }
        }
      }
      if (s1 != nullptr) {
        // input-gradient orientation: row index = k (this column), column = n-block
        const int64_t nb = rl >> 5;
        if (blocked) {
          const int64_t grp = (static_cast<int64_t>(C) + 127) / 128 * 128 * static_cast<int64_t>(s1_col_atoms) * 4;
          s1[e * grp + blocked_offset(c, static_cast<int>(nb), s1_col_atoms)] = byte;
        } else {
          s1[(e * C + c) * ((batch_rows + 31) / 32) + nb] = byte;
        }
      }
    } else {
      const int64_t rb = row0 >> 5;
      if (blocked)
        s0[blocked_offset(c, static_cast<int>(rb), s0_col_atoms)] = byte;
      else
        s0[static_cast<int64_t>(c) * ((max_rows + 31) / 32) + rb] = byte;
    }
  }
  if (!kTile && q_row != nullptr) {
    // Row-quantised copy from the same staged slab (1 x 32 blocks along the columns): warp b takes the
    // 32-column block b, lane r its row r, so the shared-memory reads of a warp hit 32 different banks.
    const int b = t >> 5, r = t & 31;
    const int colb = col0 + b * 32;
    if (row0 + r < rows && colb < C) {
      float ra = 0.f;
#pragma unroll 8
      for (int j = 0; j < 32; ++j) ra = amax_nonfinite(ra, tile[r][b * 32 + j]);
      float rrecip;
      const uint8_t rbyte = mxfp8_scale(ra, rrecip);
      uint32_t w[8];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        w[j] = e4m3x4(tile[r][b * 32 + 4 * j] * rrecip, tile[r][b * 32 + 4 * j + 1] * rrecip,
                      tile[r][b * 32 + 4 * j + 2] * rrecip, tile[r][b * 32 + 4 * j + 3] * rrecip);
      uint4* dst = reinterpret_cast<uint4*>(q_row + (row0 + r) * C + colb);
      dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
      dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
      s_row[blocked_offset(row0 + r, colb >> 5, row_col_atoms)] = rbyte;
    }
  }
  // every thread converts one column of the slab: 32 rows, written as bytes into shared memory first
  __syncthreads();
  for (int r = 0; r < 32; ++r) tile[r][t] = tile[r][t] * recip;
  __syncthreads();
  for (int i = t; i < 32 * 64; i += 256) {
    const int r = i >> 6, c4 = (i & 63) * 4;
    if (row0 + r < rows && col0 + c4 < C) {
      const uint32_t w = e4m3x4(tile[r][c4], tile[r][c4 + 1], tile[r][c4 + 2], tile[r][c4 + 3]);
      *reinterpret_cast<uint32_t*>(q + (row0 + r) * C + col0 + c4) = w;
    }
  }
}

// ---------------------------------------------------------------------------
// MXFP8 column mode, optionally with the row-quantised copy, for activations: the bandwidth-bound form.
//
// A CTA stages a slab of 32 rows x 512 columns as raw bf16 (16-byte loads, rows 1040 bytes apart so that
// 16-byte reads of eight consecutive rows fall into different bank groups).  Block maxima are taken on the
// bit patterns: |x| of a bf16 is its low 15 bits, their unsigned order is the order of the magnitudes, and
// any pattern above 0x7f80 is a NaN, which makes the block non-finite exactly as the fp32 rule does
// (bf16 -> fp32 is exact).  Two 16-bit lanes are compared per instruction.
//   column pass: thread t owns columns 2t and 2t+1 (one 32-bit word per row);
//   row pass   : lane r of a warp owns row r of one 32-column block (four 16-byte reads).
// The column pass sweeps the slab twice (maxima, then conversion) instead of holding 32 rows in registers, which
// lets six CTAs share an SM; it stores two bytes per lane, 64 contiguous bytes per warp and row.
// ---------------------------------------------------------------------------
constexpr int kSlabCols = 512;
constexpr int kSlabRawStride = kSlabCols * 2 + 16;


// Where a slab comes from: a dense [rows, C] matrix; rows named by a pointer table (a null pointer is a row of
// zeros; pointers may address peer memory); or SwiGLU of a dense [rows, 2C] matrix [gate | up], rounded to
// bf16 exactly as the standalone activation kernel rounds it.
enum SlabSource : int { kSlabDense = 0, kSlabGather = 1, kSlabSwiglu = 2 };

// Row pass, column pass and stores for one staged slab (see above).  `limit` bounds the columns this slab may
// touch (the matrix width, or the end of the gate half when a CTA stages two slabs), `C` is the row pitch of the
// outputs.  Called by every thread of the CTA after the slab has been written and a barrier has passed.
__device__ __forceinline__ void slab_quantise(uint8_t* slab, int64_t rows, int64_t row0, int col0, int limit, int C,
                                              int64_t max_rows, uint8_t* __restrict__ q_col, uint8_t* __restrict__ s_col,
                                              int blocked, int col_atoms, uint8_t* __restrict__ q_row,
                                              uint8_t* __restrict__ s_row, int row_atoms) {
  const int t = threadIdx.x;
  if (q_row != nullptr) {
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int r = t & 31, b = (t >> 5) + 8 * k;
      const int colb = col0 + b * 32;
      if (row0 + r < rows && colb < limit) {
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 v = *reinterpret_cast<const uint4*>(slab + r * kSlabRawStride + b * 64 + j * 16);
          w[4 * j] = v.x; w[4 * j + 1] = v.y; w[4 * j + 2] = v.z; w[4 * j + 3] = v.w;
        }
        uint32_t m = 0;
#pragma unroll
        for (int j = 0; j < 16; ++j) m = __vmaxu2(m, w[j] & 0x7fff7fffu);
        const uint32_t top = (m >> 16) > (m & 0xffffu) ? (m >> 16) : (m & 0xffffu);
        float recip;
        const uint8_t byte = mxfp8_scale(amax_from_bf16_bits(top), recip);
        uint32_t o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
          o[j] = e4m3x4(__uint_as_float(w[2 * j] << 16) * recip, __uint_as_float(w[2 * j] & 0xffff0000u) * recip,
                        __uint_as_float(w[2 * j + 1] << 16) * recip, __uint_as_float(w[2 * j + 1] & 0xffff0000u) * recip);
        uint4* dst = reinterpret_cast<uint4*>(q_row + (row0 + r) * C + colb);
        dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
        dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
        s_row[blocked_offset(row0 + r, colb >> 5, row_atoms)] = byte;
      }
    }
  }
  if (q_col == nullptr) return;  // uniform over the CTA

  // column pass: 32 rows of two adjacent columns per thread, in two sweeps over the staged slab (maxima, then
  // conversion) so that no row values are held in registers; a warp's 2-byte stores cover 64 contiguous bytes.
  uint32_t m = 0;
#pragma unroll
  for (int r = 0; r < 32; ++r)
    m = __vmaxu2(m, *reinterpret_cast<const uint32_t*>(slab + r * kSlabRawStride + t * 4) & 0x7fff7fffu);
  float recip0, recip1;
  const uint8_t byte0 = mxfp8_scale(amax_from_bf16_bits(m & 0xffffu), recip0);
  const uint8_t byte1 = mxfp8_scale(amax_from_bf16_bits(m >> 16), recip1);
  const int c = col0 + 2 * t;
  if (c >= limit) return;
  const int64_t rb = row0 >> 5;
  if (blocked) {
    s_col[blocked_offset(c, static_cast<int>(rb), col_atoms)] = byte0;
    s_col[blocked_offset(c + 1, static_cast<int>(rb), col_atoms)] = byte1;
  } else {
    const int64_t per_col = (max_rows + 31) / 32;
    s_col[static_cast<int64_t>(c) * per_col + rb] = byte0;
    s_col[static_cast<int64_t>(c + 1) * per_col + rb] = byte1;
  }
  const int live = rows - row0 < 32 ? static_cast<int>(rows - row0) : 32;
  uint8_t* dst = q_col + row0 * C + c;
#pragma unroll 8
  for (int r = 0; r < live; ++r) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(slab + r * kSlabRawStride + t * 4);
    const uint32_t pk = __nv_cvt_float2_to_fp8x2(
        make_float2(__uint_as_float(w << 16) * recip0, __uint_as_float(w & 0xffff0000u) * recip1), __NV_SATFINITE,
        __NV_E4M3);
    *reinterpret_cast<uint16_t*>(dst + static_cast<int64_t>(r) * C) = static_cast<uint16_t>(pk);
  }
}

// Placement chosen on the device: each pointer is an allocation base and the byte offset is read from device memory
// when the kernel starts (all null = the pointers are final).  `compact_cols` sizes the column-scale layout from the
// device row count instead of max_rows, so that a column bundle occupies exactly dim * rows / 32 bytes; `cond`
// (optional) turns the whole launch into a no-op when it reads 0.
struct PlacedOffsets {
  const int64_t* x;
  const int64_t* x2;
  const int64_t* q_col;
  const int64_t* s_col;
  const int64_t* q_row;
  const int64_t* s_row;
  const int* cond;
  int compact_cols;
};

template <class T>
__device__ __forceinline__ T* placed(T* base, const int64_t* off) {
  if (base == nullptr || off == nullptr) return base;
  return reinterpret_cast<T*>(reinterpret_cast<uintptr_t>(base) + static_cast<uintptr_t>(*off));
}

template <int kSource>
__global__ void __launch_bounds__(256) mxfp8_colrow_kernel(const uint4* __restrict__ x, const int64_t* __restrict__ row_ptrs,
                                                           ActParams act, const int32_t* num_rows,
                                                           int64_t max_rows, int C, uint8_t* __restrict__ q_col,
                                                           uint8_t* __restrict__ s_col, int blocked, int col_atoms,
                                                           uint8_t* __restrict__ q_row, uint8_t* __restrict__ s_row,
                                                           int row_atoms, PlacedOffsets at) {
  __shared__ __align__(16) uint8_t slab[32 * kSlabRawStride];
  if (at.cond != nullptr && *at.cond == 0) return;
  int64_t rows = num_rows ? *num_rows : max_rows;
  if (rows > max_rows) rows = max_rows;
  x = placed(x, at.x);
  q_col = placed(q_col, at.q_col);
  s_col = placed(s_col, at.s_col);
  q_row = placed(q_row, at.q_row);
  s_row = placed(s_row, at.s_row);
  if (at.compact_cols) col_atoms = static_cast<int>(((rows + 31) / 32 + 3) / 4);
  const int64_t row0 = static_cast<int64_t>(blockIdx.y) * 32;
  const int col0 = blockIdx.x * kSlabCols;
  if (row0 >= rows) return;
  const int t = threadIdx.x;
  const int vec_per_row = C >> 3;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int i = t + 256 * k;
    const int r = i >> 6, v = i & 63;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (row0 + r < rows && col0 + v * 8 < C) {
      if (kSource == kSlabDense) {
        val = x[(row0 + r) * vec_per_row + (col0 >> 3) + v];
      } else if (kSource == kSlabGather) {
        const uint4* src = reinterpret_cast<const uint4*>(row_ptrs[row0 + r]);
        if (src != nullptr) val = __ldcg(src + (col0 >> 3) + v);
      } else {
        const uint4 g4 = x[(row0 + r) * 2 * vec_per_row + (col0 >> 3) + v];
        const uint4 u4 = x[(row0 + r) * 2 * vec_per_row + vec_per_row + (col0 >> 3) + v];
        float g[8], u[8];
        unpack8f(g4, g);
        unpack8f(u4, u);
        uint32_t z[4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
          z[j] = pack_bf16x2(swiglu_f32(g[2 * j], u[2 * j], act), swiglu_f32(g[2 * j + 1], u[2 * j + 1], act));
        val = make_uint4(z[0], z[1], z[2], z[3]);
      }
    }
    *reinterpret_cast<uint4*>(slab + r * kSlabRawStride + v * 16) = val;
  }
  __syncthreads();
  slab_quantise(slab, rows, row0, col0, C, C, max_rows, q_col, s_col, blocked, col_atoms, q_row, s_row, row_atoms);
}

// SwiGLU backward fused in: from h1 = [gate | up] ([rows, 2F]) and dz = dL/dh2 ([rows, F]) a CTA computes the
// gate-gradient slab and the matching up-gradient slab of grad_h1 = [dgate | dup] (rounded to bf16 as the standalone
// backward kernel rounds them) and quantises both; grad_h1 itself is never written.  Either copy may be left out.
__global__ void __launch_bounds__(256) mxfp8_swiglu_bwd_colrow_kernel(const uint4* __restrict__ h1,
                                                                      const uint4* __restrict__ dz, ActParams act,
                                                                      const int32_t* num_rows, int64_t max_rows, int F,
                                                                      uint8_t* __restrict__ q_col,
                                                                      uint8_t* __restrict__ s_col, int col_atoms,
                                                                      uint8_t* __restrict__ q_row,
                                                                      uint8_t* __restrict__ s_row, int row_atoms,
                                                                      PlacedOffsets at) {
  extern __shared__ __align__(16) uint8_t slabs[];  // two slabs
  uint8_t* slab_g = slabs;
  uint8_t* slab_u = slabs + 32 * kSlabRawStride;
  int64_t rows = num_rows ? *num_rows : max_rows;
  if (rows > max_rows) rows = max_rows;
  h1 = placed(h1, at.x);
  dz = placed(dz, at.x2);
  q_col = placed(q_col, at.q_col);
  s_col = placed(s_col, at.s_col);
  q_row = placed(q_row, at.q_row);
  s_row = placed(s_row, at.s_row);
  if (at.compact_cols) col_atoms = static_cast<int>(((rows + 31) / 32 + 3) / 4);
  const int64_t row0 = static_cast<int64_t>(blockIdx.y) * 32;
  const int col0 = blockIdx.x * kSlabCols;
  if (row0 >= rows) return;
  const int t = threadIdx.x;
  const int vec_per_row = F >> 3;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int i = t + 256 * k;
    const int r = i >> 6, v = i & 63;
    uint4 dg4 = make_uint4(0, 0, 0, 0), du4 = make_uint4(0, 0, 0, 0);
    if (row0 + r < rows && col0 + v * 8 < F) {
      float x[8], y[8], d[8], dx[8], dy[8];
      unpack8f(h1[(row0 + r) * 2 * vec_per_row + (col0 >> 3) + v], x);
      unpack8f(h1[(row0 + r) * 2 * vec_per_row + vec_per_row + (col0 >> 3) + v], y);
      unpack8f(dz[(row0 + r) * vec_per_row + (col0 >> 3) + v], d);
#pragma unroll
      for (int j = 0; j < 8; ++j) swiglu_bwd_f32(x[j], y[j], d[j], act, dx[j], dy[j]);
      dg4 = make_uint4(pack_bf16x2(dx[0], dx[1]), pack_bf16x2(dx[2], dx[3]), pack_bf16x2(dx[4], dx[5]), pack_bf16x2(dx[6], dx[7]));
      du4 = make_uint4(pack_bf16x2(dy[0], dy[1]), pack_bf16x2(dy[2], dy[3]), pack_bf16x2(dy[4], dy[5]), pack_bf16x2(dy[6], dy[7]));
    }
    *reinterpret_cast<uint4*>(slab_g + r * kSlabRawStride + v * 16) = dg4;
    *reinterpret_cast<uint4*>(slab_u + r * kSlabRawStride + v * 16) = du4;
  }
  __syncthreads();
  slab_quantise(slab_g, rows, row0, col0, F, 2 * F, max_rows, q_col, s_col, 1, col_atoms, q_row, s_row, row_atoms);
  slab_quantise(slab_u, rows, row0, F + col0, 2 * F, 2 * F, max_rows, q_col, s_col, 1, col_atoms, q_row, s_row, row_atoms);
}

// ---------------------------------------------------------------------------
// NVFP4
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint8_t nvfp4_block_scale(float amax, float scale, float& mult) {
  if (amax == __int_as_float(0x7f800000)) amax = __int_as_float(0x7fc00000);
  float raw = (amax * scale) * (1.0f / 6.0f);
  raw = raw < 0.001953125f ? 0.001953125f : raw;
  raw = raw > 448.0f ? 448.0f : raw;
  const uint8_t byte =
      static_cast<uint8_t>(__nv_cvt_float2_to_fp8x2(make_float2(raw, 0.f), __NV_SATFINITE, __NV_E4M3) & 0xFF);
  const __half_raw h = __nv_cvt_fp8_to_halfraw(byte, __NV_E4M3);
  const float sf = __half2float(*reinterpret_cast<const __half*>(&h));
  mult = byte != 0 ? __fdiv_rn(scale, sf) : 0.f;
  return byte;
}

__device__ __forceinline__ uint32_t e2m1x8(const float (&f)[8], float m) {
  uint32_t out = 0;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t b = __nv_cvt_float2_to_fp4x2(make_float2(f[2 * i] * m, f[2 * i + 1] * m), __NV_E2M1, cudaRoundNearest);
    out |= (b & 0xFF) << (8 * i);
  }
  return out;
}

// One CTA (128 threads) per token row: row amax, then 16-element blocks (2 threads each).
__global__ void __launch_bounds__(128) nvfp4_token_kernel(const uint4* __restrict__ x, const int32_t* num_rows,
                                                          int64_t max_rows, int vec_per_row, uint8_t* q,
                                                          int64_t q_stride, uint8_t* s, int64_t s_stride,
                                                          uint8_t* inv, int64_t inv_stride, int blocked_atoms,
                                                          const int64_t* __restrict__ live) {
  __shared__ float red[4];
  int64_t rows = num_rows ? *num_rows : max_rows;
  if (rows > max_rows) rows = max_rows;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    if (live != nullptr && live[r] == 0) continue;  // a padding row: nothing reads its quantised form
    const uint4* xr = x + r * vec_per_row;
    float amax = 0.f;
    for (int v = threadIdx.x; v < vec_per_row; v += 128) {
      float f[8];
      unpack8f(xr[v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(f[j]));
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    const float row_scale = 2688.0f * __frcp_rn(fmaxf(amax, 1e-8f));
    if (threadIdx.x == 0 && inv != nullptr) *reinterpret_cast<float*>(inv + r * inv_stride) = __frcp_rn(row_scale);
    for (int v0 = 0; v0 < vec_per_row; v0 += 128) {
      const int v = v0 + threadIdx.x;
      float f[8];
      float bmax = 0.f;
      if (v < vec_per_row) {
        unpack8f(xr[v], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) bmax = amax_nonfinite(bmax, f[j]);
      }
      const float other = __shfl_xor_sync(0xffffffffu, bmax, 1);
      bmax = (other != other) ? other : fmaxf(bmax, other);
      float mult;
      const uint8_t byte = nvfp4_block_scale(bmax, row_scale, mult);
      if (v < vec_per_row) {
        *reinterpret_cast<uint32_t*>(q + r * q_stride + v * 4) = e2m1x8(f, mult);
        if ((v & 1) == 0) {
          if (blocked_atoms > 0)
            s[blocked_offset(r, v >> 1, blocked_atoms)] = byte;
          else
            s[r * s_stride + (v >> 1)] = byte;
        }
      }
    }
  }
}

// Rows of up to 2048 elements: one warp per row, the row stays in registers between the row-maximum pass and
// the quantising pass (no second read, no block-wide barriers).  Same arithmetic as the kernel above.
template <int kVpl>
__global__ void __launch_bounds__(256) nvfp4_token_warp_kernel(const uint4* __restrict__ x, const int32_t* num_rows,
                                                               int64_t max_rows, int vec_per_row, uint8_t* q,
                                                               int64_t q_stride, uint8_t* s, int64_t s_stride,
                                                               uint8_t* inv, int64_t inv_stride, int blocked_atoms,
                                                               const int64_t* __restrict__ live) {
  int64_t rows = num_rows ? *num_rows : max_rows;
  if (rows > max_rows) rows = max_rows;
  const int lane = threadIdx.x & 31;
  const int64_t warps = static_cast<int64_t>(gridDim.x) * (blockDim.x >> 5);
  for (int64_t r = static_cast<int64_t>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5); r < rows; r += warps) {
    if (live != nullptr && live[r] == 0) continue;  // a padding row: nothing reads its quantised form
    const uint4* xr = x + r * vec_per_row;
    uint4 raw[kVpl];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < kVpl; ++j) {
      const int v = j * 32 + lane;
      raw[j] = v < vec_per_row ? xr[v] : make_uint4(0, 0, 0, 0);
      float f[8];
      unpack8f(raw[j], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
    }
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, d));
    const float row_scale = 2688.0f * __frcp_rn(fmaxf(amax, 1e-8f));
    if (lane == 0 && inv != nullptr) *reinterpret_cast<float*>(inv + r * inv_stride) = __frcp_rn(row_scale);
#pragma unroll
    for (int j = 0; j < kVpl; ++j) {
      const int v = j * 32 + lane;
      float f[8];
      unpack8f(raw[j], f);
      float bmax = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) bmax = amax_nonfinite(bmax, f[i]);
      const float other = __shfl_xor_sync(0xffffffffu, bmax, 1);
      bmax = (other != other) ? other : fmaxf(bmax, other);
      float mult;
      const uint8_t byte = nvfp4_block_scale(bmax, row_scale, mult);
      if (v < vec_per_row) {
        *reinterpret_cast<uint32_t*>(q + r * q_stride + v * 4) = e2m1x8(f, mult);
        if ((v & 1) == 0) {
          if (blocked_atoms > 0)
            s[blocked_offset(r, v >> 1, blocked_atoms)] = byte;
          else
            s[r * s_stride + (v >> 1)] = byte;
        }
      }
    }
  }
}

// Weights: per-expert global scale given; rows of K elements; scales natural or blocked per expert.
__global__ void __launch_bounds__(256) nvfp4_weight_kernel(const uint4* __restrict__ w, const float* __restrict__ gs,
                                                           int64_t rows_per_expert, int64_t total_rows,
                                                           int vec_per_row, uint32_t* __restrict__ q,
                                                           uint8_t* __restrict__ s, int blocked, int n_col_atoms) {
  const int64_t total = total_rows * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < (total + 31) / 32 * 32;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const bool live = i < total;
    const int64_t r = live ? i / vec_per_row : 0;
    const int64_t e = r / rows_per_expert;
    float f[8];
    float bmax = 0.f;
    if (live) {
      unpack8f(w[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) bmax = amax_nonfinite(bmax, f[j]);
    }
    const float other = __shfl_xor_sync(0xffffffffu, bmax, 1);
    bmax = (other != other) ? other : fmaxf(bmax, other);
    if (!live) continue;
    float g = gs[e];
    g = g > 1e-12f ? g : 1e-12f;
    float mult;
    const uint8_t byte = nvfp4_block_scale(bmax, g, mult);
    q[i] = e2m1x8(f, mult);
    if ((i & 1) == 0) {
      const int blk = static_cast<int>(i - r * vec_per_row) >> 1;
      if (blocked) {
        const int64_t rl = r - e * rows_per_expert;
        const int64_t grp = (rows_per_expert + 127) / 128 * 128 * static_cast<int64_t>(n_col_atoms) * 4;
        s[e * grp + blocked_offset(rl, blk, n_col_atoms)] = byte;
      } else {
        s[r * (vec_per_row >> 1) + blk] = byte;
      }
    }
  }
}

// natural [rows][cols] scale bytes -> blocked atoms (padding entries are written as 0)
__global__ void sf_swizzle_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t rows, int cols,
                                  int64_t padded_rows, int n_col_atoms) {
  const int64_t total = padded_rows * n_col_atoms * 4;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / (n_col_atoms * 4);
    const int c = static_cast<int>(i - r * (n_col_atoms * 4));
    dst[blocked_offset(r, c, n_col_atoms)] = (r < rows && c < cols) ? src[r * cols + c] : 0;
  }
}

// Packed dispatch rows [q | natural scales | fp32 inverse scale | pad] fetched through a pointer table
// (sources may be peer memory) and unpacked into GEMM operand form: dense q rows, blocked scales,
// per-row inverse scales.  A null pointer yields a zero row.
__global__ void __launch_bounds__(256) gather_packed_kernel(const int64_t* __restrict__ ptrs,
                                                            const int32_t* __restrict__ num_rows, int64_t max_rows,
                                                            int q_vecs, int scale_cols, int has_inv, uint8_t* q_base,
                                                            const int64_t* q_off, uint8_t* sf_base,
                                                            const int64_t* sf_off, uint8_t* inv_base,
                                                            const int64_t* inv_off, const int* cond) {
  if (cond != nullptr && *cond == 0) return;
  int64_t rows = *num_rows;
  if (rows > max_rows) rows = max_rows;
  uint4* q = reinterpret_cast<uint4*>(q_base + (q_off ? *q_off : 0));
  uint8_t* sf = sf_base + (sf_off ? *sf_off : 0);
  float* inv = has_inv ? reinterpret_cast<float*>(inv_base + (inv_off ? *inv_off : 0)) : nullptr;
  const int atoms = (scale_cols + 3) / 4;
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  for (int64_t r = blockIdx.x * static_cast<int64_t>(wpb) + (threadIdx.x >> 5); r < rows;
       r += static_cast<int64_t>(gridDim.x) * wpb) {
    const uint8_t* src = reinterpret_cast<const uint8_t*>(ptrs[r]);
    for (int v0 = lane; v0 < q_vecs; v0 += 128) {  // four 16-byte loads in flight per lane
      uint4 t[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int v = v0 + 32 * j;
        t[j] = (src && v < q_vecs) ? __ldcg(reinterpret_cast<const uint4*>(src) + v) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int v = v0 + 32 * j;
        if (v < q_vecs) q[r * q_vecs + v] = t[j];
      }
    }
    const uint8_t* ssrc = src ? src + static_cast<int64_t>(q_vecs) * 16 : nullptr;
    for (int c4 = lane; c4 < atoms; c4 += 32) {
      uint32_t w = 0;
      if (ssrc) {
        if (c4 * 4 + 4 <= scale_cols) {
          w = __ldcg(reinterpret_cast<const uint32_t*>(ssrc) + c4);
        } else {
          for (int j = 0; c4 * 4 + j < scale_cols; ++j) w |= static_cast<uint32_t>(ssrc[c4 * 4 + j]) << (8 * j);
        }
      }
      *reinterpret_cast<uint32_t*>(sf + blocked_offset(r, c4 * 4, atoms)) = w;
    }
    if (inv != nullptr && lane == 0)
      inv[r] = src ? __ldcg(reinterpret_cast<const float*>(ssrc + scale_cols)) : 0.f;
  }
}

static int blocks_for(int64_t items, int threads, int cap) {
  int64_t b = (items + threads - 1) / threads;
  if (b > cap) b = cap;
  return b < 1 ? 1 : static_cast<int>(b);
}

}  // namespace dm

using namespace dm;

extern "C" int dm_quant_mxfp8_row(const void* x, const int32_t* num_rows, int64_t max_rows, int64_t C, void* q,
                                  int64_t q_row_stride, void* scales, int64_t scale_row_stride, int blocked,
                                  void* stream) {
  if (!x || !q || !scales || max_rows < 0 || C <= 0 || (C % 32) != 0) return kRcBadArg;
  if (q_row_stride == 0) q_row_stride = C;
  if (scale_row_stride == 0) scale_row_stride = C / 32;
  if ((q_row_stride % 8) != 0) return kRcBadArg;
  if (max_rows == 0) return kRcOk;
  const int vec = static_cast<int>(C / 8);
  const int atoms = static_cast<int>((C / 32 + 3) / 4);
  mxfp8_row_kernel<<<blocks_for(max_rows * vec, 256, grid_cap(16)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), num_rows, max_rows, vec, static_cast<uint8_t*>(q), q_row_stride,
      static_cast<uint8_t*>(scales), scale_row_stride, blocked, atoms);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_quant_mxfp8_col(const void* x, const int32_t* num_rows, int64_t max_rows, int64_t C, void* q,
                                  void* scales, int blocked, void* stream) {
  if (!x || !q || !scales || max_rows < 0 || C <= 0 || (C % 4) != 0) return kRcBadArg;
  if (max_rows == 0) return kRcOk;
  const int atoms = static_cast<int>(((max_rows + 31) / 32 + 3) / 4);
  if ((C % 16) == 0 && ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(q)) % 16) == 0) {
    const dim3 fast(static_cast<unsigned>((C + kSlabCols - 1) / kSlabCols), static_cast<unsigned>((max_rows + 31) / 32));
    mxfp8_colrow_kernel<kSlabDense><<<fast, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(x), nullptr, ActParams{0, 1.0f, 0.0f}, num_rows, max_rows, static_cast<int>(C),
        static_cast<uint8_t*>(q), static_cast<uint8_t*>(scales), blocked, atoms, nullptr, nullptr, 0, PlacedOffsets{});
    return static_cast<int>(cudaGetLastError());
  }
  const dim3 grid(static_cast<unsigned>((C + 255) / 256), static_cast<unsigned>((max_rows + 31) / 32));
  mxfp8_slab_kernel<false><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), num_rows, max_rows, static_cast<int>(C), static_cast<uint8_t*>(q),
      static_cast<uint8_t*>(scales), nullptr, blocked, atoms, 0, max_rows);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_quant_mxfp8_rowcol(const void* x, const int32_t* num_rows, int64_t max_rows, int64_t C, void* q_row,
                                     void* scales_row_blocked, void* q_col, void* scales_col_blocked, void* stream) {
  if (!x || !q_row || !scales_row_blocked || !q_col || !scales_col_blocked || max_rows < 0 || C <= 0 || (C % 32) != 0)
    return kRcBadArg;
  if (max_rows == 0) return kRcOk;
  const dim3 grid(static_cast<unsigned>((C + kSlabCols - 1) / kSlabCols), static_cast<unsigned>((max_rows + 31) / 32));
  const int col_atoms = static_cast<int>(((max_rows + 31) / 32 + 3) / 4);
  const int row_atoms = static_cast<int>((C / 32 + 3) / 4);
  mxfp8_colrow_kernel<kSlabDense><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), nullptr, ActParams{0, 1.0f, 0.0f}, num_rows, max_rows, static_cast<int>(C),
      static_cast<uint8_t*>(q_col), static_cast<uint8_t*>(scales_col_blocked), 1, col_atoms,
      static_cast<uint8_t*>(q_row), static_cast<uint8_t*>(scales_row_blocked), row_atoms, PlacedOffsets{});
  return static_cast<int>(cudaGetLastError());
}

static int launch_rowcol_gather(const int64_t* row_ptrs, const int32_t* num_rows, int64_t max_rows, int64_t C,
                                void* q_row, void* sf_row, void* q_col, void* sf_col, PlacedOffsets at, void* stream) {
  if (!row_ptrs || !q_row || !sf_row || (q_col == nullptr) != (sf_col == nullptr) || max_rows < 0 || C <= 0 ||
      (C % 32) != 0)
    return kRcBadArg;  // the column copy may be left out (a forward nothing will differentiate)
  if (max_rows == 0) return kRcOk;
  const dim3 grid(static_cast<unsigned>((C + kSlabCols - 1) / kSlabCols), static_cast<unsigned>((max_rows + 31) / 32));
  const int col_atoms = static_cast<int>(((max_rows + 31) / 32 + 3) / 4);
  const int row_atoms = static_cast<int>((C / 32 + 3) / 4);
  mxfp8_colrow_kernel<kSlabGather><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      nullptr, row_ptrs, ActParams{0, 1.0f, 0.0f}, num_rows, max_rows, static_cast<int>(C), static_cast<uint8_t*>(q_col),
      static_cast<uint8_t*>(sf_col), 1, col_atoms, static_cast<uint8_t*>(q_row), static_cast<uint8_t*>(sf_row),
      row_atoms, at);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_quant_mxfp8_rowcol_gather(const int64_t* row_ptrs, const int32_t* num_rows, int64_t max_rows, int64_t C,
                                            void* q_row, void* scales_row_blocked, void* q_col,
                                            void* scales_col_blocked, void* stream) {
  return launch_rowcol_gather(row_ptrs, num_rows, max_rows, C, q_row, scales_row_blocked, q_col, scales_col_blocked,
                              PlacedOffsets{}, stream);
}

extern "C" int dm_quant_mxfp8_rowcol_gather_at(const int64_t* row_ptrs, const int32_t* num_rows, int64_t max_rows,
                                               int64_t C, dm_operand q_row, dm_operand sf_row, dm_operand q_col,
                                               dm_operand sf_col, const int* cond, void* stream) {
  PlacedOffsets at{nullptr, nullptr, q_col.offset, sf_col.offset, q_row.offset, sf_row.offset, cond, 1};
  return launch_rowcol_gather(row_ptrs, num_rows, max_rows, C, q_row.base, sf_row.base, q_col.base, sf_col.base, at,
                              stream);
}

static int launch_swiglu_fwd_quant(const void* h1, const int32_t* num_rows, int64_t max_rows, int64_t F, int clamped,
                                   float alpha, float limit, void* q_row, void* sf_row, void* q_col, void* sf_col,
                                   PlacedOffsets at, void* stream) {
  if (!h1 || !q_row || !sf_row || (q_col == nullptr) != (sf_col == nullptr) || max_rows < 0 || F <= 0 || (F % 32) != 0)
    return kRcBadArg;
  if (max_rows == 0) return kRcOk;
  const dim3 grid(static_cast<unsigned>((F + kSlabCols - 1) / kSlabCols), static_cast<unsigned>((max_rows + 31) / 32));
  const int col_atoms = static_cast<int>(((max_rows + 31) / 32 + 3) / 4);
  const int row_atoms = static_cast<int>((F / 32 + 3) / 4);
  mxfp8_colrow_kernel<kSlabSwiglu><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(h1), nullptr, ActParams{clamped, alpha, limit}, num_rows, max_rows, static_cast<int>(F),
      static_cast<uint8_t*>(q_col), static_cast<uint8_t*>(sf_col), 1, col_atoms, static_cast<uint8_t*>(q_row),
      static_cast<uint8_t*>(sf_row), row_atoms, at);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_swiglu_fwd_quant_mxfp8_rowcol(const void* h1, const int32_t* num_rows, int64_t max_rows, int64_t F,
                                                int clamped, float alpha, float limit, void* q_row,
                                                void* scales_row_blocked, void* q_col, void* scales_col_blocked,
                                                void* stream) {
  return launch_swiglu_fwd_quant(h1, num_rows, max_rows, F, clamped, alpha, limit, q_row, scales_row_blocked, q_col,
                                 scales_col_blocked, PlacedOffsets{}, stream);
}

extern "C" int dm_swiglu_fwd_quant_mxfp8_rowcol_at(dm_operand h1, const int32_t* num_rows, int64_t max_rows, int64_t F,
                                                   int clamped, float alpha, float limit, dm_operand q_row,
                                                   dm_operand sf_row, dm_operand q_col, dm_operand sf_col,
                                                   const int* cond, void* stream) {
  PlacedOffsets at{h1.offset, nullptr, q_col.offset, sf_col.offset, q_row.offset, sf_row.offset, cond, 1};
  return launch_swiglu_fwd_quant(h1.base, num_rows, max_rows, F, clamped, alpha, limit, q_row.base, sf_row.base,
                                 q_col.base, sf_col.base, at, stream);
}

static int launch_swiglu_bwd_quant(const void* h1, const void* grad_h2, const int32_t* num_rows, int64_t max_rows,
                                   int64_t F, int clamped, float alpha, float limit, void* q_row, void* sf_row,
                                   void* q_col, void* sf_col, PlacedOffsets at, void* stream) {
  if (!h1 || !grad_h2 || max_rows < 0 || F <= 0 || (F % 32) != 0) return kRcBadArg;
  if ((q_row == nullptr) != (sf_row == nullptr) || (q_col == nullptr) != (sf_col == nullptr) ||
      (q_row == nullptr && q_col == nullptr))
    return kRcBadArg;
  if (max_rows == 0) return kRcOk;
  constexpr int kSmem = 2 * 32 * kSlabRawStride;
  static PerDeviceOnce attr_set;
  const int rc_attr = once_per_device(attr_set, [] {
    return static_cast<int>(
        cudaFuncSetAttribute(mxfp8_swiglu_bwd_colrow_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  });
  if (rc_attr != 0) return rc_attr;
  const dim3 grid(static_cast<unsigned>((F + kSlabCols - 1) / kSlabCols), static_cast<unsigned>((max_rows + 31) / 32));
  const int col_atoms = static_cast<int>(((max_rows + 31) / 32 + 3) / 4);
  const int row_atoms = static_cast<int>((2 * F / 32 + 3) / 4);
  mxfp8_swiglu_bwd_colrow_kernel<<<grid, 256, kSmem, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(h1), static_cast<const uint4*>(grad_h2), ActParams{clamped, alpha, limit}, num_rows,
      max_rows, static_cast<int>(F), static_cast<uint8_t*>(q_col), static_cast<uint8_t*>(sf_col), col_atoms,
      static_cast<uint8_t*>(q_row), static_cast<uint8_t*>(sf_row), row_atoms, at);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_swiglu_bwd_quant_mxfp8(const void* h1, const void* grad_h2, const int32_t* num_rows, int64_t max_rows,
                                        int64_t F, int clamped, float alpha, float limit, void* q_row,
                                        void* scales_row_blocked, void* q_col, void* scales_col_blocked, void* stream) {
  return launch_swiglu_bwd_quant(h1, grad_h2, num_rows, max_rows, F, clamped, alpha, limit, q_row, scales_row_blocked,
                                 q_col, scales_col_blocked, PlacedOffsets{}, stream);
}

extern "C" int dm_swiglu_bwd_quant_mxfp8_at(dm_operand h1, dm_operand grad_h2, const int32_t* num_rows,
                                           int64_t max_rows, int64_t F, int clamped, float alpha, float limit,
                                           dm_operand q_row, dm_operand sf_row, dm_operand q_col, dm_operand sf_col,
                                           void* stream) {
  PlacedOffsets at{h1.offset, grad_h2.offset, q_col.offset, sf_col.offset, q_row.offset, sf_row.offset, nullptr, 1};
  return launch_swiglu_bwd_quant(h1.base, grad_h2.base, num_rows, max_rows, F, clamped, alpha, limit, q_row.base,
                                 sf_row.base, q_col.base, sf_col.base, at, stream);
}

extern "C" int dm_quant_mxfp8_tile32(const void* w, int64_t experts, int64_t N, int64_t K, void* q, void* row_scales,
                                     void* col_scales, int blocked, void* stream) {
  if (!w || !q || !row_scales || experts <= 0 || N <= 0 || K <= 0 || (N % 32) != 0 || (K % 32) != 0) return kRcBadArg;
  const int64_t rows = experts * N;
  const dim3 grid(static_cast<unsigned>((K + 255) / 256), static_cast<unsigned>(rows / 32));
  mxfp8_slab_kernel<true><<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(w), nullptr, rows, static_cast<int>(K), static_cast<uint8_t*>(q),
      static_cast<uint8_t*>(row_scales), static_cast<uint8_t*>(col_scales), blocked,
      static_cast<int>((K / 32 + 3) / 4), static_cast<int>((N / 32 + 3) / 4), N);
  return static_cast<int>(cudaGetLastError());
}

static int nvfp4_token_impl(const int64_t* live, const void* x, const int32_t* num_rows, int64_t max_rows, int64_t C, void* q,
                                    int64_t q_row_stride, void* scales, int64_t scale_row_stride, int scales_blocked,
                                    void* scale_inv, int64_t inv_row_stride, void* stream) {
  if (!x || !q || !scales || max_rows < 0 || C <= 0 || (C % 16) != 0 || (q_row_stride % 4) != 0) return kRcBadArg;
  if (scale_inv && (inv_row_stride % 4) != 0) return kRcBadArg;
  if (max_rows == 0) return kRcOk;
  const int vec = static_cast<int>(C / 8);
  if (vec <= 256) {
    const int atoms = scales_blocked ? static_cast<int>((C / 16 + 3) / 4) : 0;
    const int blocks = blocks_for(max_rows, 8, grid_cap(8));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define DM_TOKEN_WARP(VPL)                                                                                            \
    nvfp4_token_warp_kernel<VPL><<<blocks, 256, 0, st>>>(static_cast<const uint4*>(x), num_rows, max_rows, vec,         \
                                                         static_cast<uint8_t*>(q), q_row_stride,                        \
                                                         static_cast<uint8_t*>(scales), scale_row_stride,               \
                                                         static_cast<uint8_t*>(scale_inv), inv_row_stride, atoms, live)
    if (vec <= 64) {
      DM_TOKEN_WARP(2);
    } else if (vec <= 128) {
      DM_TOKEN_WARP(4);
    } else {
      DM_TOKEN_WARP(8);
    }
#undef DM_TOKEN_WARP
    return static_cast<int>(cudaGetLastError());
  }
  nvfp4_token_kernel<<<blocks_for(max_rows, 1, grid_cap(16)), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(x), num_rows, max_rows, static_cast<int>(C / 8), static_cast<uint8_t*>(q),
      q_row_stride, static_cast<uint8_t*>(scales), scale_row_stride, static_cast<uint8_t*>(scale_inv),
      inv_row_stride, scales_blocked ? static_cast<int>((C / 16 + 3) / 4) : 0, live);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_quant_nvfp4_token(const void* x, const int32_t* num_rows, int64_t max_rows, int64_t C, void* q,
                                    int64_t q_row_stride, void* scales, int64_t scale_row_stride, int scales_blocked,
                                    void* scale_inv, int64_t inv_row_stride, void* stream) {
  return nvfp4_token_impl(nullptr, x, num_rows, max_rows, C, q, q_row_stride, scales, scale_row_stride, scales_blocked,
                          scale_inv, inv_row_stride, stream);
}

extern "C" int dm_quant_nvfp4_token_live(const int64_t* row_live, const void* x, const int32_t* num_rows,
                                         int64_t max_rows, int64_t C, void* q, int64_t q_row_stride, void* scales,
                                         int64_t scale_row_stride, int scales_blocked, void* scale_inv,
                                         int64_t inv_row_stride, void* stream) {
  if (!row_live) return kRcBadArg;
  return nvfp4_token_impl(row_live, x, num_rows, max_rows, C, q, q_row_stride, scales, scale_row_stride, scales_blocked,
                          scale_inv, inv_row_stride, stream);
}

extern "C" int dm_quant_nvfp4_weight(const void* w, const float* global_scale, int64_t experts, int64_t N, int64_t K,
                                     void* q, void* scales, int blocked, void* stream) {
  if (!w || !global_scale || !q || !scales || experts <= 0 || N <= 0 || K <= 0 || (K % 16) != 0) return kRcBadArg;
  const int vec = static_cast<int>(K / 8);
  nvfp4_weight_kernel<<<blocks_for(experts * N * vec, 256, grid_cap(16)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(w), global_scale, N, experts * N, vec, static_cast<uint32_t*>(q),
      static_cast<uint8_t*>(scales), blocked, static_cast<int>((K / 16 + 3) / 4));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_sf_swizzle(const void* natural, void* blocked_out, int64_t rows, int64_t cols, void* stream) {
  if (!natural || !blocked_out || rows <= 0 || cols <= 0) return kRcBadArg;
  const int64_t padded_rows = (rows + 127) / 128 * 128;
  const int atoms = static_cast<int>((cols + 3) / 4);
  sf_swizzle_kernel<<<blocks_for(padded_rows * atoms * 4, 256, grid_cap(8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(natural), static_cast<uint8_t*>(blocked_out), rows, static_cast<int>(cols),
      padded_rows, atoms);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_gather_packed_rows(const int64_t* ptrs, const int32_t* num_rows, int64_t max_rows, int64_t q_bytes,
                                     int64_t scale_cols, int has_inv, dm_operand q, dm_operand scales_blocked,
                                     dm_operand scale_inv, const int* cond, void* stream) {
  if (!ptrs || !num_rows || !q.base || !scales_blocked.base || q_bytes <= 0 || (q_bytes % 16) != 0 || scale_cols <= 0 ||
      (scale_cols % 4) != 0 || max_rows < 0)
    return kRcBadArg;
  if (has_inv && !scale_inv.base) return kRcBadArg;
  if (max_rows == 0) return kRcOk;
  gather_packed_kernel<<<blocks_for(max_rows * 32, 256, grid_cap(8)), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      ptrs, num_rows, max_rows, static_cast<int>(q_bytes / 16), static_cast<int>(scale_cols), has_inv,
      static_cast<uint8_t*>(q.base), q.offset, static_cast<uint8_t*>(scales_blocked.base), scales_blocked.offset,
      static_cast<uint8_t*>(scale_inv.base), scale_inv.offset, cond);
  return static_cast<int>(cudaGetLastError());
}
