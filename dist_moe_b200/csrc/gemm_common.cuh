// Helpers shared by the grouped GEMM kernels: epilogue staging tile, L2 reductions and the
// host-side tensor-map encoding (through the driver entry point, no link-time libcuda).
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "../../include/dist_moe_b200.h"

namespace dm {

constexpr uint32_t kStagingBytes = 32 * 128;   // per epilogue warp: 32 rows x 128 bytes
constexpr uint32_t kStaging64Bytes = 32 * 64;  // per epilogue warp: 32 rows x 64 bytes

// Staging tile of one epilogue warp: row r is 128 bytes, its 16-byte chunk j sits at j ^ (r & 7).
__device__ __forceinline__ void stage_put(uint8_t* stg, int row, int chunk, uint4 v) {
  reinterpret_cast<uint4*>(stg + row * 128)[chunk ^ (row & 7)] = v;
}
__device__ __forceinline__ uint4 stage_get(const uint8_t* stg, int row, int chunk) {
  return reinterpret_cast<const uint4*>(stg + row * 128)[chunk ^ (row & 7)];
}
// 64-byte variant: row r is 64 bytes, its 16-byte chunk j sits at j ^ ((r >> 1) & 3).
__device__ __forceinline__ void stage64_put(uint8_t* stg, int row, int chunk, uint4 v) {
  reinterpret_cast<uint4*>(stg + row * 64)[chunk ^ ((row >> 1) & 3)] = v;
}
__device__ __forceinline__ uint4 stage64_get(const uint8_t* stg, int row, int chunk) {
  return reinterpret_cast<const uint4*>(stg + row * 64)[chunk ^ ((row >> 1) & 3)];
}
__device__ __forceinline__ uint4 pack8_bf16(const uint32_t* r) {
  return make_uint4(pack_bf16x2(__uint_as_float(r[0]), __uint_as_float(r[1])),
                    pack_bf16x2(__uint_as_float(r[2]), __uint_as_float(r[3])),
                    pack_bf16x2(__uint_as_float(r[4]), __uint_as_float(r[5])),
                    pack_bf16x2(__uint_as_float(r[6]), __uint_as_float(r[7])));
}

// Lean forms for the single-thread issue loops: barrier given by its shared-memory address, shared-memory
// descriptors given by their lower word (address >> 4 | LBO >> 4 << 16) and a constant upper word.
__device__ __forceinline__ uint32_t mbar_poll(uint32_t bar_addr, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok) : "r"(bar_addr), "r"(parity) : "memory");
  return ok;
}
// A bare polling loop (a million polls, tens of milliseconds), then the timed wait that can give up.
__device__ __forceinline__ bool mbar_wait_lean(uint32_t bar_addr, uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (uint32_t i = 0; i < (1u << 20); ++i)
    if (mbar_poll(bar_addr, parity)) return true;
  return mbar_wait(bar, parity, abort_flag);
}
__device__ __forceinline__ void umma_bf16_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tcgen05_commit_addr(uint32_t bar_addr) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_addr) : "memory");
}

// Bulk tensor store and reduce-add of one staged box (shared memory -> global), issued by one thread.  The
// staged bytes must have been made visible to the async proxy (fence_proxy_async_smem by every writer, then
// a barrier) and stay untouched until bulk_wait_read has returned.
__device__ __forceinline__ void tma_store_3d(const void* tmap, const void* smem_src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const void* tmap, const void* smem_src, int c0, int c1, int c2) {
  asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(tmap)),
               "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------------------
// Host side: tensor-map encoding through the driver entry point (no link-time
// dependency on libcuda) and launch.
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static inline EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// bf16 matrix [rows][cols], cols contiguous; box = box_rows x 64 columns.
static inline int encode_2d(CUtensorMap* tm, const void* base, int64_t rows, int64_t cols, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return kRcNoDriver;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  cuuint32_t box[2] = {64, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kRcOk : 1000 + static_cast<int>(r);
}

// Arena view: element (c0, line, row) lives at base + 2*c0 + 128*line + pitch*row.
// `line` spans the whole allocation, so an operand at byte offset o is reached
// with line = o/128 + column/64; rows may run `guard` rows past the operand.
static inline int encode_arena(CUtensorMap* tm, const dm_operand& op, int64_t pitch_bytes, int64_t rows, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return kRcNoDriver;
  const int64_t lines = op.bytes / 128;
  if (lines <= 0 || (pitch_bytes % 128) != 0 || (reinterpret_cast<uintptr_t>(op.base) % 128) != 0) return kRcBadArg;
  cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(lines), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[2] = {128, static_cast<cuuint64_t>(pitch_bytes)};
  cuuint32_t box[3] = {64, 1, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, op.base, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kRcOk : 1000 + static_cast<int>(r);
}

// Weight-gradient destination [groups][rows][cols] (bf16 or fp32), boxes of 32 rows x 64 bytes in the
// 64-byte swizzle: the layout of an epilogue warp's staging tile.
static inline int encode_out_3d(CUtensorMap* tm, void* base, int64_t groups, int64_t rows, int64_t cols, bool fp32) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return kRcNoDriver;
  const cuuint64_t esz = fp32 ? 4 : 2;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(groups)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(cols) * esz, static_cast<cuuint64_t>(cols) * rows * esz};
  // boxes of 16 rows x 128 bytes: a reduce-add or store then moves whole 128-byte lines of dW
  cuuint32_t box[3] = {static_cast<cuuint32_t>(128 / esz), 16, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kRcOk : 1000 + static_cast<int>(r);
}

// Byte-typed variants for quantised operands: rows of `row_bytes`, boxes of 128 bytes x box_rows.
static inline int encode_2d_u8(CUtensorMap* tm, const void* base, int64_t rows, int64_t row_bytes, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return kRcNoDriver;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(row_bytes), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(row_bytes)};
  cuuint32_t box[2] = {128, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kRcOk : 1000 + static_cast<int>(r);
}

static inline int encode_arena_u8(CUtensorMap* tm, const dm_operand& op, int64_t pitch_bytes, int64_t rows,
                                  int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return kRcNoDriver;
  const int64_t lines = op.bytes / 128;
  if (lines <= 0 || (pitch_bytes % 128) != 0 || (reinterpret_cast<uintptr_t>(op.base) % 128) != 0) return kRcBadArg;
  cuuint64_t dims[3] = {128, static_cast<cuuint64_t>(lines), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[2] = {128, static_cast<cuuint64_t>(pitch_bytes)};
  cuuint32_t box[3] = {128, 1, static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, op.base, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? kRcOk : 1000 + static_cast<int>(r);
}

}  // namespace dm
