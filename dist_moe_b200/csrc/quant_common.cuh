// Conversion helpers shared by the quantiser kernels and by GEMM epilogues that quantise their output.
#pragma once
#include <cuda_fp8.h>

#include "common.cuh"

namespace dm {

__device__ __forceinline__ float amax_nonfinite(float acc, float v) {
  const float a = fabsf(v);
  return (a != a) ? __int_as_float(0x7f800000) : fmaxf(acc, a);
}

__device__ __forceinline__ uint8_t e8m0_round_up(float s) {
  return static_cast<uint8_t>(__nv_cvt_float_to_e8m0(s, __NV_NOSAT, cudaRoundPosInf));
}

__device__ __forceinline__ float e8m0_recip(uint8_t byte) {
  return byte == 0xFF ? __int_as_float(0x7fc00000) : __int_as_float((254 - static_cast<int>(byte)) << 23);
}

// Scale byte and reciprocal of one MXFP8 block from its amax.
__device__ __forceinline__ uint8_t mxfp8_scale(float amax, float& recip) {
  const float s = amax * (1.0f / 448.0f);
  const uint8_t byte = e8m0_round_up(s);
  recip = (s < __int_as_float(0x7f800000)) ? e8m0_recip(byte) : __int_as_float(0x7fc00000);
  return byte;
}

__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}

__device__ __forceinline__ void unpack8f(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

__device__ __forceinline__ int64_t blocked_offset(int64_t row, int col, int n_col_atoms) {
  const int64_t atom = (row >> 7) * n_col_atoms + (col >> 2);
  return atom * 512 + (row & 31) * 16 + ((row >> 5) & 3) * 4 + (col & 3);
}


// |x| of a bf16 given as its low 15 bits; any pattern above 0x7f80 is a NaN and makes the block non-finite.
__device__ __forceinline__ float amax_from_bf16_bits(uint32_t bits15) {
  return bits15 > 0x7f80u ? __int_as_float(0x7f800000) : __uint_as_float(bits15 << 16);
}

}  // namespace dm
