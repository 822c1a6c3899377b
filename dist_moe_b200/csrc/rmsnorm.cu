// Fused post-expert RMSNorm + score-weighted top-k reduction, forward and backward.
//
//   y[t,k,:]  = cast_norm( g * h3[t,k,:] * rstd[t,k] ),  rstd = rsqrt(mean_d((g*h3)^2) + eps)
//   out[t,:]  = cast_out( sum_k s[t,k] * y[t,k,:] )                      (routes with id < 0 skipped)
// g = gamma + gain_center when an input-scale gamma is given (inference), else 1.
// Same composition as the reference's standalone RMSNorm followed by scale_and_sum
// (dist_moe/kernels/norm/fused_rmsnorm_combine.py:427-466); the backward is its autograd:
//   grad_s[t,k]    = <y[t,k,:], go[t,:]>
//   grad_h3[t,k,:] = rstd * s * (go - y * <go, y> / D)
// HBM bound: forward reads h3 once from DRAM (the second pass of a token's K rows hits L1),
// backward reads h3 and go once and writes grad_h3 in place.
#include "common.cuh"
#include "../../include/dist_moe_b200.h"

namespace dm {

constexpr int kNormMaxK = 32;

__device__ __forceinline__ void up8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Compensated accumulation of the sum of squares (dist_moe/_postprocess.py:44-46 `use_kahan`): every thread keeps a
// running compensation term, and partial sums are merged with an error-free two-sum, so the result is the fp32
// rounding of a nearly exact sum whatever the order.
__device__ __forceinline__ void kahan_add(float& s, float& c, float x) {
  const float y = __fsub_rn(x, c);
  const float t = __fadd_rn(s, y);
  c = __fsub_rn(__fsub_rn(t, s), y);
  s = t;
}
__device__ __forceinline__ void two_sum_merge(float& s, float& c, float s2, float c2) {
  const float t = __fadd_rn(s, s2);
  const float bp = __fsub_rn(t, s);
  const float err = __fadd_rn(__fsub_rn(s, __fsub_rn(t, bp)), __fsub_rn(s2, bp));
  c = __fsub_rn(__fadd_rn(c, c2), err);  // c follows kahan_add's sign: it holds minus the lost low part
  s = t;
}
__device__ __forceinline__ void warp_reduce_sumsq(float& ss, float& cc, int kahan) {
  if (kahan) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      const float s2 = __shfl_xor_sync(0xffffffffu, ss, d), c2 = __shfl_xor_sync(0xffffffffu, cc, d);
      two_sum_merge(ss, cc, s2, c2);
    }
  } else {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, d);
  }
}

template <typename IdT>
__global__ void __launch_bounds__(256) rmsnorm_combine_fwd_kernel(
    const uint4* __restrict__ h3, const void* scores, int scores_bf16, const IdT* __restrict__ ids,
    const uint4* __restrict__ gamma, float gain_center, float eps, int norm_bf16, uint4* __restrict__ out,
    float* __restrict__ rstd_out, int64_t T, int K, int vec, uint8_t* save_base, const int64_t* save_offset,
    const int* save_cond, int save_expect, int kahan) {
  __shared__ float part[kNormMaxK][8];
  __shared__ float partc[kNormMaxK][8];
  __shared__ float rs[kNormMaxK];
  bool save = save_base != nullptr;
  if (save && save_cond != nullptr) save = ((*save_cond != 0) == (save_expect != 0));
  uint4* save_dst = save ? reinterpret_cast<uint4*>(save_base + (save_offset ? *save_offset : 0)) : nullptr;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float inv_d = 1.0f / static_cast<float>(vec * 8);
  for (int64_t t = blockIdx.x; t < T; t += gridDim.x) {
    for (int k = 0; k < K; ++k) {
      const int64_t route = t * K + k;
      float ss = 0.f, cc = 0.f;
      for (int v = threadIdx.x; v < vec; v += 256) {
        const uint4 raw = h3[route * vec + v];
        if (save) save_dst[route * vec + v] = raw;
        float h[8];
        up8(raw, h);
        if (gamma != nullptr) {
          float g[8];
          up8(gamma[v], g);
#pragma unroll
          for (int j = 0; j < 8; ++j) h[j] *= (g[j] + gain_center);
        }
        if (kahan) {
#pragma unroll
          for (int j = 0; j < 8; ++j) kahan_add(ss, cc, __fmul_rn(h[j], h[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += h[j] * h[j];
        }
      }
      warp_reduce_sumsq(ss, cc, kahan);
      if (lane == 0) {
        part[k][warp] = ss;
        partc[k][warp] = cc;
      }
    }
    __syncthreads();
    if (threadIdx.x < K) {
      float ss = 0.f;
      if (kahan) {
        float cc = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) two_sum_merge(ss, cc, part[threadIdx.x][w], partc[threadIdx.x][w]);
        ss = __fsub_rn(ss, cc);
      } else {
#pragma unroll
        for (int w = 0; w < 8; ++w) ss += part[threadIdx.x][w];
      }
      const int64_t route = t * K + threadIdx.x;
      const float r = ids[route] >= 0 ? rsqrtf(ss * inv_d + eps) : 0.f;
      rs[threadIdx.x] = r;
      if (rstd_out != nullptr) rstd_out[route] = r;
    }
    __syncthreads();
    for (int v = threadIdx.x; v < vec; v += 256) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      float g[8];
      if (gamma != nullptr) {
        up8(gamma[v], g);
#pragma unroll
        for (int j = 0; j < 8; ++j) g[j] += gain_center;
      }
      for (int k = 0; k < K; ++k) {
        const int64_t route = t * K + k;
        if (ids[route] < 0) continue;
        const float w = scores_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(scores)[route])
                                    : static_cast<const float*>(scores)[route];
        const float r = rs[k];
        float h[8];
        up8(h3[route * vec + v], h);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          float y = (gamma != nullptr ? h[j] * g[j] : h[j]) * r;
          if (norm_bf16) y = round_bf16(y);
          acc[j] += y * w;
        }
      }
      out[t * vec + v] = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                    pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
    }
    __syncthreads();
  }
}

// One warp per route.  h3 may alias grad_h3 (each lane reads a chunk before it writes it).
template <typename IdT>
__global__ void __launch_bounds__(256) rmsnorm_combine_bwd_kernel(
    const uint4* __restrict__ grad_out, const void* scores, int scores_bf16, const IdT* __restrict__ ids,
    const uint8_t* h3_base, const int64_t* h3_offset, const float* __restrict__ rstd_in, float eps, int norm_bf16,
    uint4* grad_h3, float* __restrict__ grad_scores, int64_t T, int K, int vec, int kahan) {
  const uint4* h3 = reinterpret_cast<const uint4*>(h3_base + (h3_offset ? *h3_offset : 0));
  const int lane = threadIdx.x & 31, wpb = blockDim.x >> 5;
  const float inv_d = 1.0f / static_cast<float>(vec * 8);
  const int64_t routes = T * K;
  for (int64_t route = blockIdx.x * static_cast<int64_t>(wpb) + (threadIdx.x >> 5); route < routes;
       route += static_cast<int64_t>(gridDim.x) * wpb) {
    const int64_t t = route / K;
    const bool valid = ids[route] >= 0;
    if (!valid) {
      for (int v = lane; v < vec; v += 32) grad_h3[route * vec + v] = make_uint4(0, 0, 0, 0);
      if (lane == 0 && grad_scores != nullptr) grad_scores[route] = 0.f;
      continue;
    }
    const float w = scores_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(scores)[route])
                                : static_cast<const float*>(scores)[route];
    float ss = 0.f, cc = 0.f, hg = 0.f;
    for (int v = lane; v < vec; v += 32) {
      float h[8], g[8];
      up8(h3[route * vec + v], h);
      up8(grad_out[t * vec + v], g);
      if (kahan) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          kahan_add(ss, cc, __fmul_rn(h[j], h[j]));
          hg += h[j] * g[j];
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ss += h[j] * h[j];
          hg += h[j] * g[j];
        }
      }
    }
    if (kahan) {
      warp_reduce_sumsq(ss, cc, 1);
      ss = __fsub_rn(ss, cc);
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) hg += __shfl_xor_sync(0xffffffffu, hg, d);
    } else {
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, d);
        hg += __shfl_xor_sync(0xffffffffu, hg, d);
      }
    }
    const float r = rstd_in != nullptr ? rstd_in[route] : rsqrtf(ss * inv_d + eps);
    // <go, y> with y = h * r (the rounding of y to bf16 is ignored inside this inner product)
    const float gy = hg * r;
    float dot_y = 0.f;
    const float c = gy * inv_d;
    for (int v = lane; v < vec; v += 32) {
      float h[8], g[8], o[8];
      up8(h3[route * vec + v], h);
      up8(grad_out[t * vec + v], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float y = h[j] * r;
        if (norm_bf16) y = round_bf16(y);
        dot_y += y * g[j];
        o[j] = r * w * (g[j] - (h[j] * r) * c);
      }
      grad_h3[route * vec + v] = make_uint4(pack_bf16x2(o[0], o[1]), pack_bf16x2(o[2], o[3]),
                                            pack_bf16x2(o[4], o[5]), pack_bf16x2(o[6], o[7]));
    }
    if (grad_scores != nullptr) {
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) dot_y += __shfl_xor_sync(0xffffffffu, dot_y, d);
      if (lane == 0) grad_scores[route] = dot_y;
    }
  }
}

}  // namespace dm

using namespace dm;

extern "C" int dm_rmsnorm_combine_fwd(const void* h3, const void* scores, int scores_are_bf16, const void* ids,
                                      int ids_are_int64, const void* gamma, float gain_center, float eps,
                                      int norm_is_bf16, int use_kahan, void* out, float* rstd_out, int64_t T, int K,
                                      int64_t D, void* save_base, const int64_t* save_offset, const int* save_cond,
                                      int save_expect, void* stream) {
  if (!h3 || !scores || !ids || !out || T <= 0 || K <= 0 || K > kNormMaxK || D <= 0 || (D % 8) != 0) return kRcBadArg;
  const int vec = static_cast<int>(D / 8);
  const int blocks = static_cast<int>(T < grid_cap(8) ? T : grid_cap(8));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ids_are_int64)
    rmsnorm_combine_fwd_kernel<int64_t><<<blocks, 256, 0, st>>>(
        static_cast<const uint4*>(h3), scores, scores_are_bf16, static_cast<const int64_t*>(ids),
        static_cast<const uint4*>(gamma), gain_center, eps, norm_is_bf16, static_cast<uint4*>(out), rstd_out, T, K, vec,
        static_cast<uint8_t*>(save_base), save_offset, save_cond, save_expect, use_kahan ? 1 : 0);
  else
    rmsnorm_combine_fwd_kernel<int32_t><<<blocks, 256, 0, st>>>(
        static_cast<const uint4*>(h3), scores, scores_are_bf16, static_cast<const int32_t*>(ids),
        static_cast<const uint4*>(gamma), gain_center, eps, norm_is_bf16, static_cast<uint4*>(out), rstd_out, T, K, vec,
        static_cast<uint8_t*>(save_base), save_offset, save_cond, save_expect, use_kahan ? 1 : 0);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_rmsnorm_combine_bwd(const void* grad_out, const void* scores, int scores_are_bf16, const void* ids,
                                      int ids_are_int64, const void* h3_base, const int64_t* h3_offset,
                                      const float* rstd, float eps, int norm_is_bf16, int use_kahan, void* grad_h3,
                                      float* grad_scores, int64_t T, int K, int64_t D, void* stream) {
  if (!grad_out || !scores || !ids || !h3_base || !grad_h3 || T <= 0 || K <= 0 || D <= 0 || (D % 8) != 0)
    return kRcBadArg;
  const int vec = static_cast<int>(D / 8);
  int64_t blocks = (T * K + 7) / 8;
  if (blocks > grid_cap(16)) blocks = grid_cap(16);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ids_are_int64)
    rmsnorm_combine_bwd_kernel<int64_t><<<static_cast<int>(blocks), 256, 0, st>>>(
        static_cast<const uint4*>(grad_out), scores, scores_are_bf16, static_cast<const int64_t*>(ids),
        static_cast<const uint8_t*>(h3_base), h3_offset, rstd, eps, norm_is_bf16, static_cast<uint4*>(grad_h3),
        grad_scores, T, K, vec, use_kahan ? 1 : 0);
  else
    rmsnorm_combine_bwd_kernel<int32_t><<<static_cast<int>(blocks), 256, 0, st>>>(
        static_cast<const uint4*>(grad_out), scores, scores_are_bf16, static_cast<const int32_t*>(ids),
        static_cast<const uint8_t*>(h3_base), h3_offset, rstd, eps, norm_is_bf16, static_cast<uint4*>(grad_h3),
        grad_scores, T, K, vec, use_kahan ? 1 : 0);
  return static_cast<int>(cudaGetLastError());
}
