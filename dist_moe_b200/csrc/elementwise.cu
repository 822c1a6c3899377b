// HBM-bound row kernels: SwiGLU forward/backward, weighted top-k reduction and
// its backward.  All of them move 16-byte vectors (8 bf16), keep fp32 math, and
// read their row counts from device memory so that no host read is needed.
#include "common.cuh"
#include "../../include/dist_moe_b200.h"

namespace dm {

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]),
                    pack_bf16x2(f[6], f[7]));
}

// ---------------------------------------------------------------------------
// SwiGLU forward: h2[r, f] = act(h1[r, f], h1[r, F + f])
// ---------------------------------------------------------------------------
template <bool kClip>
__global__ void __launch_bounds__(256) swiglu_fwd_kernel(const uint8_t* h1_base, const int64_t* h1_offset,
                                                         uint8_t* h2_base, const int64_t* h2_offset,
                                                         const int32_t* num_rows, int64_t max_rows, int vec_per_row,
                                                         ActParams act, float* clip_stats, float clip_limit,
                                                         const int* cond) {
  if (cond != nullptr && *cond == 0) return;
  int64_t rows = *num_rows;
  if (rows > max_rows) rows = max_rows;
  const uint4* h1 = reinterpret_cast<const uint4*>(h1_base + (h1_offset ? *h1_offset : 0));
  uint4* h2 = reinterpret_cast<uint4*>(h2_base + (h2_offset ? *h2_offset : 0));
  const int64_t total = rows * vec_per_row;
  float n_gate = 0.f, n_up = 0.f, n_all = 0.f;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int v = static_cast<int>(i - r * vec_per_row);
    const uint4 g4 = h1[r * 2 * vec_per_row + v];
    const uint4 u4 = h1[r * 2 * vec_per_row + vec_per_row + v];
    float g[8], u[8], z[8];
    unpack8(g4, g);
    unpack8(u4, u);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      z[j] = swiglu_f32(g[j], u[j], act);
      if (kClip) {
        n_gate += g[j] > clip_limit ? 1.f : 0.f;
        n_up += fabsf(u[j]) > clip_limit ? 1.f : 0.f;
      }
    }
    if (kClip) n_all += 8.f;
    h2[r * vec_per_row + v] = pack8(z);
  }
  if (kClip) {
    __shared__ float red[3][8];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      n_gate += __shfl_xor_sync(0xffffffffu, n_gate, d);
      n_up += __shfl_xor_sync(0xffffffffu, n_up, d);
      n_all += __shfl_xor_sync(0xffffffffu, n_all, d);
    }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) {
      red[0][warp] = n_gate;
      red[1][warp] = n_up;
      red[2][warp] = n_all;
    }
    __syncthreads();
    if (threadIdx.x < 3) {
      float s = 0.f;
      for (int w = 0; w < 8; ++w) s += red[threadIdx.x][w];
      if (s != 0.f) atomicAdd(clip_stats + threadIdx.x, s);
    }
  }
}

// ---------------------------------------------------------------------------
// SwiGLU backward: grad_h1[r, :F] = d/d gate, grad_h1[r, F:] = d/d up
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) swiglu_bwd_kernel(const uint8_t* h1_base, const int64_t* h1_offset,
                                                         const uint8_t* gh2_base, const int64_t* gh2_offset,
                                                         uint8_t* gh1_base, const int64_t* gh1_offset,
                                                         const int32_t* num_rows, int64_t max_rows, int vec_per_row,
                                                         ActParams act) {
  int64_t rows = *num_rows;
  if (rows > max_rows) rows = max_rows;
  const uint4* h1 = reinterpret_cast<const uint4*>(h1_base + (h1_offset ? *h1_offset : 0));
  const uint4* gh2 = reinterpret_cast<const uint4*>(gh2_base + (gh2_offset ? *gh2_offset : 0));
  uint4* gh1 = reinterpret_cast<uint4*>(gh1_base + (gh1_offset ? *gh1_offset : 0));
  const int64_t total = rows * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t r = i / vec_per_row;
    const int v = static_cast<int>(i - r * vec_per_row);
    float x[8], y[8], dz[8], dx[8], dy[8];
    unpack8(h1[r * 2 * vec_per_row + v], x);
    unpack8(h1[r * 2 * vec_per_row + vec_per_row + v], y);
    unpack8(gh2[r * vec_per_row + v], dz);
#pragma unroll
    for (int j = 0; j < 8; ++j) swiglu_bwd_f32(x[j], y[j], dz[j], act, dx[j], dy[j]);
    gh1[r * 2 * vec_per_row + v] = pack8(dx);
    gh1[r * 2 * vec_per_row + vec_per_row + v] = pack8(dy);
  }
}

// ---------------------------------------------------------------------------
// out[t, :] = bf16( sum_k w[t,k] * h3[t,k,:] )
// ---------------------------------------------------------------------------
template <typename IdT>
__global__ void __launch_bounds__(256) scale_and_sum_kernel(const uint4* __restrict__ h3, const void* scores,
                                                            int scores_are_bf16, const IdT* __restrict__ ids,
                                                            uint4* __restrict__ out, int64_t T, int K, int vec_per_row,
                                                            uint8_t* save_base, const int64_t* save_offset,
                                                            const int* save_cond, int save_expect) {
  bool save = save_base != nullptr;
  if (save && save_cond != nullptr) save = ((*save_cond != 0) == (save_expect != 0));
  uint4* save_dst = save ? reinterpret_cast<uint4*>(save_base + (save_offset ? *save_offset : 0)) : nullptr;
  const int64_t total = T * vec_per_row;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int64_t t = i / vec_per_row;
    const int v = static_cast<int>(i - t * vec_per_row);
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // Four routes are fetched before any is used (independent 16-byte loads in flight); they are then added in
    // ascending k, the order of the one-at-a-time loop, so the fp32 sums are unchanged.
    for (int k0 = 0; k0 < K; k0 += 4) {
      uint4 raw[4];
      float w[4];
      bool ok[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        ok[q] = false;
        w[q] = 1.0f;
        if (k0 + q < K) {
          const int64_t route = t * K + k0 + q;
          raw[q] = h3[route * vec_per_row + v];
          ok[q] = ids[route] >= 0;
          if (scores != nullptr)
            w[q] = scores_are_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(scores)[route])
                                   : static_cast<const float*>(scores)[route];
        }
      }
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        if (k0 + q < K) {
          if (save) save_dst[(t * K + k0 + q) * vec_per_row + v] = raw[q];
          if (ok[q]) {
            float h[8];
            unpack8(raw[q], h);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += h[j] * w[q];
          }
        }
      }
    }
    out[i] = pack8(acc);
  }
}

// ---------------------------------------------------------------------------
// grad_h3[t,k,:] = bf16(w[t,k] * grad_out[t,:]);  grad_w[t,k] = <h3[t,k,:], grad_out[t,:]>
// One warp per route.  h3 may alias grad_h3: every lane reads its h3 vector
// before it writes the same position.
// ---------------------------------------------------------------------------
template <typename IdT>
__global__ void __launch_bounds__(256) broadcast_and_scale_kernel(const uint4* __restrict__ grad_out,
                                                                  const void* scores, int scores_are_bf16,
                                                                  const IdT* __restrict__ ids, const uint8_t* h3_base,
                                                                  const int64_t* h3_offset, const uint8_t* h3_alt,
                                                                  const int* use_alt, uint4* grad_h3,
                                                                  float* grad_scores, int64_t T, int K,
                                                                  int vec_per_row) {
  const uint4* h3 = h3_base ? reinterpret_cast<const uint4*>(h3_base + (h3_offset ? *h3_offset : 0)) : nullptr;
  if (h3_alt != nullptr && use_alt != nullptr && *use_alt != 0) h3 = reinterpret_cast<const uint4*>(h3_alt);
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int64_t routes = T * K;
  for (int64_t route = blockIdx.x * static_cast<int64_t>(warps_per_block) + (threadIdx.x >> 5); route < routes;
       route += static_cast<int64_t>(gridDim.x) * warps_per_block) {
    const int64_t t = route / K;
    const bool valid = ids[route] >= 0;
    float w = 0.0f;
    if (valid)
      w = scores_are_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(scores)[route])
                          : static_cast<const float*>(scores)[route];
    float dot = 0.0f;
    for (int v = lane; v < vec_per_row; v += 32) {
      float g[8], o[8];
      unpack8(grad_out[t * vec_per_row + v], g);
      if (h3 != nullptr && grad_scores != nullptr && valid) {
        float h[8];
        unpack8(h3[route * vec_per_row + v], h);
#pragma unroll
        for (int j = 0; j < 8; ++j) dot += h[j] * g[j];
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = g[j] * w;
      grad_h3[route * vec_per_row + v] = pack8(o);
    }
    if (grad_scores != nullptr) {
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, d);
      if (lane == 0) grad_scores[route] = valid ? dot : 0.0f;
    }
  }
}

inline int grid_for(int64_t work_items, int threads, int max_blocks) {
  int64_t blocks = (work_items + threads - 1) / threads;
  if (blocks > max_blocks) blocks = max_blocks;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace dm

using namespace dm;

extern "C" int dm_swiglu_fwd(const void* h1_base, const int64_t* h1_offset, void* h2_base, const int64_t* h2_offset,
                             const int32_t* num_rows, int64_t max_rows, int64_t F, int clamped, float alpha,
                             float limit, float* clip_stats, float clip_limit, const int* cond, void* stream) {
  if (!h1_base || !h2_base || !num_rows || F <= 0 || (F % 8) != 0 || max_rows < 0) return kRcBadArg;
  if (max_rows == 0) return kRcOk;
  const int vec = static_cast<int>(F / 8);
  const int blocks = grid_for(max_rows * vec, 256, grid_cap(8));
  ActParams act{clamped, alpha, limit};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (clip_stats)
    swiglu_fwd_kernel<true><<<blocks, 256, 0, st>>>(static_cast<const uint8_t*>(h1_base), h1_offset,
                                                    static_cast<uint8_t*>(h2_base), h2_offset, num_rows, max_rows, vec,
                                                    act, clip_stats, clip_limit, cond);
  else
    swiglu_fwd_kernel<false><<<blocks, 256, 0, st>>>(static_cast<const uint8_t*>(h1_base), h1_offset,
                                                     static_cast<uint8_t*>(h2_base), h2_offset, num_rows, max_rows,
                                                     vec, act, nullptr, 0.f, cond);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_swiglu_bwd(const void* h1_base, const int64_t* h1_offset, const void* grad_h2_base,
                             const int64_t* grad_h2_offset, void* grad_h1_base, const int64_t* grad_h1_offset,
                             const int32_t* num_rows, int64_t max_rows, int64_t F, int clamped, float alpha,
                             float limit, void* stream) {
  if (!h1_base || !grad_h2_base || !grad_h1_base || !num_rows || F <= 0 || (F % 8) != 0 || max_rows < 0)
    return kRcBadArg;
  if (max_rows == 0) return kRcOk;
  const int vec = static_cast<int>(F / 8);
  const int blocks = grid_for(max_rows * vec, 256, grid_cap(8));
  ActParams act{clamped, alpha, limit};
  swiglu_bwd_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(h1_base), h1_offset, static_cast<const uint8_t*>(grad_h2_base), grad_h2_offset,
      static_cast<uint8_t*>(grad_h1_base), grad_h1_offset, num_rows, max_rows, vec, act);
  return static_cast<int>(cudaGetLastError());
}

// Rows of a [T, K, D] route tensor whose expert id is negative are set to zero (one warp per route), so that Python
// callbacks never see the stale bytes a dropped route leaves in the communication buffer
// (dist_moe/kernels/triton/conditional_copy.py:215-235 `zero_out_padded_rows_`).
template <typename IdT>
__global__ void zero_padded_rows_kernel(uint4* __restrict__ rows, const IdT* __restrict__ ids, int64_t routes, int vec) {
  const int lane = threadIdx.x & 31;
  const int64_t warps = (static_cast<int64_t>(gridDim.x) * blockDim.x) >> 5;
  for (int64_t r = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5; r < routes; r += warps) {
    if (static_cast<int64_t>(ids[r]) >= 0) continue;
    uint4* row = rows + r * vec;
    for (int v = lane; v < vec; v += 32) row[v] = make_uint4(0, 0, 0, 0);
  }
}

extern "C" int dm_zero_padded_rows(void* routes_TKD, const void* ids, int ids_are_int64, int64_t T, int K, int64_t D,
                                   void* stream) {
  if (!routes_TKD || !ids || T <= 0 || K <= 0 || D <= 0 || (D % 8) != 0) return kRcBadArg;
  const int64_t routes = T * K;
  const int blocks = grid_for(routes * 32, 256, grid_cap(16));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ids_are_int64)
    zero_padded_rows_kernel<int64_t><<<blocks, 256, 0, st>>>(static_cast<uint4*>(routes_TKD),
                                                             static_cast<const int64_t*>(ids), routes, static_cast<int>(D / 8));
  else
    zero_padded_rows_kernel<int32_t><<<blocks, 256, 0, st>>>(static_cast<uint4*>(routes_TKD),
                                                             static_cast<const int32_t*>(ids), routes, static_cast<int>(D / 8));
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_scale_and_sum(const void* h3, const void* scores, int scores_are_bf16, const void* ids,
                                int ids_are_int64, void* out, int64_t T, int K, int64_t D, void* save_base,
                                const int64_t* save_offset, const int* save_cond, int save_expect, void* stream) {
  if (!h3 || !ids || !out || T <= 0 || K <= 0 || D <= 0 || (D % 8) != 0) return kRcBadArg;
  const int vec = static_cast<int>(D / 8);
  const int blocks = grid_for(T * vec, 256, grid_cap(16));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ids_are_int64)
    scale_and_sum_kernel<int64_t><<<blocks, 256, 0, st>>>(static_cast<const uint4*>(h3), scores, scores_are_bf16,
                                                          static_cast<const int64_t*>(ids), static_cast<uint4*>(out),
                                                          T, K, vec, static_cast<uint8_t*>(save_base), save_offset,
                                                          save_cond, save_expect);
  else
    scale_and_sum_kernel<int32_t><<<blocks, 256, 0, st>>>(static_cast<const uint4*>(h3), scores, scores_are_bf16,
                                                          static_cast<const int32_t*>(ids), static_cast<uint4*>(out),
                                                          T, K, vec, static_cast<uint8_t*>(save_base), save_offset,
                                                          save_cond, save_expect);
  return static_cast<int>(cudaGetLastError());
}

static int broadcast_and_scale_launch(const void* grad_out, const void* scores, int scores_are_bf16, const void* ids,
                                      int ids_are_int64, const void* h3_base, const int64_t* h3_offset,
                                      const void* h3_alt, const int* use_alt, void* grad_h3, float* grad_scores,
                                      int64_t T, int K, int64_t D, void* stream) {
  if (!grad_out || !scores || !ids || !grad_h3 || T <= 0 || K <= 0 || D <= 0 || (D % 8) != 0) return kRcBadArg;
  const int vec = static_cast<int>(D / 8);
  const int blocks = grid_for(T * K * 32, 256, grid_cap(16));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ids_are_int64)
    broadcast_and_scale_kernel<int64_t><<<blocks, 256, 0, st>>>(
        static_cast<const uint4*>(grad_out), scores, scores_are_bf16, static_cast<const int64_t*>(ids),
        static_cast<const uint8_t*>(h3_base), h3_offset, static_cast<const uint8_t*>(h3_alt), use_alt,
        static_cast<uint4*>(grad_h3), grad_scores, T, K, vec);
  else
    broadcast_and_scale_kernel<int32_t><<<blocks, 256, 0, st>>>(
        static_cast<const uint4*>(grad_out), scores, scores_are_bf16, static_cast<const int32_t*>(ids),
        static_cast<const uint8_t*>(h3_base), h3_offset, static_cast<const uint8_t*>(h3_alt), use_alt,
        static_cast<uint4*>(grad_h3), grad_scores, T, K, vec);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_broadcast_and_scale(const void* grad_out, const void* scores, int scores_are_bf16, const void* ids,
                                      int ids_are_int64, const void* h3_base, const int64_t* h3_offset, void* grad_h3,
                                      float* grad_scores, int64_t T, int K, int64_t D, void* stream) {
  return broadcast_and_scale_launch(grad_out, scores, scores_are_bf16, ids, ids_are_int64, h3_base, h3_offset, nullptr,
                                    nullptr, grad_h3, grad_scores, T, K, D, stream);
}

// The same with the expert outputs read from one of two places chosen on the device: `h3_alt` when *use_alt != 0
// (they were recomputed into the communication buffer), else h3_base + *h3_offset (they were saved in the slot).
// Saves the copy of the saved outputs back into the communication buffer.
extern "C" int dm_broadcast_and_scale_select(const void* grad_out, const void* scores, int scores_are_bf16,
                                             const void* ids, int ids_are_int64, const void* h3_base,
                                             const int64_t* h3_offset, const void* h3_alt, const int* use_alt,
                                             void* grad_h3, float* grad_scores, int64_t T, int K, int64_t D,
                                             void* stream) {
  if (!h3_base || !h3_alt || !use_alt) return kRcBadArg;
  return broadcast_and_scale_launch(grad_out, scores, scores_are_bf16, ids, ids_are_int64, h3_base, h3_offset, h3_alt,
                                    use_alt, grad_h3, grad_scores, T, K, D, stream);
}
