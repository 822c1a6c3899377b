// Publication, expert-parallel barrier, routing metadata and row gather.
//
// Routing order contract (must equal the reference's general path): output rows
// are sorted by (local expert ascending, source rank ascending, token ascending).
// The three kernels below reach it without any sort:
//   route_count : one CTA per (source rank, 256-token chunk) builds, per local
//                 expert, a 32-bit lane mask per warp in shared memory and stores
//                 the chunk's per-expert totals; a global histogram over all E
//                 experts is accumulated with integer atomics (order free).
//   route_scan  : one CTA turns the chunk totals into exclusive offsets inside
//                 every expert segment (warp-shuffle scans), pads the segments,
//                 checks capacity and writes counts / per-rank totals / offsets.
//   route_fill  : same decomposition as route_count; a row's slot is
//                 segment offset + popc(lower warps) + popc(lower lanes).
#include "common.cuh"
#include "../../include/dist_moe_b200.h"

namespace dm {

constexpr int kChunkTokens = 256;  // tokens per CTA in route_count / route_fill
constexpr int kChunkWarps = kChunkTokens / 32;
constexpr int kMaxExpertsSmem = 2048;

// ---------------------------------------------------------------------------
// Publication
// ---------------------------------------------------------------------------
template <typename IdT>
__global__ void publish_kernel(const uint4* __restrict__ x, const IdT* __restrict__ ids, uint4* __restrict__ dispatch,
                               uint8_t* __restrict__ routing, int64_t n_vec, int64_t n_ids, int T, int E, int validate,
                               int* status) {
  const int64_t tid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
  if (tid == 0) *reinterpret_cast<int32_t*>(routing) = T;
  int16_t* ids_out = reinterpret_cast<int16_t*>(routing + DM_ROUTING_HEADER_BYTES);
  for (int64_t i = tid; i < n_ids; i += stride) {
    const int64_t v = static_cast<int64_t>(ids[i]);
    if (validate && (v < -1 || v >= E)) set_status(status, kInvalidExpertId, static_cast<int>(i), static_cast<int>(v));
    ids_out[i] = static_cast<int16_t>(v);
  }
  if (x != nullptr) {
    for (int64_t i = tid; i < n_vec; i += stride) dispatch[i] = x[i];
  }
}

// ---------------------------------------------------------------------------
// Barrier over per-rank signal pads: pad[channel][peer].
// Thread p (< ep, p != rank) sets slot `rank` of peer p's pad from 0 to 1 and
// then takes slot `p` of the own pad from 1 back to 0.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cas_release_sys(uint32_t* addr, uint32_t cmp, uint32_t val) {
  uint32_t old;
  asm volatile("atom.release.sys.global.cas.b32 %0, [%1], %2, %3;" : "=r"(old) : "l"(addr), "r"(cmp), "r"(val) : "memory");
  return old;
}
__device__ __forceinline__ uint32_t cas_acquire_sys(uint32_t* addr, uint32_t cmp, uint32_t val) {
  uint32_t old;
  asm volatile("atom.acquire.sys.global.cas.b32 %0, [%1], %2, %3;" : "=r"(old) : "l"(addr), "r"(cmp), "r"(val) : "memory");
  return old;
}

__global__ void barrier_kernel(const uint64_t* __restrict__ pads, int rank, int ep, int channel, const int* cond,
                               uint64_t timeout_ns, int* status) {
  if (cond != nullptr && *cond == 0) return;
  const int p = threadIdx.x;
  if (p >= ep || p == rank) return;
  __threadfence_system();
  uint32_t* peer = reinterpret_cast<uint32_t*>(pads[p]) + static_cast<int64_t>(channel) * ep + rank;
  uint32_t* own = reinterpret_cast<uint32_t*>(pads[rank]) + static_cast<int64_t>(channel) * ep + p;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (cas_release_sys(peer, 0u, 1u) != 0u) {
    if ((++spins & 0x3f) == 0 && globaltimer_ns() - t0 > timeout_ns) {
      set_status(status, kBarrierTimeout, p, channel, 0);
      return;
    }
  }
  while (cas_acquire_sys(own, 1u, 0u) != 1u) {
    if ((++spins & 0x3f) == 0 && globaltimer_ns() - t0 > timeout_ns) {
      set_status(status, kBarrierTimeout, p, channel, 1);
      return;
    }
  }
}

// ---------------------------------------------------------------------------
// Routing
// ---------------------------------------------------------------------------
struct RouteParams {
  const uint64_t* routing_ptrs;
  const uint64_t* dispatch_ptrs;
  const uint64_t* combine_ptrs;
  int rank, ep, T, K, E, e_local, chunks;
  int64_t gather_stride, bwd_stride, scatter_stride;
  int m_mult;
  int64_t capacity_rows, ptrs_size;
  int32_t* counts;
  int32_t* real_counts;  // optional: rows per expert before padding
  int32_t* per_rank;
  int32_t* expert_offsets;
  int64_t* fwd;
  int64_t* bwd;
  int64_t* sct;
  int32_t* chunk_counts;   // [ep*chunks][e_local]
  int32_t* chunk_offsets;  // [ep*chunks][e_local], exclusive inside the expert segment
  int32_t* hist;           // [E]
  int* status;
};

// Build the per-warp lane masks of this chunk: mask[w][el] bit l = token (w*32+l)
// routes to local expert el.  Returns through shared memory.
__device__ __forceinline__ void build_masks(const RouteParams& p, int s, int c, uint32_t* mask, int32_t* hist_s,
                                            bool do_hist) {
  const int tok = c * kChunkTokens + threadIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < kChunkWarps * p.e_local; i += blockDim.x) mask[i] = 0u;
  if (do_hist)
    for (int i = threadIdx.x; i < p.E; i += blockDim.x) hist_s[i] = 0;
  __syncthreads();
  if (tok < p.T) {
    const int16_t* ids = reinterpret_cast<const int16_t*>(p.routing_ptrs[s] + DM_ROUTING_HEADER_BYTES) +
                         static_cast<int64_t>(tok) * p.K;
    const int first = p.rank * p.e_local;
    for (int k = 0; k < p.K; ++k) {
      const int e = ids[k];
      if (e < 0 || e >= p.E) continue;
      if (do_hist) atomicAdd(&hist_s[e], 1);
      const int el = e - first;
      if (el >= 0 && el < p.e_local) atomicOr(&mask[warp * p.e_local + el], 1u << lane);
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kChunkTokens) route_count_kernel(RouteParams p) {
  extern __shared__ uint32_t smem_u[];
  uint32_t* mask = smem_u;
  int32_t* hist_s = reinterpret_cast<int32_t*>(smem_u + kChunkWarps * p.e_local);
  const int s = blockIdx.y, c = blockIdx.x;
  if (c == 0 && threadIdx.x == 0) {
    const int peer_t = *reinterpret_cast<const int32_t*>(p.routing_ptrs[s]);
    if (peer_t != p.T) set_status(p.status, kTokenCountMismatch, s, peer_t, p.T);
  }
  build_masks(p, s, c, mask, hist_s, true);
  int32_t* out = p.chunk_counts + (static_cast<int64_t>(s) * p.chunks + c) * p.e_local;
  for (int el = threadIdx.x; el < p.e_local; el += blockDim.x) {
    int n = 0;
#pragma unroll
    for (int w = 0; w < kChunkWarps; ++w) n += __popc(mask[w * p.e_local + el]);
    out[el] = n;
  }
  for (int e = threadIdx.x; e < p.E; e += blockDim.x) {
    const int n = hist_s[e];
    if (n) atomicAdd(&p.hist[e], n);
  }
}

__device__ __forceinline__ int pad_rows(int n, int m) { return m > 0 ? (n + m - 1) / m * m : n; }

__global__ void __launch_bounds__(1024) route_scan_kernel(RouteParams p) {
  extern __shared__ int32_t smem_i[];
  int32_t* total = smem_i;              // [e_local] real rows
  int32_t* base = smem_i + p.e_local;   // [e_local + 1] padded exclusive prefix
  __shared__ int overflow;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int n = p.ep * p.chunks;
  for (int el = warp; el < p.e_local; el += nwarps) {
    int running = 0;
    for (int i0 = 0; i0 < n; i0 += 32) {
      const int i = i0 + lane;
      const int v = i < n ? p.chunk_counts[static_cast<int64_t>(i) * p.e_local + el] : 0;
      int incl = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += t;
      }
      if (i < n) p.chunk_offsets[static_cast<int64_t>(i) * p.e_local + el] = running + incl - v;
      running += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) total[el] = running;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int64_t acc = 0;
    for (int el = 0; el < p.e_local; ++el) {
      base[el] = static_cast<int32_t>(acc);
      acc += pad_rows(total[el], p.m_mult);
    }
    base[p.e_local] = static_cast<int32_t>(acc);
    overflow = (acc > p.capacity_rows || acc > p.ptrs_size) ? 1 : 0;
    if (overflow) set_status(p.status, kCapacityExceeded, static_cast<int>(acc), static_cast<int>(p.capacity_rows));
    // ranks that disagree on T cannot be routed: the call becomes a no-op (zero rows), like an overflow
    if (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) == kTokenCountMismatch) overflow = 1;
  }
  __syncthreads();
  const bool bad = overflow != 0;
  for (int el = threadIdx.x; el <= p.e_local; el += blockDim.x) {
    p.expert_offsets[el] = bad ? 0 : base[el];
    if (el < p.e_local) p.counts[el] = bad ? 0 : pad_rows(total[el], p.m_mult);
    if (el < p.e_local && p.real_counts != nullptr) p.real_counts[el] = bad ? 0 : total[el];
  }
  for (int q = threadIdx.x; q < p.ep; q += blockDim.x) {
    int acc = 0;
    for (int el = 0; el < p.e_local; ++el) acc += pad_rows(p.hist[q * p.e_local + el], p.m_mult);
    p.per_rank[q] = acc;
  }
  if (p.m_mult > 0 && !bad) {
    // Padding rows of every expert segment hold a null pointer.
    for (int el = warp; el < p.e_local; el += nwarps) {
      const int lo = base[el] + total[el], hi = base[el + 1];
      for (int r = lo + lane; r < hi; r += 32) {
        p.fwd[r] = 0;
        p.sct[r] = 0;
        if (p.bwd != nullptr) p.bwd[r] = 0;
      }
    }
  }
}

__global__ void __launch_bounds__(kChunkTokens) route_fill_kernel(RouteParams p) {
  extern __shared__ uint32_t smem_u[];
  uint32_t* mask = smem_u;
  const int s = blockIdx.y, c = blockIdx.x;
  if (p.expert_offsets[p.e_local] == 0) return;  // nothing routed here, or capacity exceeded
  build_masks(p, s, c, mask, nullptr, false);
  const int tok = c * kChunkTokens + threadIdx.x;
  if (tok >= p.T) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int16_t* ids = reinterpret_cast<const int16_t*>(p.routing_ptrs[s] + DM_ROUTING_HEADER_BYTES) +
                       static_cast<int64_t>(tok) * p.K;
  const int32_t* seg = p.chunk_offsets + (static_cast<int64_t>(s) * p.chunks + c) * p.e_local;
  const int first = p.rank * p.e_local;
  const uint64_t dbase = p.dispatch_ptrs[s], cbase = p.combine_ptrs[s];
  for (int k = 0; k < p.K; ++k) {
    const int el = static_cast<int>(ids[k]) - first;
    if (ids[k] < 0 || ids[k] >= p.E || el < 0 || el >= p.e_local) continue;
    int pos = p.expert_offsets[el] + seg[el];
    for (int w = 0; w < warp; ++w) pos += __popc(mask[w * p.e_local + el]);
    pos += __popc(mask[warp * p.e_local + el] & ((1u << lane) - 1u));
    const int64_t route = static_cast<int64_t>(tok) * p.K + k;
    p.fwd[pos] = static_cast<int64_t>(dbase + static_cast<uint64_t>(tok) * p.gather_stride);
    p.sct[pos] = static_cast<int64_t>(cbase + static_cast<uint64_t>(route) * p.scatter_stride);
    if (p.bwd != nullptr) p.bwd[pos] = static_cast<int64_t>(dbase + static_cast<uint64_t>(route) * p.bwd_stride);
  }
}

// ---------------------------------------------------------------------------
// Decode regime: the whole routing step in one CTA and one launch (the reference's single-launch path,
// dist_moe/_routing_metadata.py:265-300 and kernels/triton/dist_dispatch_routing_kernel.py:120-260, which
// orders rows inside an expert by an atomic counter; this kernel keeps the general path's deterministic order).
//
// Thread i = source_rank * T + token (ep * T <= 1024), so ascending thread index is the (source rank, token)
// order of the output rows inside an expert: a row's position is its expert's base + the routes of lower warps
// + the routes of lower lanes of its own warp, all from per-warp lane masks in shared memory.  No workspace,
// no histogram in global memory, no memset.
// ---------------------------------------------------------------------------
constexpr int kDecodeThreads = 1024;
constexpr int kDecodeWarps = kDecodeThreads / 32;

__global__ void __launch_bounds__(kDecodeThreads) route_decode_kernel(RouteParams p) {
  extern __shared__ uint32_t smem_u[];
  uint32_t* mask = smem_u;                                                // [32][e_local] lane masks
  uint32_t* wprefix = mask + kDecodeWarps * p.e_local;                    // [32][e_local] routes of lower warps
  int32_t* hist_s = reinterpret_cast<int32_t*>(wprefix + kDecodeWarps * p.e_local);  // [E]
  int32_t* total = hist_s + p.E;                                          // [e_local] real rows
  int32_t* base = total + p.e_local;                                      // [e_local + 1] padded exclusive prefix
  __shared__ int overflow;
  __shared__ int mismatch;
  const int i = threadIdx.x, warp = i >> 5, lane = i & 31;
  if (i == 0) mismatch = 0;
  for (int j = i; j < kDecodeWarps * p.e_local; j += kDecodeThreads) mask[j] = 0u;
  for (int j = i; j < p.E; j += kDecodeThreads) hist_s[j] = 0;
  __syncthreads();
  const int s = i / p.T, tok = i - s * p.T;
  const bool live = s < p.ep;
  const int first = p.rank * p.e_local;
  const int16_t* ids = nullptr;
  if (live) {
    if (tok == 0) {
      const int peer_t = *reinterpret_cast<const int32_t*>(p.routing_ptrs[s]);
      if (peer_t != p.T) {
        set_status(p.status, kTokenCountMismatch, s, peer_t, p.T);
        mismatch = 1;
      }
    }
    ids = reinterpret_cast<const int16_t*>(p.routing_ptrs[s] + DM_ROUTING_HEADER_BYTES) + static_cast<int64_t>(tok) * p.K;
    for (int k = 0; k < p.K; ++k) {
      const int e = ids[k];
      if (e < 0 || e >= p.E) continue;
      atomicAdd(&hist_s[e], 1);
      const int el = e - first;
      if (el >= 0 && el < p.e_local) atomicOr(&mask[warp * p.e_local + el], 1u << lane);
    }
  }
  __syncthreads();
  for (int el = i; el < p.e_local; el += kDecodeThreads) {
    int running = 0;
    for (int w = 0; w < kDecodeWarps; ++w) {
      wprefix[w * p.e_local + el] = running;
      running += __popc(mask[w * p.e_local + el]);
    }
    total[el] = running;
  }
  __syncthreads();
  if (i == 0) {
    int64_t acc = 0;
    for (int el = 0; el < p.e_local; ++el) {
      base[el] = static_cast<int32_t>(acc);
      acc += pad_rows(total[el], p.m_mult);
    }
    base[p.e_local] = static_cast<int32_t>(acc);
    overflow = (acc > p.capacity_rows || acc > p.ptrs_size) ? 1 : 0;
    if (overflow) set_status(p.status, kCapacityExceeded, static_cast<int>(acc), static_cast<int>(p.capacity_rows));
    if (mismatch) overflow = 1;  // ranks that disagree on T: zero rows, the call becomes a no-op
  }
  __syncthreads();
  const bool bad = overflow != 0;
  for (int el = i; el <= p.e_local; el += kDecodeThreads) {
    p.expert_offsets[el] = bad ? 0 : base[el];
    if (el < p.e_local) p.counts[el] = bad ? 0 : pad_rows(total[el], p.m_mult);
    if (el < p.e_local && p.real_counts != nullptr) p.real_counts[el] = bad ? 0 : total[el];
  }
  for (int q = i; q < p.ep; q += kDecodeThreads) {
    int acc = 0;
    for (int el = 0; el < p.e_local; ++el) acc += pad_rows(hist_s[q * p.e_local + el], p.m_mult);
    p.per_rank[q] = acc;
  }
  if (bad) return;
  if (p.m_mult > 0) {
    // Padding rows of every expert segment hold a null pointer.
    for (int el = warp; el < p.e_local; el += kDecodeWarps) {
      const int lo = base[el] + total[el], hi = base[el + 1];
      for (int r = lo + lane; r < hi; r += 32) {
        p.fwd[r] = 0;
        p.sct[r] = 0;
        if (p.bwd != nullptr) p.bwd[r] = 0;
      }
    }
  }
  if (!live) return;
  const uint64_t dbase = p.dispatch_ptrs[s], cbase = p.combine_ptrs[s];
  for (int k = 0; k < p.K; ++k) {
    const int el = static_cast<int>(ids[k]) - first;
    if (ids[k] < 0 || ids[k] >= p.E || el < 0 || el >= p.e_local) continue;
    const int pos = base[el] + static_cast<int>(wprefix[warp * p.e_local + el]) +
                    __popc(mask[warp * p.e_local + el] & ((1u << lane) - 1u));
    const int64_t route = static_cast<int64_t>(tok) * p.K + k;
    p.fwd[pos] = static_cast<int64_t>(dbase + static_cast<uint64_t>(tok) * p.gather_stride);
    p.sct[pos] = static_cast<int64_t>(cbase + static_cast<uint64_t>(route) * p.scatter_stride);
    if (p.bwd != nullptr) p.bwd[pos] = static_cast<int64_t>(dbase + static_cast<uint64_t>(route) * p.bwd_stride);
  }
}

// ---------------------------------------------------------------------------
// Row gather through a pointer table (sources may be peer memory)
// ---------------------------------------------------------------------------
__global__ void gather_rows_kernel(const int64_t* __restrict__ ptrs, const int32_t* __restrict__ num_rows,
                                   uint8_t* dst_base, const int64_t* dst_offset, int vec_per_row, int64_t max_rows,
                                   const int* cond) {
  if (cond != nullptr && *cond == 0) return;
  int64_t rows = *num_rows;
  if (rows > max_rows) rows = max_rows;
  uint4* dst = reinterpret_cast<uint4*>(dst_base + (dst_offset ? *dst_offset : 0));
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int64_t r = blockIdx.x * static_cast<int64_t>(warps_per_block) + (threadIdx.x >> 5); r < rows;
       r += static_cast<int64_t>(gridDim.x) * warps_per_block) {
    const uint4* src = reinterpret_cast<const uint4*>(ptrs[r]);
    uint4* out = dst + r * vec_per_row;
    if (src == nullptr) {
      for (int v = lane; v < vec_per_row; v += 32) out[v] = make_uint4(0, 0, 0, 0);
    } else {
#pragma unroll 4
      for (int v = lane; v < vec_per_row; v += 32) out[v] = __ldcg(src + v);
    }
  }
}

__global__ void cond_copy_kernel(const uint8_t* src_base, const int64_t* src_offset, uint8_t* dst_base,
                                 const int64_t* dst_offset, int64_t n_vec, const int* cond, int expect) {
  if (cond != nullptr && ((*cond != 0) != (expect != 0))) return;
  const uint4* src = reinterpret_cast<const uint4*>(src_base + (src_offset ? *src_offset : 0));
  uint4* dst = reinterpret_cast<uint4*>(dst_base + (dst_offset ? *dst_offset : 0));
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n_vec;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    dst[i] = src[i];
}

}  // namespace dm

using namespace dm;

extern "C" int dm_version(void) { return 1000; }

extern "C" int dm_publish(const void* x_bf16, const void* ids, int ids_are_int64, void* dispatch_local,
                          void* routing_local, int64_t T, int64_t D, int K, int E, int validate, int* status,
                          void* stream) {
  if (ids == nullptr || routing_local == nullptr || T <= 0 || K <= 0 || E <= 0 || E > 32767) return kRcBadArg;
  if (x_bf16 != nullptr && (dispatch_local == nullptr || D <= 0 || (D % 8) != 0)) return kRcBadArg;
  const int64_t n_vec = x_bf16 ? T * D / 8 : 0;
  const int64_t n_ids = T * K;
  const int64_t work = n_vec > n_ids ? n_vec : n_ids;
  int blocks = static_cast<int>((work + 255) / 256);
  if (blocks > grid_cap(16)) blocks = grid_cap(16);
  if (blocks < 1) blocks = 1;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (ids_are_int64)
    publish_kernel<int64_t><<<blocks, 256, 0, st>>>(static_cast<const uint4*>(x_bf16), static_cast<const int64_t*>(ids),
                                                    static_cast<uint4*>(dispatch_local),
                                                    static_cast<uint8_t*>(routing_local), n_vec, n_ids,
                                                    static_cast<int>(T), E, validate, status);
  else
    publish_kernel<int32_t><<<blocks, 256, 0, st>>>(static_cast<const uint4*>(x_bf16), static_cast<const int32_t*>(ids),
                                                    static_cast<uint4*>(dispatch_local),
                                                    static_cast<uint8_t*>(routing_local), n_vec, n_ids,
                                                    static_cast<int>(T), E, validate, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_barrier(const uint64_t* signal_pads, int rank, int ep, int channel, const int* cond,
                          uint64_t timeout_ns, int* status, void* stream) {
  if (ep <= 0 || ep > 1024 || rank < 0 || rank >= ep || channel < 0) return kRcBadArg;
  if (ep == 1) return kRcOk;
  if (signal_pads == nullptr) return kRcBadArg;
  const int threads = (ep + 31) / 32 * 32;
  barrier_kernel<<<1, threads, 0, static_cast<cudaStream_t>(stream)>>>(signal_pads, rank, ep, channel, cond,
                                                                       timeout_ns, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int64_t dm_route_workspace_words(int64_t T, int ep, int E) {
  if (T <= 0 || ep <= 0 || E <= 0) return 0;
  const int64_t chunks = (T + kChunkTokens - 1) / kChunkTokens;
  const int64_t e_local = E / ep;
  return 2 * ep * chunks * e_local + E;
}

static int g_route_decode = 1;

extern "C" int dm_set_route_decode_kernel(int enabled) {
  const int previous = g_route_decode;
  g_route_decode = enabled ? 1 : 0;
  return previous;
}

extern "C" int dm_route_decode_kernel_enabled(void) { return g_route_decode; }

static int route_launch(const uint64_t* routing_ptrs, const uint64_t* dispatch_ptrs, const uint64_t* combine_ptrs,
                        int rank, int ep, int64_t T, int K, int E, int64_t gather_stride_bytes,
                        int64_t bwd_gather_stride_bytes, int64_t scatter_stride_bytes, int m_multiple_of,
                        int64_t capacity_rows, int64_t ptrs_size, int32_t* counts, int32_t* per_rank,
                        int32_t* expert_offsets, int64_t* fwd_gather_ptrs, int64_t* bwd_gather_ptrs,
                        int64_t* scatter_ptrs, int32_t* workspace, int64_t workspace_words, int* status,
                        void* stream, int32_t* real_counts = nullptr) {
  if (!routing_ptrs || !dispatch_ptrs || !combine_ptrs || !counts || !per_rank || !expert_offsets ||
      !fwd_gather_ptrs || !scatter_ptrs || !workspace)
    return kRcBadArg;
  if (ep <= 0 || rank < 0 || rank >= ep || T <= 0 || T > (1 << 24) || K <= 0 || E <= 0 || E % ep != 0 ||
      m_multiple_of < 0 || capacity_rows < 0 || ptrs_size < 0)
    return kRcBadArg;
  if (E > kMaxExpertsSmem) return kRcUnsupportedShape;
  if (workspace_words < dm_route_workspace_words(T, ep, E)) return kRcTooLarge;
  RouteParams p;
  p.routing_ptrs = routing_ptrs;
  p.dispatch_ptrs = dispatch_ptrs;
  p.combine_ptrs = combine_ptrs;
  p.rank = rank;
  p.ep = ep;
  p.T = static_cast<int>(T);
  p.K = K;
  p.E = E;
  p.e_local = E / ep;
  p.chunks = static_cast<int>((T + kChunkTokens - 1) / kChunkTokens);
  p.gather_stride = gather_stride_bytes;
  p.bwd_stride = bwd_gather_stride_bytes;
  p.scatter_stride = scatter_stride_bytes;
  p.m_mult = m_multiple_of;
  p.capacity_rows = capacity_rows;
  p.ptrs_size = ptrs_size;
  p.counts = counts;
  p.real_counts = real_counts;
  p.per_rank = per_rank;
  p.expert_offsets = expert_offsets;
  p.fwd = fwd_gather_ptrs;
  p.bwd = bwd_gather_ptrs;
  p.sct = scatter_ptrs;
  const int64_t n = static_cast<int64_t>(ep) * p.chunks * p.e_local;
  p.chunk_counts = workspace;
  p.chunk_offsets = workspace + n;
  p.hist = workspace + 2 * n;
  p.status = status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (g_route_decode && static_cast<int64_t>(ep) * T <= kDecodeThreads && p.e_local <= 512) {
    const size_t smem = sizeof(uint32_t) * (2 * kDecodeWarps * p.e_local + E + 2 * p.e_local + 1);
    static PerDeviceOnce attr_set;
    const int rc_attr = once_per_device(attr_set, [] {
      return static_cast<int>(
          cudaFuncSetAttribute(route_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               static_cast<int>(sizeof(uint32_t) * (2 * kDecodeWarps * 512 + kMaxExpertsSmem + 1025))));
    });
    if (rc_attr != 0) return rc_attr;
    route_decode_kernel<<<1, kDecodeThreads, smem, st>>>(p);
    return static_cast<int>(cudaGetLastError());
  }
  cudaError_t err = cudaMemsetAsync(p.hist, 0, sizeof(int32_t) * E, st);
  if (err != cudaSuccess) return static_cast<int>(err);
  const dim3 grid(p.chunks, ep);
  const size_t smem_count = sizeof(uint32_t) * (kChunkWarps * p.e_local + E);
  const size_t smem_fill = sizeof(uint32_t) * (kChunkWarps * p.e_local);
  route_count_kernel<<<grid, kChunkTokens, smem_count, st>>>(p);
  route_scan_kernel<<<1, 1024, sizeof(int32_t) * (2 * p.e_local + 1), st>>>(p);
  route_fill_kernel<<<grid, kChunkTokens, smem_fill, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_route(const uint64_t* routing_ptrs, const uint64_t* dispatch_ptrs, const uint64_t* combine_ptrs,
                        int rank, int ep, int64_t T, int K, int E, int64_t gather_stride_bytes,
                        int64_t bwd_gather_stride_bytes, int64_t scatter_stride_bytes, int m_multiple_of,
                        int64_t capacity_rows, int64_t ptrs_size, int32_t* counts, int32_t* per_rank,
                        int32_t* expert_offsets, int64_t* fwd_gather_ptrs, int64_t* bwd_gather_ptrs,
                        int64_t* scatter_ptrs, int32_t* workspace, int64_t workspace_words, int* status,
                        void* stream) {
  return route_launch(routing_ptrs, dispatch_ptrs, combine_ptrs, rank, ep, T, K, E, gather_stride_bytes,
                      bwd_gather_stride_bytes, scatter_stride_bytes, m_multiple_of, capacity_rows, ptrs_size, counts,
                      per_rank, expert_offsets, fwd_gather_ptrs, bwd_gather_ptrs, scatter_ptrs, workspace,
                      workspace_words, status, stream);
}

// dm_route that also reports the rows of every expert before padding to m_multiple_of (the swapped-operand
// block-scaled GEMMs size their N side from it).
extern "C" int dm_route_counted(const uint64_t* routing_ptrs, const uint64_t* dispatch_ptrs,
                                const uint64_t* combine_ptrs, int rank, int ep, int64_t T, int K, int E,
                                int64_t gather_stride_bytes, int64_t bwd_gather_stride_bytes,
                                int64_t scatter_stride_bytes, int m_multiple_of, int64_t capacity_rows,
                                int64_t ptrs_size, int32_t* counts, int32_t* real_counts, int32_t* per_rank,
                                int32_t* expert_offsets, int64_t* fwd_gather_ptrs, int64_t* bwd_gather_ptrs,
                                int64_t* scatter_ptrs, int32_t* workspace, int64_t workspace_words, int* status,
                                void* stream) {
  if (!real_counts) return kRcBadArg;
  return route_launch(routing_ptrs, dispatch_ptrs, combine_ptrs, rank, ep, T, K, E, gather_stride_bytes,
                      bwd_gather_stride_bytes, scatter_stride_bytes, m_multiple_of, capacity_rows, ptrs_size, counts,
                      per_rank, expert_offsets, fwd_gather_ptrs, bwd_gather_ptrs, scatter_ptrs, workspace,
                      workspace_words, status, stream, real_counts);
}

// ---------------------------------------------------------------------------
// Routing for callers that cannot allocate: the chunk counters, chunk offsets and the
// expert histogram live in a fixed array that is part of the library image.
// ---------------------------------------------------------------------------
namespace dm {
constexpr int64_t kStaticRouteWords = DM_ROUTE_STATIC_MAX_WORDS;
static __device__ __align__(256) int32_t g_route_scratch[kStaticRouteWords];
static int32_t* g_route_scratch_addr[kMaxDevices];  // device address of the array, per device
}  // namespace dm

extern "C" int dm_route_static(const uint64_t* routing_ptrs, const uint64_t* dispatch_ptrs,
                               const uint64_t* combine_ptrs, int rank, int ep, int64_t T, int K, int E,
                               int64_t gather_stride_bytes, int64_t bwd_gather_stride_bytes,
                               int64_t scatter_stride_bytes, int m_multiple_of, int64_t capacity_rows,
                               int64_t ptrs_size, int32_t* counts, int32_t* per_rank, int32_t* expert_offsets,
                               int64_t* fwd_gather_ptrs, int64_t* bwd_gather_ptrs, int64_t* scatter_ptrs, int* status,
                               void* stream) {
  const int64_t need = dm_route_workspace_words(T, ep, E);
  if (need <= 0) return kRcBadArg;
  if (need > kStaticRouteWords) return kRcTooLarge;
  int dev = 0;
  cudaError_t err = cudaGetDevice(&dev);
  if (err != cudaSuccess) return static_cast<int>(err);
  if (dev < 0 || dev >= kMaxDevices) return kRcTooLarge;
  if (g_route_scratch_addr[dev] == nullptr) {
    // In host code the array's name is only a handle; the kernels need its address on the current device.
    void* addr = nullptr;
    err = cudaGetSymbolAddress(&addr, g_route_scratch);
    if (err != cudaSuccess) return static_cast<int>(err);
    if (addr == nullptr) return kRcBadArg;
    g_route_scratch_addr[dev] = static_cast<int32_t*>(addr);
  }
  return route_launch(routing_ptrs, dispatch_ptrs, combine_ptrs, rank, ep, T, K, E, gather_stride_bytes,
                      bwd_gather_stride_bytes, scatter_stride_bytes, m_multiple_of, capacity_rows, ptrs_size, counts,
                      per_rank, expert_offsets, fwd_gather_ptrs, bwd_gather_ptrs, scatter_ptrs,
                      g_route_scratch_addr[dev], kStaticRouteWords, status, stream);
}

extern "C" int dm_gather_rows(const int64_t* ptrs, const int32_t* num_rows, void* dst_base, const int64_t* dst_offset,
                              int64_t row_bytes, int64_t max_rows, const int* cond, void* stream) {
  if (!ptrs || !num_rows || !dst_base || row_bytes <= 0 || (row_bytes % 16) != 0 || max_rows < 0) return kRcBadArg;
  if (max_rows == 0) return kRcOk;
  const int warps = 8;
  int64_t blocks = (max_rows + warps - 1) / warps;
  if (blocks > grid_cap(8)) blocks = grid_cap(8);
  gather_rows_kernel<<<static_cast<int>(blocks), warps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
      ptrs, num_rows, static_cast<uint8_t*>(dst_base), dst_offset, static_cast<int>(row_bytes / 16), max_rows, cond);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int dm_cond_copy(const void* src_base, const int64_t* src_offset, void* dst_base, const int64_t* dst_offset,
                            int64_t bytes, const int* cond, int expect, void* stream) {
  if (!src_base || !dst_base || bytes < 0 || (bytes % 16) != 0) return kRcBadArg;
  if (bytes == 0) return kRcOk;
  const int64_t n_vec = bytes / 16;
  int64_t blocks = (n_vec + 255) / 256;
  if (blocks > grid_cap(16)) blocks = grid_cap(16);
  cond_copy_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src_base), src_offset, static_cast<uint8_t*>(dst_base), dst_offset, n_vec, cond,
      expect);
  return static_cast<int>(cudaGetLastError());
}
