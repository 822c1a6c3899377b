// Shared device helpers for the routed-expert kernels (sm_100a only).
//
// Everything here is a thin wrapper over one PTX instruction or a tiny
// bounded-wait loop.  No kernel in this library spins without a deadline: a wait
// that runs out records a status code and lets the CTA drain and exit.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace dm {

// Status codes written to the status words (int32[8]) owned by the context.
// word 0 = first error code (0 = ok), words 1..3 = detail values.
enum Status : int {
  kOk = 0,
  kTokenCountMismatch = 1,   // peers published different T
  kCapacityExceeded = 2,     // routed rows exceed the scratch row capacity
  kInvalidExpertId = 3,      // id outside [-1, E)
  kBarrierTimeout = 4,       // a peer did not arrive in time
  kPipelineTimeout = 5,      // an mbarrier wait inside a GEMM ran out
  kArenaOverflow = 6,        // planner: slot or scratch would overflow
};

// Return codes of the extern "C" entry points (negative = argument error,
// positive = cudaError_t of the failing runtime call).
enum Rc : int {
  kRcOk = 0,
  kRcBadArg = -1,
  kRcUnsupportedShape = -2,
  kRcTooLarge = -3,
  kRcNoDriver = -4,
};

__device__ __forceinline__ void set_status(int* status, int code, int a = 0, int b = 0, int c = 0) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0, code) == 0) {
    status[1] = a;
    status[2] = b;
    status[3] = c;
    __threadfence_system();
  }
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the deadline passed (the caller records a
// status and drains).  `abort_flag` is a shared-memory word any role sets when
// it gave up, so that the other roles stop waiting too.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          uint64_t budget_ns = 2000000000ull) {
  uint32_t ok;
  for (int fast = 0; fast < 64; ++fast) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    if (ok) return true;
  }
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    if (ok) return true;
    if ((++spins & 0xff) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > budget_ns) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// ----------------------------------------------------------------------------
// TMA (tiled, no multicast) and proxy fences
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tmap, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const void* tmap, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// Untiled bulk copy global -> shared (both 16-byte aligned, size a multiple of 16), no multicast.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }
__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* p, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ----------------------------------------------------------------------------
// tcgen05 / TMEM (cta_group::1)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrive on an mbarrier once every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Block-scaled MMAs: scale factors live in TMEM (copied there by tcgen05.cp from shared memory).
__device__ __forceinline__ void umma_mxf8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
__device__ __forceinline__ void umma_nvf4(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t"
      "}\n"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}
// Copy one 128-row x 4-scale atom (32 rows x 16 bytes in shared memory) into 4 TMEM columns, replicated
// over the four 32-lane sub-partitions.
__device__ __forceinline__ void tmem_cp_sf_atom(uint32_t taddr, uint64_t smem_desc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
}
// Shared-memory descriptor of a scale atom: no swizzle, rows 16 bytes apart, 8-row groups 128 bytes apart.
__device__ __forceinline__ uint64_t sf_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>(16 >> 4) << 16;
  d |= static_cast<uint64_t>(128 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  return d;
}
// Instruction descriptor of the block-scaled kinds (M128, K-major operands).
//   fp4 == 0: kind::mxf8f6f4, E4M3 data, UE8M0 scales, sf ids select the scale byte of the K=32 step.
//   fp4 != 0: kind::mxf4nvf4, E2M1 data, UE4M3 scales (4 per K=64 step).
__host__ __device__ constexpr uint32_t umma_idesc_blockscaled(int n, int fp4, int a_sf_id, int b_sf_id,
                                                              int a_mn_major = 0, int b_mn_major = 0) {
  return (static_cast<uint32_t>(a_mn_major) << 15) | (static_cast<uint32_t>(b_mn_major) << 16) |
         (static_cast<uint32_t>(b_sf_id) << 4) | (static_cast<uint32_t>(fp4 ? 1 : 0) << 7) |
         (static_cast<uint32_t>(fp4 ? 1 : 0) << 10) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(fp4 ? 0 : 1) << 23) | (static_cast<uint32_t>(128 >> 4) << 24) |
         (static_cast<uint32_t>(a_sf_id) << 29);
}

// 32 lanes x 32 consecutive fp32 columns: thread i of the warp reads TMEM lane
// (lane_base + i), columns [col, col+32).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for tcgen05.mma, 128-byte swizzle.
//   K-major operand : rows of 128 B (64 bf16 of K), 8-row groups 1024 B apart (SBO).
//   MN-major operand: lines of 128 B (64 bf16 of M/N), one line per k, 8-k groups
//                     1024 B apart (SBO), 64-element M/N groups `lbo_bytes` apart.
// Bits: [0,14) start>>4, [16,30) LBO>>4, [32,46) SBO>>4, [46,48) version=1, [61,64) layout=2.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

// Instruction descriptor, kind::f16, bf16 x bf16 -> fp32.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n, int a_mn_major, int b_mn_major) {
  return (1u << 4)                                   // D format fp32
         | (1u << 7)                                 // A format bf16
         | (1u << 10)                                // B format bf16
         | (static_cast<uint32_t>(a_mn_major) << 15)
         | (static_cast<uint32_t>(b_mn_major) << 16)
         | (static_cast<uint32_t>(n >> 3) << 17)
         | (static_cast<uint32_t>(m >> 4) << 24);
}

// ----------------------------------------------------------------------------
// Small numeric helpers
// ----------------------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) { return __uint_as_float(bits16 << 16); }

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// sigmoid(x) = 1 / (1 + exp(-x)) with an IEEE round-to-nearest reciprocal.
__device__ __forceinline__ float sigmoid_rn(float x) { return __frcp_rn(1.0f + expf(-x)); }

struct ActParams {
  int clamped;   // 0 = plain SwiGLU, 1 = clamped
  float alpha;   // sigmoid multiplier (clamped only)
  float limit;   // clamp bound (clamped only)
};

// h2 = SwiGLU(gate, up) in fp32.
__device__ __forceinline__ float swiglu_f32(float gate, float up, const ActParams& act) {
  if (act.clamped) {
    float g = fminf(gate, act.limit);
    float u = fminf(fmaxf(up, -act.limit), act.limit);
    return g * sigmoid_rn(act.alpha * g) * (u + 1.0f);
  }
  return gate * sigmoid_rn(gate) * up;
}

// Gradients of h2 = SwiGLU(x, y) with respect to the gate x and the up value y, given dz = dL/dh2
// (dist_moe/kernels/triton/swiglu.py:639-668: where a clamp saturates, that input's gradient is zero).
__device__ __forceinline__ void swiglu_bwd_f32(float x, float y, float dz, const ActParams& act, float& dx, float& dy) {
  if (act.clamped) {
    const float g = fminf(x, act.limit);
    const float u = fminf(fmaxf(y, -act.limit), act.limit);
    const float s = sigmoid_rn(act.alpha * g);
    const float silu = g * s;
    const float d_silu = s + act.alpha * g * s * (1.0f - s);
    float a = dz * (u + 1.0f) * d_silu;
    float b = dz * silu;
    dx = x > act.limit ? 0.0f : a;
    dy = (y > act.limit || y < -act.limit) ? 0.0f : b;
  } else {
    const float s = sigmoid_rn(x);
    dx = dz * y * s * (1.0f + x - x * s);
    dy = dz * x * s;
  }
}

// ---- per-device host state ------------------------------------------------------------------------------
// cudaFuncSetAttribute and the SM count belong to ONE device; a process may drive several, so every cache of
// such a fact is indexed by the current device.
constexpr int kMaxDevices = 64;

static inline int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

struct PerDeviceOnce {
  bool done[kMaxDevices] = {};
};

// Runs `setup` (returning a cudaError_t-compatible int) once per device; on an unknown device, every call.
template <class Fn>
static inline int once_per_device(PerDeviceOnce& once, Fn&& setup) {
  const int slot = current_device_slot();
  if (slot >= 0 && once.done[slot]) return 0;
  const int rc = setup();
  if (rc == 0 && slot >= 0) once.done[slot] = true;
  return rc;
}

static inline int sm_count() {
  static int cached[kMaxDevices] = {};
  const int slot = current_device_slot();
  if (slot >= 0 && cached[slot] > 0) return cached[slot];
  int n = 0;
  if (slot < 0 || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, slot) != cudaSuccess || n <= 0) return 148;
  cached[slot] = n;
  return n;
}

// Grid of a persistent one-CTA-per-SM kernel: the caller's wish, never more than the device has SMs.  The fused
// dispatch launches make CTAs wait on counters that other CTAs publish, so every CTA must be resident.
static inline int persistent_grid(int num_sms) {
  const int n = sm_count();
  return (num_sms > 0 && num_sms < n) ? num_sms : n;
}

// Grid cap for grid-stride kernels: `per_sm` CTAs per SM of the current device.
static inline int grid_cap(int per_sm) { return sm_count() * per_sm; }

__host__ __device__ constexpr int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ constexpr int64_t align_up64(int64_t a, int64_t b) { return (a + b - 1) / b * b; }

}  // namespace dm
