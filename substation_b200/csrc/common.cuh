// Shared device/host helpers for the fused operators: strided tensor views,
// 128-bit vector access with a scalar fallback, warp reductions and the
// counter-based dropout generator.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstring>
#include <string>

#include "../../include/substation_b200.h"

// ---------------------------------------------------------------------------
// Storage type of activations and parameters.  The library is built once per type (fp16 by default, bf16 with
// -DSB_BF16): sb_half / sb_half2 and the handful of conversions below are all that differs; every reduction and
// accumulation is fp32 in both.  The reference selects the type the same way, at compile time
// (pytorch_module/encoder.py:13-17, `Real`).
// ---------------------------------------------------------------------------
#ifdef SB_BF16
typedef __nv_bfloat16 sb_half;
typedef __nv_bfloat162 sb_half2;
#define SB_ONE_BITS 0x3F80u                      /* 1.0 */
#define SB_TMAP_DTYPE CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
#define SB_IDESC_AB_FMT ((1u << 7) | (1u << 10)) /* tcgen05 instruction descriptor: A and B are bf16 */
#define SB_DTYPE_NAME "bf16"
#else
typedef __half sb_half;
typedef __half2 sb_half2;
#define SB_ONE_BITS 0x3C00u
#define SB_TMAP_DTYPE CU_TENSOR_MAP_DATA_TYPE_FLOAT16
#define SB_IDESC_AB_FMT 0u
#define SB_DTYPE_NAME "fp16"
#endif

#ifdef __CUDACC__
#ifdef SB_BF16
__host__ __device__ __forceinline__ float sb_h2f(sb_half h) { return __bfloat162float(h); }
__host__ __device__ __forceinline__ sb_half sb_f2h(float f) { return __float2bfloat16_rn(f); }
__device__ __forceinline__ float2 sb_h22f2(sb_half2 h) { return __bfloat1622float2(h); }
__device__ __forceinline__ sb_half2 sb_f2h2(float a, float b) { return __floats2bfloat162_rn(a, b); }
__device__ __forceinline__ sb_half2 sb_f2h2_dup(float a) { return __float2bfloat162_rn(a); }
__device__ __forceinline__ sb_half2 sb_h2h2(sb_half h) { return __bfloat162bfloat162(h); }
#else
__host__ __device__ __forceinline__ float sb_h2f(sb_half h) { return __half2float(h); }
__host__ __device__ __forceinline__ sb_half sb_f2h(float f) { return __float2half_rn(f); }
__device__ __forceinline__ float2 sb_h22f2(sb_half2 h) { return __half22float2(h); }
__device__ __forceinline__ sb_half2 sb_f2h2(float a, float b) { return __floats2half2_rn(a, b); }
__device__ __forceinline__ sb_half2 sb_f2h2_dup(float a) { return __float2half2_rn(a); }
__device__ __forceinline__ sb_half2 sb_h2h2(sb_half h) { return __half2half2(h); }
#endif
#endif

namespace sb {

// ---------------------------------------------------------------------------
// Error plumbing (host)
// ---------------------------------------------------------------------------
void set_error(const std::string& msg);
int fail(int status, const std::string& msg);

#define SB_CUDA_OK(expr)                                                                  \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess)                                                                \
      return ::sb::fail(SB_ERR_CUDA, std::string(#expr) + ": " + cudaGetErrorString(_e)); \
  } while (0)

#define SB_TRY(expr)             \
  do {                           \
    int _s = (expr);             \
    if (_s != SB_OK) return _s;  \
  } while (0)

// ---------------------------------------------------------------------------
// Views.  "vec" means: innermost logical dim has unit stride, its extent is a
// multiple of 8, every other stride is a multiple of 8 elements and the base
// is 16-byte aligned (8-byte for uint8 masks), so each aligned group of eight
// elements along that dim is one 128-bit (64-bit) access.
// ---------------------------------------------------------------------------
struct View3 {  // [B, J, F]
  void* p;
  long long sB, sJ, sF;
  int vec;
};
struct View2 {  // [B, J]
  void* p;
  long long sB, sJ;
};
struct View4 {  // [H, B, J, K]
  void* p;
  long long sH, sB, sJ, sK;
  int vec;
};
struct View5 {  // [N, P, H, B, J]
  void* p;
  long long sN, sP, sH, sB, sJ;
  int vec;
};

struct Rng {
  uint32_t seed_lo, seed_hi, off_lo, off_hi;
  uint32_t thr;  // drop when 16 random bits < thr
  int philox;    // 0: masks are inputs; 1: masks are generated and written
};

#ifdef __CUDACC__

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  Every kernel of the library is launched with
// the programmatic-stream-serialization attribute and begins with
// grid_dependency_sync(): the next kernel's CTAs may be scheduled, and run
// whatever set-up precedes that call, while the previous kernel drains; nothing
// touches global memory before the previous grid has completed and flushed.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void grid_dependency_sync() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

bool pdl_enabled();  // false when the environment sets SUBSTATION_B200_PDL=0

// ---- per-device facts asked of the runtime once per thread, not once per launch ----------------
struct DeviceFacts {
  int device = -1;
  int sms = 148;
};
// Current device and its SM count (one cudaGetDevice per call; the attribute is cached per device).
inline const DeviceFacts& device_facts() {
  static thread_local DeviceFacts facts[64];
  static thread_local DeviceFacts fallback;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) {
    fallback.device = dev;
    cudaDeviceGetAttribute(&fallback.sms, cudaDevAttrMultiProcessorCount, dev);
    return fallback;
  }
  DeviceFacts& f = facts[dev];
  if (f.device != dev) {
    f.device = dev;
    if (cudaDeviceGetAttribute(&f.sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) f.sms = 148;
  }
  return f;
}
// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per (kernel, device, size) and thread.
inline cudaError_t ensure_dynamic_smem(const void* kernel, int bytes) {
  struct Done { const void* fn; int dev; int bytes; };
  static thread_local Done done[64];
  static thread_local int ndone = 0;
  const int dev = device_facts().device;
  for (int i = 0; i < ndone; ++i)
    if (done[i].fn == kernel && done[i].dev == dev && done[i].bytes == bytes) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess && ndone < 64) done[ndone++] = Done{kernel, dev, bytes};
  return e;
}
// Resident CTAs per SM of a kernel at a block size (no dynamic shared memory), cached like the above.
inline int cached_blocks_per_sm(const void* kernel, int threads) {
  struct Occ { const void* fn; int dev; int threads; int per_sm; };
  static thread_local Occ occ[64];
  static thread_local int nocc = 0;
  const int dev = device_facts().device;
  for (int i = 0; i < nocc; ++i)
    if (occ[i].fn == kernel && occ[i].dev == dev && occ[i].threads == threads) return occ[i].per_sm;
  int per_sm = 1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess || per_sm < 1) {
    cudaGetLastError();
    per_sm = 1;
  }
  if (nocc < 64) occ[nocc++] = Occ{kernel, dev, threads, per_sm};
  return per_sm;
}

// Kernels launched through launch_k by this thread (the layer handle reports the difference over a pass).
extern thread_local long long g_kernel_launches;

template <class... KArgs, class... Args>
cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                     Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  ++g_kernel_launches;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define SB_LAUNCH_OK(expr)                                                              \
  do {                                                                                  \
    cudaError_t _e = (expr);                                                            \
    if (_e != cudaSuccess)                                                              \
      return ::sb::fail(SB_ERR_CUDA, std::string("kernel launch: ") + cudaGetErrorString(_e)); \
  } while (0)

constexpr int kWarp = 32;
constexpr float kLnEps = 1e-5f;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <int LANES>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
template <int LANES>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
  for (int o = LANES / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- 8-element accessors -------------------------------------------------
__device__ __forceinline__ void unpack8(const uint4& u, float v[8]) {
  const sb_half2* h = reinterpret_cast<const sb_half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = sb_h22f2(h[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float v[8]) {
  uint4 u;
  sb_half2* h = reinterpret_cast<sb_half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = sb_f2h2(v[2 * i], v[2 * i + 1]);
  return u;
}

// Load eight fp16 values base[(f..f+7)*sF] as float; elements at or beyond F read as `fill`.
__device__ __forceinline__ void load8h(const void* base, long long off, long long sF, int vec,
                                       int f, int F, float v[8], float fill = 0.f) {
  const sb_half* p = reinterpret_cast<const sb_half*>(base) + off;
  if (vec) {
    uint4 u = *reinterpret_cast<const uint4*>(p + f);
    unpack8(u, v);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = (f + e < F) ? sb_h2f(p[(long long)(f + e) * sF]) : fill;
  }
}
__device__ __forceinline__ void store8h(void* base, long long off, long long sF, int vec, int f,
                                        int F, const float v[8]) {
  sb_half* p = reinterpret_cast<sb_half*>(base) + off;
  if (vec) {
    *reinterpret_cast<uint4*>(p + f) = pack8(v);
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (f + e < F) p[(long long)(f + e) * sF] = sb_f2h(v[e]);
  }
}
__device__ __forceinline__ void load8m(const void* base, long long off, long long sF, int vec,
                                       int f, int F, uint32_t m[8]) {
  const uint8_t* p = reinterpret_cast<const uint8_t*>(base) + off;
  if (vec) {
    uint2 u = *reinterpret_cast<const uint2*>(p + f);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      m[e] = (u.x >> (8 * e)) & 0xffu;
      m[4 + e] = (u.y >> (8 * e)) & 0xffu;
    }
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) m[e] = (f + e < F) ? p[(long long)(f + e) * sF] : 0u;
  }
}
__device__ __forceinline__ void store8m(void* base, long long off, long long sF, int vec, int f,
                                        int F, const uint32_t m[8]) {
  uint8_t* p = reinterpret_cast<uint8_t*>(base) + off;
  if (vec) {
    uint2 u;
    u.x = m[0] | (m[1] << 8) | (m[2] << 16) | (m[3] << 24);
    u.y = m[4] | (m[5] << 8) | (m[6] << 16) | (m[7] << 24);
    *reinterpret_cast<uint2*>(p + f) = u;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (f + e < F) p[(long long)(f + e) * sF] = (uint8_t)m[e];
  }
}
// ---- raw forms: eight fp16 values stay packed in one uint4 and eight mask bytes in one
// uint2 until they are used, so data in flight costs 4 (2) registers per access ------------
__device__ __forceinline__ uint4 load8h_raw(const void* base, long long off, long long sF, int vec,
                                            int f, int F) {
  const sb_half* p = reinterpret_cast<const sb_half*>(base) + off;
  if (vec) return *reinterpret_cast<const uint4*>(p + f);
  uint4 u;
  sb_half* h = reinterpret_cast<sb_half*>(&u);
#pragma unroll
  for (int e = 0; e < 8; ++e) h[e] = (f + e < F) ? p[(long long)(f + e) * sF] : sb_f2h(0.f);
  return u;
}
__device__ __forceinline__ void store8h_raw(void* base, long long off, long long sF, int vec, int f,
                                            int F, const uint4& u) {
  sb_half* p = reinterpret_cast<sb_half*>(base) + off;
  if (vec) {
    *reinterpret_cast<uint4*>(p + f) = u;
  } else {
    const sb_half* h = reinterpret_cast<const sb_half*>(&u);
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (f + e < F) p[(long long)(f + e) * sF] = h[e];
  }
}
__device__ __forceinline__ uint2 load8m_raw(const void* base, long long off, long long sF, int vec,
                                            int f, int F) {
  const uint8_t* p = reinterpret_cast<const uint8_t*>(base) + off;
  if (vec) return *reinterpret_cast<const uint2*>(p + f);
  uint32_t w[2] = {0u, 0u};
#pragma unroll
  for (int e = 0; e < 8; ++e)
    if (f + e < F) w[e >> 2] |= (uint32_t)p[(long long)(f + e) * sF] << (8 * (e & 3));
  return make_uint2(w[0], w[1]);
}
__device__ __forceinline__ void store8m_raw(void* base, long long off, long long sF, int vec, int f,
                                            int F, const uint2& u) {
  uint8_t* p = reinterpret_cast<uint8_t*>(base) + off;
  if (vec) {
    *reinterpret_cast<uint2*>(p + f) = u;
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e)
      if (f + e < F) p[(long long)(f + e) * sF] = (uint8_t)(((e < 4 ? u.x : u.y) >> (8 * (e & 3))) & 0xffu);
  }
}
// keep flag of element e (0..7) of a packed mask
__device__ __forceinline__ bool mask_keep(const uint2& m, int e) {
  return (((e < 4 ? m.x : m.y) >> (8 * (e & 3))) & 0xffu) != 0u;
}
__device__ __forceinline__ uint2 mask_pack(const uint32_t m[8]) {
  return make_uint2(m[0] | (m[1] << 8) | (m[2] << 16) | (m[3] << 24),
                    m[4] | (m[5] << 8) | (m[6] << 16) | (m[7] << 24));
}

// Two mask bytes (0/1) -> half2 of 0.0/1.0: spread the bytes to 16-bit lanes, multiply by 0x3C00.
__device__ __forceinline__ sb_half2 mask_half2(uint32_t word, int pair) {
  const uint32_t spread = __byte_perm(word, 0u, pair ? 0x4342 : 0x4140);  // (b_lo, 0, b_hi, 0)
  const uint32_t bits = spread * SB_ONE_BITS;
  return *reinterpret_cast<const sb_half2*>(&bits);
}
// out = v (8 packed halves) times the 0/1 mask, lane for lane
__device__ __forceinline__ uint4 mask_apply(const uint4& v, const uint2& m) {
  uint4 o;
  const sb_half2* h = reinterpret_cast<const sb_half2*>(&v);
  sb_half2* q = reinterpret_cast<sb_half2*>(&o);
  q[0] = __hmul2(h[0], mask_half2(m.x, 0));
  q[1] = __hmul2(h[1], mask_half2(m.x, 1));
  q[2] = __hmul2(h[2], mask_half2(m.y, 0));
  q[3] = __hmul2(h[3], mask_half2(m.y, 1));
  return o;
}

// lane-wise sum of 8 packed halves (fp16 arithmetic, one rounding, like the flat elementwise kernels)
__device__ __forceinline__ uint4 hadd8(const uint4& a, const uint4& b) {
  uint4 o;
  const sb_half2* x = reinterpret_cast<const sb_half2*>(&a);
  const sb_half2* y = reinterpret_cast<const sb_half2*>(&b);
  sb_half2* q = reinterpret_cast<sb_half2*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) q[i] = __hadd2(x[i], y[i]);
  return o;
}

__device__ __forceinline__ float act_fwd(float x, int activation) {
  if (activation == SB_ACT_RELU) return fmaxf(x, 0.f);
  // tanh-form GELU
  const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.f + tanhf(u));
}

// Contiguous per-feature vectors (bias, gamma, beta): [F], unit stride.
__device__ __forceinline__ void load8p(const void* base, int f, int F, int vec, float v[8]) {
  load8h(base, 0, 1, vec, f, F, v, 0.f);
}

// ---- Philox4x32-10 ---------------------------------------------------------
__device__ __forceinline__ uint4 philox4x32_10(uint4 c, uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c.x), lo0 = 0xD2511F53u * c.x;
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c.z), lo1 = 0xCD9E8D57u * c.z;
    c = make_uint4(hi1 ^ c.y ^ k0, lo1, hi0 ^ c.w ^ k1, lo0);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  return c;
}
// Keep flags (0/1) of the eight elements of logical group g (= linear index >> 3).
__device__ __forceinline__ void philox_keep8(const Rng& r, unsigned long long g, uint32_t m[8]) {
  uint4 w = philox4x32_10(make_uint4((uint32_t)g, (uint32_t)(g >> 32), r.off_lo, r.off_hi),
                          r.seed_lo, r.seed_hi);
  const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
  for (int t = 0; t < 8; ++t) m[t] = (((ww[t >> 1] >> (16 * (t & 1))) & 0xffffu) >= r.thr) ? 1u : 0u;
}
// Keep flags for eight consecutive logical indices e0..e0+7 that need not be group aligned.
__device__ __forceinline__ void philox_keep8_unaligned(const Rng& r, unsigned long long e0,
                                                       uint32_t m[8]) {
  if ((e0 & 7ull) == 0) {
    philox_keep8(r, e0 >> 3, m);
    return;
  }
  uint32_t a[8], b[8];
  philox_keep8(r, e0 >> 3, a);
  philox_keep8(r, (e0 >> 3) + 1, b);
  const int s = (int)(e0 & 7ull);
#pragma unroll
  for (int t = 0; t < 8; ++t) m[t] = (t + s < 8) ? a[(t + s) & 7] : b[(t + s) & 7];
}

#endif  // __CUDACC__

}  // namespace sb
