// Fused LayerNorm-backward operators: the LayerNorm scale/bias gradients, the
// LayerNorm backward-data with dropout, and the bias gradients that are plain
// sums over tokens of tensors this pass touches anyway, in ONE pass over the data.
//
//   mode A  = backward_scale_bias + backward_layernorm_residual_dropout
//             (pytorch_module/block_bsb_ebsb.cuh:171-216, block_blnrd.cuh:71-129)
//   mode B  = extended_backward_scale_bias + backward_layernorm_residual_dropout
//             + backward_attn_out_bias
//             (block_bsb_ebsb.cuh:368-420, block_blnrd.cuh:195-259, block_baob.cuh:75-97)
//
// Both need sums over features (per token) AND sums over tokens (per feature).
// Mapping: a CTA has 4 row groups of 128 threads; the 128 threads of a group span
// one token (8 features each, up to 1024 features) and walk tokens with a grid
// stride, two tokens in flight.  Per-token sums: warp shuffles, then the group's
// 4 warps exchange through shared memory behind a group-local named barrier.
// Per-feature sums: each thread accumulates its 8 features in registers over all
// of its tokens; at the end the 4 groups are added in order, the CTA writes one
// fp32 partial row per quantity, and a second small kernel adds the partial rows
// in order (deterministic).

#include <algorithm>

#include "ops.h"

namespace sb {

namespace {

constexpr int kGroups = 4;
constexpr int kGroupThreads = 128;
constexpr int kThreads = kGroups * kGroupThreads;  // 512
constexpr int kRows = 2;                           // tokens in flight per group
constexpr int kMaxF = 1024;

struct LnBwdParams {
  Dims3 d;
  // mode A: y = DY, n = LN, (r2, w, l2 unused).  mode B: n = LN1, r2 = DRESID2, w = DLIN1_LINW1, l2 = DLIN2
  View3 y, n, r2, w, l2;
  View3 diff, mask;
  View2 istd;
  View3 dln, dresid, dlin;  // outputs: g*gamma, LayerNorm backward-data, its dropout-masked copy
  const void* gamma;
  float* partial;           // [NQ][P][1024]
};

__device__ __forceinline__ void group_barrier(int group) {
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(kGroupThreads) : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(kThreads, 1)
lnbwd_kernel(LnBwdParams p) {
  grid_dependency_sync();
  constexpr int NQ = MODE == 0 ? 2 : 4;
  constexpr int NIN = MODE == 0 ? 2 : 4;
  __shared__ float red[kGroups][2][4][2 * kRows];
  extern __shared__ float colred[];  // [kGroups][NQ][1024]
  const int tid = threadIdx.x;
  const int group = tid / kGroupThreads, t = tid % kGroupThreads;
  const int warp_in_group = t >> 5, lane = t & 31;
  const int f = t * 8;
  const int F = p.d.F;
  const bool active = f < F;
  const unsigned R = (unsigned)p.d.B * (unsigned)p.d.J;
  const unsigned stride = gridDim.x * kGroups;
  const float invn = 1.f / (float)F;

  float gm[8];
  if (active) unpack8(load8h_raw(p.gamma, 0, 1, 1, f, F), gm);
  float acc[NQ][8];
#pragma unroll
  for (int q = 0; q < NQ; ++q)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[q][e] = 0.f;

  unsigned iter = 0;
  for (unsigned row0 = blockIdx.x * kGroups + group; row0 < R; row0 += stride * kRows, ++iter) {
    uint4 in[kRows][NIN], df[kRows];
    uint2 mk[kRows];
    long long off_out[kRows][3];
    float s[kRows];
    bool valid[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      const unsigned row = row0 + r * stride;
      valid[r] = row < R;
      const unsigned rr = valid[r] ? row : R - 1;
      const int b = (int)(rr / (unsigned)p.d.J), j = (int)(rr % (unsigned)p.d.J);
      if (active) {
        if (MODE == 0) {
          in[r][0] = load8h_raw(p.y.p, b * p.y.sB + j * p.y.sJ, 1, 1, f, F);
          in[r][1] = load8h_raw(p.n.p, b * p.n.sB + j * p.n.sJ, 1, 1, f, F);
        } else {
          in[r][0] = load8h_raw(p.n.p, b * p.n.sB + j * p.n.sJ, 1, 1, f, F);
          in[r][1] = load8h_raw(p.r2.p, b * p.r2.sB + j * p.r2.sJ, 1, 1, f, F);
          in[r][2] = load8h_raw(p.w.p, b * p.w.sB + j * p.w.sJ, 1, 1, f, F);
          in[r][3] = load8h_raw(p.l2.p, b * p.l2.sB + j * p.l2.sJ, 1, 1, f, F);
        }
        df[r] = load8h_raw(p.diff.p, b * p.diff.sB + j * p.diff.sJ, 1, 1, f, F);
        mk[r] = load8m_raw(p.mask.p, b * p.mask.sB + j * p.mask.sJ, 1, 1, f, F);
      }
      s[r] = __half2float(reinterpret_cast<const __half*>(p.istd.p)[b * p.istd.sB + j * p.istd.sJ]);
      off_out[r][0] = b * p.dln.sB + j * p.dln.sJ;
      off_out[r][1] = b * p.dresid.sB + j * p.dresid.sJ;
      off_out[r][2] = b * p.dlin.sB + j * p.dlin.sJ;
    }
    // g = (upstream gradient) * gamma; per-token partial sums of g and g*diff
    float g[kRows][8], d8[kRows][8];
    float part[2 * kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      float sg = 0.f, sgd = 0.f;
      if (active) {
        float a[8], n8[8];
        unpack8(df[r], d8[r]);
        if (MODE == 0) {
          unpack8(in[r][0], a);
          unpack8(in[r][1], n8);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            g[r][e] = a[e] * gm[e];
            if (valid[r]) {
              acc[0][e] = fmaf(a[e], n8[e], acc[0][e]);
              acc[1][e] += a[e];
            }
          }
        } else {
          float r2[8], w8[8], l28[8];
          unpack8(in[r][0], n8);
          unpack8(in[r][1], r2);
          unpack8(in[r][2], w8);
          unpack8(in[r][3], l28);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            a[e] = r2[e] + w8[e];
            g[r][e] = a[e] * gm[e];
            if (valid[r]) {
              acc[0][e] = fmaf(a[e], n8[e], acc[0][e]);
              acc[1][e] += a[e];
              acc[2][e] += l28[e];
            }
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          sg += g[r][e];
          sgd = fmaf(g[r][e], d8[r][e], sgd);
        }
      }
      part[2 * r] = warp_sum(sg);
      part[2 * r + 1] = warp_sum(sgd);
    }
    const int buf = iter & 1;
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < 2 * kRows; ++i) red[group][buf][warp_in_group][i] = part[i];
    }
    group_barrier(group);
#pragma unroll
    for (int i = 0; i < 2 * kRows; ++i)
      part[i] = red[group][buf][0][i] + red[group][buf][1][i] + red[group][buf][2][i] + red[group][buf][3][i];
    if (active) {
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        if (!valid[r]) continue;
        const float c1 = part[2 * r] * s[r] * invn, c2 = part[2 * r + 1] * s[r] * s[r] * s[r] * invn;
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = fmaf(g[r][e], s[r], -c1) - d8[r][e] * c2;
        const uint4 dres = pack8(o);
        const uint4 dl = mask_apply(dres, mk[r]);
        if (p.dln.p) store8h_raw(p.dln.p, off_out[r][0], 1, 1, f, F, pack8(g[r]));
        store8h_raw(p.dresid.p, off_out[r][1], 1, 1, f, F, dres);
        store8h_raw(p.dlin.p, off_out[r][2], 1, 1, f, F, dl);
        if (MODE == 1) {
          float dv[8];
          unpack8(dl, dv);  // the fp16 values just stored: the bias gradient sums exactly them
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[3][e] += dv[e];
        }
      }
    }
  }
  // add the four row groups in order, then one partial row per quantity for this CTA
#pragma unroll
  for (int q = 0; q < NQ; ++q)
#pragma unroll
    for (int e = 0; e < 8; ++e) colred[(group * NQ + q) * kMaxF + f + e] = acc[q][e];
  __syncthreads();
  for (int i = tid; i < NQ * kMaxF; i += kThreads) {
    const int q = i / kMaxF, ff = i % kMaxF;
    float v = 0.f;
#pragma unroll
    for (int gq = 0; gq < kGroups; ++gq) v += colred[(gq * NQ + q) * kMaxF + ff];
    p.partial[((long long)q * gridDim.x + blockIdx.x) * kMaxF + ff] = v;
  }
}

// out[q][f] = sum over the P partial rows in a fixed order: 16 thread groups take every 16th row each (loads
// issued eight at a time, then added in row order) and are combined through shared memory in group order.
constexpr int kFinishParts = 16;
__global__ void __launch_bounds__(64 * kFinishParts)
colsum_finish_kernel(const float* __restrict__ partial, int P, int F, int NQ, void* o0, void* o1, void* o2, void* o3) {
  grid_dependency_sync();
  __shared__ float sm[kFinishParts][64];
  const int q = blockIdx.y;
  const int fl = threadIdx.x & 63, part = threadIdx.x >> 6;
  const int f = blockIdx.x * 64 + fl;
  float v = 0.f;
  if (f < F) {
    const float* base = partial + (long long)q * P * kMaxF + f;
    for (int c0 = part; c0 < P; c0 += 8 * kFinishParts) {
      float x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int c = c0 + u * kFinishParts;
        x[u] = c < P ? __ldcg(base + (long long)c * kMaxF) : 0.f;
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) v += x[u];
    }
  }
  sm[part][fl] = v;
  __syncthreads();
  if (part == 0 && f < F) {
    float total = 0.f;
#pragma unroll
    for (int g = 0; g < kFinishParts; ++g) total += sm[g][fl];
    void* outs[4] = {o0, o1, o2, o3};
    reinterpret_cast<__half*>(outs[q])[f] = __float2half_rn(total);
  }
}

bool eligible(const Dims3& d, std::initializer_list<const View3*> views, const void* gamma) {
  if (d.F > kMaxF || d.F % 8 != 0) return false;
  if ((long long)d.B * d.J > 0x3fffffffLL) return false;
  if (reinterpret_cast<uintptr_t>(gamma) & 15u) return false;
  for (const View3* v : views)
    if (!v->vec) return false;
  return true;
}

template <int MODE>
int launch(cudaStream_t s, void* ws, const LnBwdParams& p0, void* const outs[4]) {
  constexpr int NQ = MODE == 0 ? 2 : 4;
  LnBwdParams p = p0;
  const long long R = (long long)p.d.B * p.d.J;
  const int sms = device_facts().sms;
  const int P = (int)std::max<long long>(1, std::min<long long>(sms, (R + kGroups * kRows - 1) / (kGroups * kRows)));
  if ((size_t)NQ * P * kMaxF * sizeof(float) > kWsBytes - kWsCounterBytes)
    return fail(SB_ERR_UNSUPPORTED, "fused LayerNorm backward: workspace too small");
  p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + kWsCounterBytes);
  const size_t smem = (size_t)kGroups * NQ * kMaxF * sizeof(float);
  SB_CUDA_OK(ensure_dynamic_smem(reinterpret_cast<const void*>(lnbwd_kernel<MODE>), (int)smem));
  SB_LAUNCH_OK(launch_k(lnbwd_kernel<MODE>, P, kThreads, smem, s, p));
  SB_CUDA_OK(cudaGetLastError());
  dim3 grid((p.d.F + 63) / 64, NQ);
  SB_LAUNCH_OK(launch_k(colsum_finish_kernel, grid, 64 * kFinishParts, 0, s, p.partial, P, p.d.F, NQ, outs[0], outs[1], outs[2], outs[3]));
  SB_CUDA_OK(cudaGetLastError());
  return SB_OK;
}

}  // namespace

int launch_lnbwd_a(cudaStream_t s, void* ws, Dims3 d, View3 dy, View3 ln, const void* gamma, View2 istd, View3 diff,
                   View3 mask, View3 dln, View3 dresid, View3 dlin, void* dgamma, void* dbeta) {
  if (!ws) return fail(SB_ERR_ARG, "fused LayerNorm backward called without a workspace");
  if ((long long)d.B * d.J == 0 || d.F == 0) return SB_OK;
  if (!eligible(d, {&dy, &ln, &diff, &mask, &dln, &dresid, &dlin}, gamma))
    return fail(SB_ERR_UNSUPPORTED, "fused LayerNorm backward needs feature-innermost views of at most 1024 features");
  LnBwdParams p{};
  p.d = d; p.y = dy; p.n = ln; p.diff = diff; p.mask = mask; p.istd = istd;
  p.dln = dln; p.dresid = dresid; p.dlin = dlin; p.gamma = gamma;
  void* outs[4] = {dgamma, dbeta, nullptr, nullptr};
  return launch<0>(s, ws, p, outs);
}

int launch_lnbwd_b(cudaStream_t s, void* ws, Dims3 d, View3 ln1, const void* gamma1, View3 dresid2, View3 dlw,
                   View3 dlin2, View2 istd, View3 diff, View3 mask, View3 dln1, View3 dresid1, View3 datt,
                   void* dgamma1, void* dbeta1, void* dlinb2, void* dbo) {
  if (!ws) return fail(SB_ERR_ARG, "fused LayerNorm backward called without a workspace");
  if ((long long)d.B * d.J == 0 || d.F == 0) return SB_OK;
  if (!eligible(d, {&ln1, &dresid2, &dlw, &dlin2, &diff, &mask, &dln1, &dresid1, &datt}, gamma1))
    return fail(SB_ERR_UNSUPPORTED, "fused LayerNorm backward needs feature-innermost views of at most 1024 features");
  LnBwdParams p{};
  p.d = d; p.n = ln1; p.r2 = dresid2; p.w = dlw; p.l2 = dlin2; p.diff = diff; p.mask = mask; p.istd = istd;
  p.dln = dln1; p.dresid = dresid1; p.dlin = datt; p.gamma = gamma1;
  void* outs[4] = {dgamma1, dbeta1, dlinb2, dbo};
  return launch<1>(s, ws, p, outs);
}

}  // namespace sb
