// Memory-bound fused operators of the encoder layer, written for sm_100a.
//
// Common structure: a warp owns one row (token, or attention row) at a time and
// its lanes walk the row's innermost logical dim in 128-bit groups, so a row is
// read once into registers, reduced with warp shuffles and written once.  Every
// tensor is addressed through its own strides; a tensor whose innermost dim is
// not contiguous falls back to scalar accesses inside the same kernel.
// Reductions over tokens (parameter gradients) use per-CTA fp32 partial sums in
// a workspace and a ticket counter: the last CTA of a feature slice adds the
// partials in a fixed order, so results are deterministic and need one launch.

#include <math.h>

#include <algorithm>
#include <mutex>

#include "ops.h"

namespace sb {

namespace {

constexpr int kRowThreads = 128;  // 4 warps per CTA for the row kernels
constexpr int kColThreads = 256;  // 8 warps per CTA for the token-reduction kernels

// AV ("all vector") is a compile-time promise that every view of the launch takes the 128-bit
// path, which removes the per-access branch so that a row's loads issue back to back.
#define SB_VEC(view) (AV || (view).vec)

// Keep flags of logical elements e0..e0+7; under AV the extent is a multiple of 8, so e0 is group aligned.
template <bool AV>
__device__ __forceinline__ void philox8(const Rng& r, unsigned long long e0, uint32_t m[8]) {
  if (AV) philox_keep8(r, e0 >> 3, m);
  else philox_keep8_unaligned(r, e0, m);
}

__device__ __forceinline__ float act_bwd(float x, float dy, int activation) {
  if (activation == SB_ACT_RELU) return x > 0.f ? dy : 0.f;
  const float x3 = x * x * x;
  const float inner = 0.0356774f * x3 + 0.797885f * x;
  const float th = tanhf(inner);
  const float sech2 = 1.f - th * th;
  return (0.5f * th + (0.0535161f * x3 + 0.398942f * x) * sech2 + 0.5f) * dy;
}

__device__ __forceinline__ uint4 hmul8(const uint4& a, const uint4& b) {
  uint4 o;
  const sb_half2* x = reinterpret_cast<const sb_half2*>(&a);
  const sb_half2* y = reinterpret_cast<const sb_half2*>(&b);
  sb_half2* q = reinterpret_cast<sb_half2*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) q[i] = __hmul2(x[i], y[i]);
  return o;
}

// ---------------------------------------------------------------------------
// Softmax (+scale, +dropout) forward and backward over [H,B,J,K].
// LPR lanes cooperate on one row, each holding NV groups of eight elements.
// Persistent: a warp walks row groups with a grid stride and keeps ROWS rows in
// flight (all of their loads are issued before the first is consumed); loaded
// data stays packed (uint4 / uint2) until it is used.
// ---------------------------------------------------------------------------
constexpr int kSmThreads = 256;

struct RowPos4 {
  long long o_a, o_b, o_c, o_d;  // element offsets of the row in up to four views
  unsigned row;
  bool valid;
};
__device__ __forceinline__ RowPos4 row_pos4(const Dims4& d, unsigned row, unsigned R, const View4& a,
                                            const View4& b, const View4& c, const View4& e) {
  RowPos4 p;
  p.valid = row < R;
  p.row = p.valid ? row : R - 1;
  const unsigned j = p.row % (unsigned)d.J, hb = p.row / (unsigned)d.J;
  const unsigned bb = hb % (unsigned)d.B, h = hb / (unsigned)d.B;
  p.o_a = h * a.sH + bb * a.sB + j * a.sJ;
  p.o_b = h * b.sH + bb * b.sB + j * b.sJ;
  p.o_c = h * c.sH + bb * c.sB + j * c.sJ;
  p.o_d = h * e.sH + bb * e.sB + j * e.sJ;
  return p;
}

template <int LPR, int NV, int ROWS, bool AV>
__global__ void __launch_bounds__(kSmThreads, (NV * ROWS <= 4) ? 4 : 1)
softmax_fwd_kernel(Dims4 d, View4 beta, View4 alpha, View4 mask, View4 drop, float scale, Rng rng,
                   unsigned R, unsigned ngroups) {
  grid_dependency_sync();
  constexpr int RPW = kWarp / LPR;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / LPR, sl = lane % LPR;
  const unsigned nwarps = gridDim.x * (kSmThreads / kWarp);
  const float c2 = scale * 1.4426950408889634f;
  for (unsigned g = blockIdx.x * (kSmThreads / kWarp) + warp; g < ngroups; g += nwarps) {
    RowPos4 pos[ROWS];
    uint4 xr[ROWS][NV];
    uint2 mr[ROWS][NV];
#pragma unroll
    for (int rr = 0; rr < ROWS; ++rr) {
      pos[rr] = row_pos4(d, (g * ROWS + rr) * RPW + sub, R, beta, alpha, mask, drop);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int k = (sl + LPR * i) * 8;
        if (k < d.K) {
          xr[rr][i] = load8h_raw(beta.p, pos[rr].o_a, beta.sK, SB_VEC(beta), k, d.K);
          if (!rng.philox) mr[rr][i] = load8m_raw(mask.p, pos[rr].o_c, mask.sK, SB_VEC(mask), k, d.K);
        }
      }
    }
#pragma unroll
    for (int rr = 0; rr < ROWS; ++rr) {
      // t = x * (scale * log2 e); softmax = 2^(t - max t) / sum
      float x[NV][8];
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int k = (sl + LPR * i) * 8;
        unpack8(xr[rr][i], x[i]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const bool in = AV ? (k < d.K) : (k + e < d.K);
          x[i][e] = in ? x[i][e] * c2 : -INFINITY;
          mx = fmaxf(mx, x[i][e]);
        }
      }
      mx = group_max<LPR>(mx);
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          x[i][e] = exp2f(x[i][e] - mx);
          sum += x[i][e];
        }
      sum = group_sum<LPR>(sum);
      const float inv = 1.f / sum;
      if (!pos[rr].valid) continue;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int k = (sl + LPR * i) * 8;
        if (k >= d.K) continue;
        uint2 m = mr[rr][i];
        if (rng.philox) {
          uint32_t mm[8];
          philox8<AV>(rng, (unsigned long long)pos[rr].row * d.K + k, mm);
          m = mask_pack(mm);
          store8m_raw(mask.p, pos[rr].o_c, mask.sK, SB_VEC(mask), k, d.K, m);
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) x[i][e] *= inv;
        const uint4 a = pack8(x[i]);
        store8h_raw(alpha.p, pos[rr].o_b, alpha.sK, SB_VEC(alpha), k, d.K, a);
        store8h_raw(drop.p, pos[rr].o_d, drop.sK, SB_VEC(drop), k, d.K, mask_apply(a, m));
      }
    }
  }
}

template <int LPR, int NV, int ROWS, bool AV>
__global__ void __launch_bounds__(kSmThreads, (NV * ROWS <= 4) ? 4 : 1)
softmax_bwd_kernel(Dims4 d, View4 alpha, View4 mask, View4 dad, View4 dbeta, unsigned R, unsigned ngroups) {
  grid_dependency_sync();
  constexpr int RPW = kWarp / LPR;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / LPR, sl = lane % LPR;
  const unsigned nwarps = gridDim.x * (kSmThreads / kWarp);
  for (unsigned g = blockIdx.x * (kSmThreads / kWarp) + warp; g < ngroups; g += nwarps) {
    RowPos4 pos[ROWS];
    uint4 ar[ROWS][NV], gr[ROWS][NV];
    uint2 mr[ROWS][NV];
#pragma unroll
    for (int rr = 0; rr < ROWS; ++rr) {
      pos[rr] = row_pos4(d, (g * ROWS + rr) * RPW + sub, R, alpha, mask, dad, dbeta);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int k = (sl + LPR * i) * 8;
        if (k < d.K) {
          ar[rr][i] = load8h_raw(alpha.p, pos[rr].o_a, alpha.sK, SB_VEC(alpha), k, d.K);
          gr[rr][i] = load8h_raw(dad.p, pos[rr].o_c, dad.sK, SB_VEC(dad), k, d.K);
          mr[rr][i] = load8m_raw(mask.p, pos[rr].o_b, mask.sK, SB_VEC(mask), k, d.K);
        } else {
          ar[rr][i] = make_uint4(0, 0, 0, 0);
          gr[rr][i] = make_uint4(0, 0, 0, 0);
          mr[rr][i] = make_uint2(0, 0);
        }
      }
    }
#pragma unroll
    for (int rr = 0; rr < ROWS; ++rr) {
      float a[NV][8], gg[NV][8];
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        unpack8(ar[rr][i], a[i]);
        unpack8(gr[rr][i], gg[i]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          gg[i][e] = mask_keep(mr[rr][i], e) ? gg[i][e] : 0.f;
          s += gg[i][e] * a[i][e];
        }
      }
      s = group_sum<LPR>(s);
      if (!pos[rr].valid) continue;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int k = (sl + LPR * i) * 8;
        if (k >= d.K) continue;
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = a[i][e] * (gg[i][e] - s);
        store8h_raw(dbeta.p, pos[rr].o_d, dbeta.sK, SB_VEC(dbeta), k, d.K, pack8(o));
      }
    }
  }
}

// ---------------------------------------------------------------------------
// bias + dropout + residual + LayerNorm over [B,J,F]; one warp per token, persistent
// grid-stride over tokens, a token's inputs stay packed until they are consumed.
// ---------------------------------------------------------------------------
template <int NV, bool AV>
__global__ void __launch_bounds__(kSmThreads, NV <= 2 ? 3 : (NV <= 4 ? 2 : 1))
bdrln_kernel(Dims3 d, View3 in, const void* bias, View3 resid, const void* gamma, const void* beta,
             View3 mask, View3 lin, View3 diff, View2 istd, View3 ln, View3 out, Rng rng, int pvec) {
  grid_dependency_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned R = (unsigned)d.B * (unsigned)d.J;
  const unsigned nwarps = gridDim.x * (kSmThreads / kWarp);
  const float invF = 1.f / (float)d.F;
  for (unsigned row = blockIdx.x * (kSmThreads / kWarp) + warp; row < R; row += nwarps) {
    const int b = (int)(row / (unsigned)d.J), j = (int)(row % (unsigned)d.J);
    const long long o_in = b * in.sB + j * in.sJ, o_res = b * resid.sB + j * resid.sJ;
    const long long o_mask = b * mask.sB + j * mask.sJ, o_lin = b * lin.sB + j * lin.sJ;
    uint4 xr[NV], rr[NV];
    uint2 mr[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int f = (lane + kWarp * i) * 8;
      if (f < d.F) {
        xr[i] = load8h_raw(in.p, o_in, in.sF, SB_VEC(in), f, d.F);
        rr[i] = load8h_raw(resid.p, o_res, resid.sF, SB_VEC(resid), f, d.F);
        if (!rng.philox) mr[i] = load8m_raw(mask.p, o_mask, mask.sF, SB_VEC(mask), f, d.F);
      }
    }
    float r[NV][8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int f = (lane + kWarp * i) * 8;
      if (f < d.F) {
        if (rng.philox) {
          uint32_t mm[8];
          philox8<AV>(rng, (unsigned long long)row * d.F + f, mm);
          mr[i] = mask_pack(mm);
          store8m_raw(mask.p, o_mask, mask.sF, SB_VEC(mask), f, d.F, mr[i]);
        }
        const uint4 bs = load8h_raw(bias, 0, 1, AV || pvec, f, d.F);
        float x[8], bb[8], rs[8];
        unpack8(xr[i], x);
        unpack8(bs, bb);
        unpack8(rr[i], rs);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] += bb[e];
        if (lin.p) store8h_raw(lin.p, o_lin, lin.sF, SB_VEC(lin), f, d.F, pack8(x));  // null: the caller does not want it
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          r[i][e] = (AV || f + e < d.F) ? (mask_keep(mr[i], e) ? x[e] : 0.f) + rs[e] : 0.f;
          sum += r[i][e];
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) r[i][e] = 0.f;
      }
    }
    const float mean = warp_sum(sum) * invF;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int f = (lane + kWarp * i) * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        r[i][e] = (f + e < d.F) ? r[i][e] - mean : 0.f;
        sq = fmaf(r[i][e], r[i][e], sq);
      }
    }
    const float rstd = rsqrtf(warp_sum(sq) * invF + kLnEps);
    if (lane == 0) reinterpret_cast<sb_half*>(istd.p)[b * istd.sB + j * istd.sJ] = sb_f2h(rstd);
    const long long o_diff = b * diff.sB + j * diff.sJ, o_ln = b * ln.sB + j * ln.sJ;
    const long long o_out = b * out.sB + j * out.sJ;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int f = (lane + kWarp * i) * 8;
      if (f >= d.F) continue;
      float gm[8], bt[8], n[8], o[8];
      unpack8(load8h_raw(gamma, 0, 1, AV || pvec, f, d.F), gm);
      unpack8(load8h_raw(beta, 0, 1, AV || pvec, f, d.F), bt);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        n[e] = r[i][e] * rstd;
        o[e] = fmaf(n[e], gm[e], bt[e]);
      }
      store8h_raw(diff.p, o_diff, diff.sF, SB_VEC(diff), f, d.F, pack8(r[i]));
      store8h_raw(ln.p, o_ln, ln.sF, SB_VEC(ln), f, d.F, pack8(n));
      store8h_raw(out.p, o_out, out.sF, SB_VEC(out), f, d.F, pack8(o));
    }
  }
}

// LayerNorm backward-data + dropout backward; one warp per token, persistent.
template <int NV, bool AV>
__global__ void __launch_bounds__(kSmThreads, NV <= 2 ? 3 : (NV <= 4 ? 2 : 1))
blnrd_kernel(Dims3 d, View3 dln, View2 istd, View3 diff, View3 mask, View3 dresid, View3 dlin) {
  grid_dependency_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned R = (unsigned)d.B * (unsigned)d.J;
  const unsigned nwarps = gridDim.x * (kSmThreads / kWarp);
  const float invn = 1.f / (float)d.F;
  for (unsigned row = blockIdx.x * (kSmThreads / kWarp) + warp; row < R; row += nwarps) {
    const int b = (int)(row / (unsigned)d.J), j = (int)(row % (unsigned)d.J);
    const long long o_g = b * dln.sB + j * dln.sJ, o_d = b * diff.sB + j * diff.sJ;
    const long long o_m = b * mask.sB + j * mask.sJ;
    uint4 gr[NV], dr_[NV];
    uint2 mr[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int f = (lane + kWarp * i) * 8;
      if (f < d.F) {
        gr[i] = load8h_raw(dln.p, o_g, dln.sF, SB_VEC(dln), f, d.F);
        dr_[i] = load8h_raw(diff.p, o_d, diff.sF, SB_VEC(diff), f, d.F);
        mr[i] = load8m_raw(mask.p, o_m, mask.sF, SB_VEC(mask), f, d.F);
      } else {
        gr[i] = make_uint4(0, 0, 0, 0);
        dr_[i] = make_uint4(0, 0, 0, 0);
        mr[i] = make_uint2(0, 0);
      }
    }
    const float s = sb_h2f(reinterpret_cast<const sb_half*>(istd.p)[b * istd.sB + j * istd.sJ]);
    float sg = 0.f, sgd = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      float g[8], df[8];
      unpack8(gr[i], g);
      unpack8(dr_[i], df);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        sg += g[e];
        sgd = fmaf(g[e], df[e], sgd);
      }
    }
    sg = warp_sum(sg);
    sgd = warp_sum(sgd);
    const float c1 = sg * s * invn, c2 = sgd * s * s * s * invn;
    const long long o_r = b * dresid.sB + j * dresid.sJ, o_l = b * dlin.sB + j * dlin.sJ;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int f = (lane + kWarp * i) * 8;
      if (f >= d.F) continue;
      float g[8], df[8], o[8];
      unpack8(gr[i], g);
      unpack8(dr_[i], df);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = fmaf(g[e], s, -c1) - df[e] * c2;
      const uint4 packed = pack8(o);
      store8h_raw(dresid.p, o_r, dresid.sF, SB_VEC(dresid), f, d.F, packed);
      store8h_raw(dlin.p, o_l, dlin.sF, SB_VEC(dlin), f, d.F, mask_apply(packed, mr[i]));
    }
  }
}

// ---------------------------------------------------------------------------
// Elementwise kernels.  Flat form: every tensor is dense in logical order, so element i of one
// is element i of all; a thread takes UNR groups of eight, a grid stride apart (persistent).
// Row form: strided views, a warp takes one token and a span of 4 * 256 features.
// ---------------------------------------------------------------------------
constexpr int kEwNV = 4;
constexpr int kFlatUnr = 4;

template <int ACT>
__global__ void __launch_bounds__(kSmThreads, 4)
bad_flat_kernel(unsigned long long ngroups, int groups_per_row, const uint4* __restrict__ in,
                const uint4* __restrict__ bias, uint2* mask, uint4* __restrict__ lin1,
                uint4* __restrict__ drop2, Rng rng) {
  grid_dependency_sync();
  const unsigned long long stride = (unsigned long long)gridDim.x * kSmThreads;
  for (unsigned long long g0 = (unsigned long long)blockIdx.x * kSmThreads + threadIdx.x; g0 < ngroups;
       g0 += stride * kFlatUnr) {
    uint4 x[kFlatUnr];
    uint2 m[kFlatUnr];
#pragma unroll
    for (int u = 0; u < kFlatUnr; ++u) {
      const unsigned long long g = g0 + u * stride;
      if (g < ngroups) {
        x[u] = in[g];
        if (!rng.philox) m[u] = mask[g];
      }
    }
#pragma unroll
    for (int u = 0; u < kFlatUnr; ++u) {
      const unsigned long long g = g0 + u * stride;
      if (g >= ngroups) continue;
      if (rng.philox) {
        uint32_t mm[8];
        philox_keep8(rng, g, mm);
        m[u] = mask_pack(mm);
        mask[g] = m[u];
      }
      const uint4 l = hadd8(x[u], bias[g % (unsigned)groups_per_row]);
      lin1[g] = l;
      uint4 a;
      if (ACT == SB_ACT_RELU) {
        const sb_half2* h = reinterpret_cast<const sb_half2*>(&l);
        sb_half2* q = reinterpret_cast<sb_half2*>(&a);
        const sb_half2 zero = sb_f2h2_dup(0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i) q[i] = __hmax2(h[i], zero);
      } else {
        float v[8];
        unpack8(l, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = act_fwd(v[e], SB_ACT_GELU);
        a = pack8(v);
      }
      drop2[g] = mask_apply(a, m[u]);
    }
  }
}

__global__ void __launch_bounds__(kSmThreads, 4)
add_flat_kernel(unsigned long long ngroups, const uint4* __restrict__ a, const uint4* __restrict__ b,
                uint4* __restrict__ out) {
  grid_dependency_sync();
  const unsigned long long stride = (unsigned long long)gridDim.x * kSmThreads;
  for (unsigned long long g0 = (unsigned long long)blockIdx.x * kSmThreads + threadIdx.x; g0 < ngroups;
       g0 += stride * kFlatUnr) {
    uint4 x[kFlatUnr], y[kFlatUnr];
#pragma unroll
    for (int u = 0; u < kFlatUnr; ++u) {
      const unsigned long long g = g0 + u * stride;
      if (g < ngroups) { x[u] = a[g]; y[u] = b[g]; }
    }
#pragma unroll
    for (int u = 0; u < kFlatUnr; ++u) {
      const unsigned long long g = g0 + u * stride;
      if (g < ngroups) out[g] = hadd8(x[u], y[u]);
    }
  }
}

// out[r, :] = in[r, :] + bias[r] over dense rows of `groups_per_row` groups of eight
__global__ void __launch_bounds__(kSmThreads, 4)
rowbias_flat_kernel(unsigned long long ngroups, unsigned groups_per_row, const uint4* __restrict__ in,
                    const sb_half* __restrict__ bias, uint4* __restrict__ out) {
  grid_dependency_sync();
  const unsigned long long stride = (unsigned long long)gridDim.x * kSmThreads;
  for (unsigned long long g0 = (unsigned long long)blockIdx.x * kSmThreads + threadIdx.x; g0 < ngroups;
       g0 += stride * kFlatUnr) {
    uint4 x[kFlatUnr];
    sb_half bv[kFlatUnr];
#pragma unroll
    for (int u = 0; u < kFlatUnr; ++u) {
      const unsigned long long g = g0 + u * stride;
      if (g < ngroups) { x[u] = in[g]; bv[u] = bias[g / groups_per_row]; }
    }
#pragma unroll
    for (int u = 0; u < kFlatUnr; ++u) {
      const unsigned long long g = g0 + u * stride;
      if (g >= ngroups) continue;
      const sb_half2 b2 = sb_h2h2(bv[u]);
      uint4 o;
      const sb_half2* h = reinterpret_cast<const sb_half2*>(&x[u]);
      sb_half2* q = reinterpret_cast<sb_half2*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) q[i] = __hadd2(h[i], b2);
      out[g] = o;
    }
  }
}

template <bool AV>
__global__ void __launch_bounds__(kRowThreads)
bad_kernel(Dims3 d, int spans, View3 in, const void* bias, View3 mask, View3 lin1, View3 drop2,
           int activation, Rng rng, int pvec) {
  grid_dependency_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long R = (long long)d.B * d.J;
  const long long item = (long long)blockIdx.x * (kRowThreads / kWarp) + warp;
  if (item >= R * spans) return;
  const long long row = item / spans;
  const int span = (int)(item % spans);
  const int b = (int)(row / d.J), j = (int)(row % d.J);
  const long long o_in = b * in.sB + j * in.sJ, o_m = b * mask.sB + j * mask.sJ;
  const long long o_l = b * lin1.sB + j * lin1.sJ, o_d = b * drop2.sB + j * drop2.sJ;
  float x[kEwNV][8];
  uint32_t m[kEwNV][8];
#pragma unroll
  for (int i = 0; i < kEwNV; ++i) {
    const int f = span * (kEwNV * 256) + (lane + kWarp * i) * 8;
    if (f < d.F) {
      load8h(in.p, o_in, in.sF, SB_VEC(in), f, d.F, x[i]);
      if (!rng.philox) load8m(mask.p, o_m, mask.sF, SB_VEC(mask), f, d.F, m[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < kEwNV; ++i) {
    const int f = span * (kEwNV * 256) + (lane + kWarp * i) * 8;
    if (f >= d.F) continue;
    float bs[8], o[8];
    load8p(bias, f, d.F, AV || pvec, bs);
    if (rng.philox) {
      philox8<AV>(rng, (unsigned long long)row * d.F + f, m[i]);
      store8m(mask.p, o_m, mask.sF, SB_VEC(mask), f, d.F, m[i]);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      x[i][e] += bs[e];
      o[e] = m[i][e] ? act_fwd(x[i][e], activation) : 0.f;
    }
    store8h(lin1.p, o_l, lin1.sF, SB_VEC(lin1), f, d.F, x[i]);
    store8h(drop2.p, o_d, drop2.sF, SB_VEC(drop2), f, d.F, o);
  }
}

template <bool AV>
__global__ void __launch_bounds__(kRowThreads)
bei_kernel(Dims3 d, int spans, View3 a, View3 b_, View3 out) {
  grid_dependency_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long R = (long long)d.B * d.J;
  const long long item = (long long)blockIdx.x * (kRowThreads / kWarp) + warp;
  if (item >= R * spans) return;
  const long long row = item / spans;
  const int span = (int)(item % spans);
  const int b = (int)(row / d.J), j = (int)(row % d.J);
  const long long o_a = b * a.sB + j * a.sJ, o_b = b * b_.sB + j * b_.sJ;
  const long long o_o = b * out.sB + j * out.sJ;
  float x[kEwNV][8], y[kEwNV][8];
#pragma unroll
  for (int i = 0; i < kEwNV; ++i) {
    const int f = span * (kEwNV * 256) + (lane + kWarp * i) * 8;
    if (f < d.F) {
      load8h(a.p, o_a, a.sF, SB_VEC(a), f, d.F, x[i]);
      load8h(b_.p, o_b, b_.sF, SB_VEC(b_), f, d.F, y[i]);
    }
  }
#pragma unroll
  for (int i = 0; i < kEwNV; ++i) {
    const int f = span * (kEwNV * 256) + (lane + kWarp * i) * 8;
    if (f >= d.F) continue;
#pragma unroll
    for (int e = 0; e < 8; ++e) x[i][e] += y[i][e];
    store8h(out.p, o_o, out.sF, SB_VEC(out), f, d.F, x[i]);
  }
}

// out[n,p,h,b,j] = in[n,p,h,b,j] + bias[n,p,h]; a warp takes one (n,p,h,b) row and a span of J.
template <bool AV>
__global__ void __launch_bounds__(kRowThreads)
aib_kernel(Dims5 d, int spans, View5 in, const void* bias, long long bsN, long long bsP,
           long long bsH, View5 out) {
  grid_dependency_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const long long R = (long long)d.N * d.P * d.H * d.B;
  const long long item = (long long)blockIdx.x * (kRowThreads / kWarp) + warp;
  if (item >= R * spans) return;
  long long row = item / spans;
  const int span = (int)(item % spans);
  const int b = (int)(row % d.B); row /= d.B;
  const int h = (int)(row % d.H); row /= d.H;
  const int p = (int)(row % d.P);
  const int n = (int)(row / d.P);
  const long long o_in = n * in.sN + p * in.sP + h * in.sH + b * in.sB;
  const long long o_out = n * out.sN + p * out.sP + h * out.sH + b * out.sB;
  const float bv = sb_h2f(reinterpret_cast<const sb_half*>(bias)[n * bsN + p * bsP + h * bsH]);
  float x[kEwNV][8];
#pragma unroll
  for (int i = 0; i < kEwNV; ++i) {
    const int f = span * (kEwNV * 256) + (lane + kWarp * i) * 8;
    if (f < d.J) load8h(in.p, o_in, in.sJ, SB_VEC(in), f, d.J, x[i]);
  }
#pragma unroll
  for (int i = 0; i < kEwNV; ++i) {
    const int f = span * (kEwNV * 256) + (lane + kWarp * i) * 8;
    if (f >= d.J) continue;
#pragma unroll
    for (int e = 0; e < 8; ++e) x[i][e] += bv;
    store8h(out.p, o_out, out.sJ, SB_VEC(out), f, d.J, x[i]);
  }
}

// Dense rows: out[r] = sum of the `groups` groups of eight of row r; one warp per row, eight
// 128-bit loads in flight per lane.
__global__ void __launch_bounds__(kSmThreads)
rowsum_flat_kernel(unsigned rows, unsigned groups, const uint4* __restrict__ in, sb_half* __restrict__ out) {
  grid_dependency_sync();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned nwarps = gridDim.x * (kSmThreads / kWarp);
  for (unsigned r = blockIdx.x * (kSmThreads / kWarp) + warp; r < rows; r += nwarps) {
    const uint4* p = in + (unsigned long long)r * groups;
    float acc = 0.f;
    for (unsigned g0 = lane; g0 < groups; g0 += kWarp * 8) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const unsigned g = g0 + u * kWarp;
        v[u] = g < groups ? p[g] : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        float x[8];
        unpack8(v[u], x);
#pragma unroll
        for (int e = 0; e < 8; ++e) acc += x[e];
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) out[r] = sb_f2h(acc);
  }
}

// dbias[n,p,h] = sum_{b,j} in[n,p,h,b,j]; one CTA per output element.
template <bool AV>
__global__ void __launch_bounds__(kColThreads)
baib_kernel(Dims5 d, View5 in, void* dbias, long long bsN, long long bsP, long long bsH) {
  grid_dependency_sync();
  long long row = blockIdx.x;
  const int h = (int)(row % d.H); row /= d.H;
  const int p = (int)(row % d.P);
  const int n = (int)(row / d.P);
  const long long base = n * in.sN + p * in.sP + h * in.sH;
  const int groups = (d.J + 7) / 8;
  float acc = 0.f;
  for (long long idx = threadIdx.x; idx < (long long)d.B * groups; idx += kColThreads) {
    const int b = (int)(idx / groups);
    const int f = (int)(idx % groups) * 8;
    float x[8];
    load8h(in.p, base + b * in.sB, in.sJ, SB_VEC(in), f, d.J, x);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc += x[e];
  }
  acc = warp_sum(acc);
  __shared__ float sm[kColThreads / kWarp];
  if ((threadIdx.x & 31) == 0) sm[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < kColThreads / kWarp; ++w) s += sm[w];
    reinterpret_cast<sb_half*>(dbias)[n * bsN + p * bsP + h * bsH] = sb_f2h(s);
  }
}

// ---------------------------------------------------------------------------
// Token reductions fused with elementwise work.
// grid = (feature slices of 256, row chunks); see file header for the scheme.
// ---------------------------------------------------------------------------
template <int NQ>
struct ColOut {
  void* out[NQ];  // fp16 [F], unit stride
};

// Each operator supplies: NQ reduced quantities, NIN fp16 inputs per row, UNR rows kept in
// flight per warp, load<AV>() of one row's eight features (kept packed) and finish<AV>() =
// elementwise output + accumulation.
template <int NIN>
struct RowRegs {
  uint4 v[NIN];
  uint2 m;
};

struct BsbOp {
  static constexpr int NQ = 2, NIN = 2, UNR = 4, MINB = 3;
  View3 dy, ln, dln;
  const void* gamma;
  int pvec;
  template <bool AV>
  __device__ __forceinline__ void load(int b, int j, int f, int F, RowRegs<NIN>& r) const {
    r.v[0] = load8h_raw(dy.p, b * dy.sB + j * dy.sJ, dy.sF, SB_VEC(dy), f, F);
    r.v[1] = load8h_raw(ln.p, b * ln.sB + j * ln.sJ, ln.sF, SB_VEC(ln), f, F);
  }
  template <bool AV>
  __device__ __forceinline__ void finish(int b, int j, int f, int F, const uint4& gm,
                                         const RowRegs<NIN>& r, float acc[NQ][8]) const {
    float y[8], n[8];
    unpack8(r.v[0], y);
    unpack8(r.v[1], n);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      acc[0][e] = fmaf(y[e], n[e], acc[0][e]);
      acc[1][e] += y[e];
    }
    // a product of two fp16 values is exact in fp32, so one half-precision multiply rounds the same
    store8h_raw(dln.p, b * dln.sB + j * dln.sJ, dln.sF, SB_VEC(dln), f, F, hmul8(r.v[0], gm));
  }
  template <bool AV>
  __device__ __forceinline__ uint4 scale(int f, int F) const { return load8h_raw(gamma, 0, 1, AV || pvec, f, F); }
};

struct EbsbOp {
  static constexpr int NQ = 3, NIN = 4, UNR = 2, MINB = 3;
  View3 ln1, dresid2, dlw, dlin2, dln1;
  const void* gamma;
  int pvec;
  template <bool AV>
  __device__ __forceinline__ void load(int b, int j, int f, int F, RowRegs<NIN>& r) const {
    r.v[0] = load8h_raw(ln1.p, b * ln1.sB + j * ln1.sJ, ln1.sF, SB_VEC(ln1), f, F);
    r.v[1] = load8h_raw(dresid2.p, b * dresid2.sB + j * dresid2.sJ, dresid2.sF, SB_VEC(dresid2), f, F);
    r.v[2] = load8h_raw(dlw.p, b * dlw.sB + j * dlw.sJ, dlw.sF, SB_VEC(dlw), f, F);
    r.v[3] = load8h_raw(dlin2.p, b * dlin2.sB + j * dlin2.sJ, dlin2.sF, SB_VEC(dlin2), f, F);
  }
  template <bool AV>
  __device__ __forceinline__ void finish(int b, int j, int f, int F, const uint4& gm,
                                         const RowRegs<NIN>& r, float acc[NQ][8]) const {
    float n[8], rr[8], w[8], l2[8], g8[8], o[8];
    unpack8(r.v[0], n);
    unpack8(r.v[1], rr);
    unpack8(r.v[2], w);
    unpack8(r.v[3], l2);
    unpack8(gm, g8);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float g = rr[e] + w[e];
      o[e] = g * g8[e];
      acc[0][e] = fmaf(g, n[e], acc[0][e]);
      acc[1][e] += g;
      acc[2][e] += l2[e];
    }
    store8h_raw(dln1.p, b * dln1.sB + j * dln1.sJ, dln1.sF, SB_VEC(dln1), f, F, pack8(o));
  }
  template <bool AV>
  __device__ __forceinline__ uint4 scale(int f, int F) const { return load8h_raw(gamma, 0, 1, AV || pvec, f, F); }
};

struct BdrlbOp {
  static constexpr int NQ = 1, NIN = 2, UNR = 4, MINB = 4;
  View3 ddrop2, mask, lin1, dlin1;
  int activation;
  template <bool AV>
  __device__ __forceinline__ void load(int b, int j, int f, int F, RowRegs<NIN>& r) const {
    r.v[0] = load8h_raw(ddrop2.p, b * ddrop2.sB + j * ddrop2.sJ, ddrop2.sF, SB_VEC(ddrop2), f, F);
    r.v[1] = load8h_raw(lin1.p, b * lin1.sB + j * lin1.sJ, lin1.sF, SB_VEC(lin1), f, F);
    r.m = load8m_raw(mask.p, b * mask.sB + j * mask.sJ, mask.sF, SB_VEC(mask), f, F);
  }
  template <bool AV>
  __device__ __forceinline__ void finish(int b, int j, int f, int F, const uint4&,
                                         const RowRegs<NIN>& r, float acc[NQ][8]) const {
    uint4 out;
    float o[8];
    if (activation == SB_ACT_RELU) {
      // dlin1 = [lin1 > 0] * mask * ddrop2, all exact selections of fp16 values
      const uint4 g = mask_apply(r.v[0], r.m);
      const sb_half2* x = reinterpret_cast<const sb_half2*>(&r.v[1]);
      const sb_half2* gg = reinterpret_cast<const sb_half2*>(&g);
      sb_half2* q = reinterpret_cast<sb_half2*>(&out);
      const sb_half2 zero = sb_f2h2_dup(0.f);
#pragma unroll
      for (int i = 0; i < 4; ++i) q[i] = __hmul2(gg[i], __hgt2(x[i], zero));
      unpack8(out, o);
    } else {
      float g[8], x[8];
      unpack8(r.v[0], g);
      unpack8(r.v[1], x);
#pragma unroll
      for (int e = 0; e < 8; ++e) o[e] = act_bwd(x[e], mask_keep(r.m, e) ? g[e] : 0.f, activation);
      out = pack8(o);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[0][e] += (AV || f + e < F) ? o[e] : 0.f;
    store8h_raw(dlin1.p, b * dlin1.sB + j * dlin1.sJ, dlin1.sF, SB_VEC(dlin1), f, F, out);
  }
  template <bool AV>
  __device__ __forceinline__ uint4 scale(int, int) const { return make_uint4(0, 0, 0, 0); }
};

struct BaobOp {
  static constexpr int NQ = 1, NIN = 1, UNR = 8, MINB = 4;
  View3 datt;
  template <bool AV>
  __device__ __forceinline__ void load(int b, int j, int f, int F, RowRegs<NIN>& r) const {
    r.v[0] = load8h_raw(datt.p, b * datt.sB + j * datt.sJ, datt.sF, SB_VEC(datt), f, F);
  }
  template <bool AV>
  __device__ __forceinline__ void finish(int, int, int, int, const uint4&, const RowRegs<NIN>& r,
                                         float acc[NQ][8]) const {
    float x[8];
    unpack8(r.v[0], x);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[0][e] += x[e];
  }
  template <bool AV>
  __device__ __forceinline__ uint4 scale(int, int) const { return make_uint4(0, 0, 0, 0); }
};

template <class Op, bool AV>
__global__ void __launch_bounds__(kColThreads, Op::MINB)
colreduce_kernel(Op op, Dims3 d, int rows_per_chunk, float* partial, unsigned* counters,
                 ColOut<Op::NQ> outs) {
  grid_dependency_sync();
  constexpr int NQ = Op::NQ;
  constexpr int NW = kColThreads / kWarp;
  constexpr int UNR = Op::UNR;  // rows in flight per warp
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slice = blockIdx.x, chunk = blockIdx.y, P = gridDim.y;
  const int Fp = gridDim.x * 256;
  const int f = slice * 256 + lane * 8;
  const unsigned R = (unsigned)d.B * (unsigned)d.J;
  const unsigned r0 = (unsigned)chunk * (unsigned)rows_per_chunk;
  const unsigned r1 = (r0 + rows_per_chunk < R) ? r0 + rows_per_chunk : R;

  float acc[NQ][8];
#pragma unroll
  for (int q = 0; q < NQ; ++q)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[q][e] = 0.f;
  if (f < d.F) {
    const uint4 gm = op.template scale<AV>(f, d.F);
    for (unsigned r = r0 + warp; r < r1; r += NW * UNR) {
      RowRegs<Op::NIN> regs[UNR];
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const unsigned rr = r + u * NW;
        if (rr < r1) op.template load<AV>((int)(rr / (unsigned)d.J), (int)(rr % (unsigned)d.J), f, d.F, regs[u]);
      }
#pragma unroll
      for (int u = 0; u < UNR; ++u) {
        const unsigned rr = r + u * NW;
        if (rr < r1) op.template finish<AV>((int)(rr / (unsigned)d.J), (int)(rr % (unsigned)d.J), f, d.F, gm, regs[u], acc);
      }
    }
  }
  __shared__ float sm[NW][NQ][256];
  __shared__ int is_last;
#pragma unroll
  for (int q = 0; q < NQ; ++q)
#pragma unroll
    for (int e = 0; e < 8; ++e) sm[warp][q][lane * 8 + e] = acc[q][e];
  __syncthreads();
  const int t = threadIdx.x;
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) s += sm[w][q][t];
    partial[((long long)q * P + chunk) * Fp + slice * 256 + t] = s;
  }
  __threadfence();
  __syncthreads();
  if (t == 0) is_last = (atomicAdd(&counters[slice], 1u) == (unsigned)(P - 1));
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // Last CTA of this slice adds the P partial rows in a fixed order: warp w takes chunks
  // w, w+NW, ... (eight independent loads in flight per lane), then the warps are summed in order.
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    float a[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) a[e] = 0.f;
    const float* base = partial + (long long)q * P * Fp + slice * 256 + lane * 8;
    for (int c0 = warp; c0 < P; c0 += NW * 4) {
      float4 u[4], v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int c = c0 + i * NW;
        if (c < P) {
          const float4* src = reinterpret_cast<const float4*>(base + (long long)c * Fp);
          u[i] = __ldcg(src);
          v[i] = __ldcg(src + 1);
        } else {
          u[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          v[i] = u[i];
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        a[0] += u[i].x; a[1] += u[i].y; a[2] += u[i].z; a[3] += u[i].w;
        a[4] += v[i].x; a[5] += v[i].y; a[6] += v[i].z; a[7] += v[i].w;
      }
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) sm[warp][q][lane * 8 + e] = a[e];
  }
  __syncthreads();
  if (slice * 256 + t < d.F) {
#pragma unroll
    for (int q = 0; q < NQ; ++q) {
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) s += sm[w][q][t];
      reinterpret_cast<sb_half*>(outs.out[q])[slice * 256 + t] = sb_f2h(s);
    }
  }
  if (t == 0) counters[slice] = 0u;
}

template <class Op>
int launch_colreduce(cudaStream_t s, void* ws, Dims3 d, const Op& op, ColOut<Op::NQ> outs, bool all_vec) {
  if (!ws) return fail(SB_ERR_ARG, "token-reduction operator called without a workspace");
  const int slices = (d.F + 255) / 256;
  if (slices > (int)(kWsCounterBytes / sizeof(unsigned)))
    return fail(SB_ERR_UNSUPPORTED, "feature dim too large for the workspace counters");
  const long long R = (long long)d.B * d.J;
  if (R > 0x7fffffffLL) return fail(SB_ERR_UNSUPPORTED, "token reductions over more than 2^31-1 tokens are not supported");
  const long long Fp = (long long)slices * 256;
  // as many 8-warp CTAs per SM as the kernel's register budget allows; bounded by rows and by the workspace
  long long P = ((long long)usable_sms(device_facts().sms) * Op::MINB + slices - 1) / slices;
  const long long cap = (long long)((kWsBytes - kWsCounterBytes) / (Op::NQ * Fp * sizeof(float)));
  if (cap < 1) return fail(SB_ERR_UNSUPPORTED, "feature dim too large for the workspace");
  if (P > cap) P = cap;
  if (P > (R + 7) / 8) P = (R + 7) / 8;
  if (P < 1) P = 1;
  const int rpc = (int)((R + P - 1) / P);
  P = (R + rpc - 1) / rpc;
  unsigned* counters = reinterpret_cast<unsigned*>(ws);
  float* partial = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + kWsCounterBytes);
  dim3 grid(slices, (unsigned)P);
  if (all_vec) SB_LAUNCH_OK(launch_k(colreduce_kernel<Op, true>, grid, kColThreads, 0, s, op, d, rpc, partial, counters, outs));
  else SB_LAUNCH_OK(launch_k(colreduce_kernel<Op, false>, grid, kColThreads, 0, s, op, d, rpc, partial, counters, outs));
  SB_CUDA_OK(cudaGetLastError());
  return SB_OK;
}

int param_vec(std::initializer_list<const void*> ptrs, int F) {
  if (F % 8) return 0;
  for (const void* p : ptrs)
    if (reinterpret_cast<uintptr_t>(p) & 15u) return 0;
  return 1;
}

}  // namespace

// ---------------------------------------------------------------------------
// Host launchers
// ---------------------------------------------------------------------------
template <class... V>
bool all_vec(const V&... v) {
  return ((v.vec != 0) && ...);
}

// Persistent grid: enough CTAs to fill every SM at the kernel's occupancy, no more than the work needs.
template <class K>
unsigned persistent_blocks(K kernel, int threads, unsigned long long work_blocks) {
  const int per_sm = cached_blocks_per_sm(reinterpret_cast<const void*>(kernel), threads);
  const unsigned long long cap = (unsigned long long)usable_sms(device_facts().sms) * per_sm;
  return (unsigned)std::max<unsigned long long>(1, std::min(work_blocks, cap));
}

#define SB_SOFTMAX_ONE(KERNEL, LPR, NV, ROWS, AVFLAG, ...)                                          \
  do {                                                                                              \
    const unsigned ngroups = (unsigned)((R + (32 / (LPR)) * (ROWS) - 1) / ((32 / (LPR)) * (ROWS))); \
    auto k = KERNEL<LPR, NV, ROWS, AVFLAG>;                                                         \
    const unsigned blocks = persistent_blocks(k, kSmThreads, (ngroups + 7) / 8);                    \
    SB_LAUNCH_OK(launch_k(k, blocks, kSmThreads, 0, s, __VA_ARGS__, (unsigned)R, ngroups));                             \
  } while (0)

#define SB_SOFTMAX_LAUNCH(KERNEL, AVFLAG, ...)                                    \
  do {                                                                            \
    if (d.K <= 64) SB_SOFTMAX_ONE(KERNEL, 8, 1, 2, AVFLAG, __VA_ARGS__);          \
    else if (d.K <= 128) SB_SOFTMAX_ONE(KERNEL, 16, 1, 2, AVFLAG, __VA_ARGS__);   \
    else if (d.K <= 256) SB_SOFTMAX_ONE(KERNEL, 32, 1, 2, AVFLAG, __VA_ARGS__);   \
    else if (d.K <= 512) SB_SOFTMAX_ONE(KERNEL, 32, 2, 2, AVFLAG, __VA_ARGS__);   \
    else if (d.K <= 1024) SB_SOFTMAX_ONE(KERNEL, 32, 4, 1, AVFLAG, __VA_ARGS__);  \
    else SB_SOFTMAX_ONE(KERNEL, 32, 8, 1, AVFLAG, __VA_ARGS__);                   \
  } while (0)

int launch_softmax_fwd(cudaStream_t s, Dims4 d, View4 beta, View4 alpha, View4 mask, View4 drop,
                       float scale, Rng rng) {
  const long long R = (long long)d.H * d.B * d.J;
  if (R == 0 || d.K == 0) return SB_OK;
  if (d.K > 2048) return fail(SB_ERR_UNSUPPORTED, "softmax rows longer than 2048 are not supported");
  if (R > 0x3fffffffLL) return fail(SB_ERR_UNSUPPORTED, "softmax over more than 2^30 rows is not supported");
  if (all_vec(beta, alpha, mask, drop))
    SB_SOFTMAX_LAUNCH(softmax_fwd_kernel, true, d, beta, alpha, mask, drop, scale, rng);
  else
    SB_SOFTMAX_LAUNCH(softmax_fwd_kernel, false, d, beta, alpha, mask, drop, scale, rng);
  SB_CUDA_OK(cudaGetLastError());
  return SB_OK;
}

int launch_softmax_bwd(cudaStream_t s, Dims4 d, View4 alpha, View4 mask, View4 dattn_drop,
                       View4 dbeta) {
  const long long R = (long long)d.H * d.B * d.J;
  if (R == 0 || d.K == 0) return SB_OK;
  if (d.K > 2048) return fail(SB_ERR_UNSUPPORTED, "softmax rows longer than 2048 are not supported");
  if (R > 0x3fffffffLL) return fail(SB_ERR_UNSUPPORTED, "softmax over more than 2^30 rows is not supported");
  if (all_vec(alpha, mask, dattn_drop, dbeta))
    SB_SOFTMAX_LAUNCH(softmax_bwd_kernel, true, d, alpha, mask, dattn_drop, dbeta);
  else
    SB_SOFTMAX_LAUNCH(softmax_bwd_kernel, false, d, alpha, mask, dattn_drop, dbeta);
  SB_CUDA_OK(cudaGetLastError());
  return SB_OK;
}

#define SB_ROW_ONE(KERNEL, NV, AVFLAG, ...)                                                  \
  do {                                                                                       \
    auto k = KERNEL<NV, AVFLAG>;                                                             \
    const unsigned blocks = persistent_blocks(k, kSmThreads, (unsigned long long)((R + 7) / 8)); \
    SB_LAUNCH_OK(launch_k(k, blocks, kSmThreads, 0, s, __VA_ARGS__));                                            \
  } while (0)

#define SB_ROW_LAUNCH(KERNEL, AVFLAG, F, ...)                            \
  do {                                                                   \
    if ((F) <= 256) SB_ROW_ONE(KERNEL, 1, AVFLAG, __VA_ARGS__);          \
    else if ((F) <= 512) SB_ROW_ONE(KERNEL, 2, AVFLAG, __VA_ARGS__);     \
    else if ((F) <= 1024) SB_ROW_ONE(KERNEL, 4, AVFLAG, __VA_ARGS__);    \
    else SB_ROW_ONE(KERNEL, 8, AVFLAG, __VA_ARGS__);                     \
  } while (0)

// dense, logical-order [B,J,F] (so that flat element i is the same element in every tensor)
bool dense3(const Dims3& d, const View3& v) {
  return v.vec && v.sF == 1 && (d.J <= 1 || v.sJ == d.F) && (d.B <= 1 || v.sB == (long long)d.J * d.F);
}
template <class... V>
bool all_dense3(const Dims3& d, const V&... v) {
  return (dense3(d, v) && ...);
}

int launch_bdrln(cudaStream_t s, Dims3 d, View3 in, const void* bias, View3 resid,
                 const void* gamma, const void* beta, View3 mask, View3 lin, View3 diff,
                 View2 istd, View3 ln, View3 out, Rng rng) {
  const long long R = (long long)d.B * d.J;
  if (R == 0 || d.F == 0) return SB_OK;
  if (d.F > 2048) return fail(SB_ERR_UNSUPPORTED, "LayerNorm rows longer than 2048 are not supported");
  if (R > 0x3fffffffLL) return fail(SB_ERR_UNSUPPORTED, "more than 2^30 tokens are not supported");
  const int pvec = param_vec({bias, gamma, beta}, d.F);
  if (pvec && all_vec(in, resid, mask, lin, diff, ln, out)) {
    // rows stream through a shared-memory ring when they can be moved with bulk copies
    const int st = launch_bdrln_ring(s, d, in, bias, resid, gamma, beta, mask, lin, diff, istd, ln, out, rng);
    if (st != SB_ERR_UNSUPPORTED) return st;
  }
  if (pvec && all_vec(in, resid, mask, lin, diff, ln, out))
    SB_ROW_LAUNCH(bdrln_kernel, true, d.F, d, in, bias, resid, gamma, beta, mask, lin, diff, istd, ln, out, rng, pvec);
  else
    SB_ROW_LAUNCH(bdrln_kernel, false, d.F, d, in, bias, resid, gamma, beta, mask, lin, diff, istd, ln, out, rng, pvec);
  SB_CUDA_OK(cudaGetLastError());
  return SB_OK;
}

int launch_blnrd(cudaStream_t s, Dims3 d, View3 dln, View2 istd, View3 diff, View3 mask,
                 View3 dresid, View3 dlin) {
  const long long R = (long long)d.B * d.J;
  if (R == 0 || d.F == 0) return SB_OK;
  if (d.F > 2048) return fail(SB_ERR_UNSUPPORTED, "LayerNorm rows longer than 2048 are not supported");
  if (R > 0x3fffffffLL) return fail(SB_ERR_UNSUPPORTED, "more than 2^30 tokens are not supported");
  if (all_vec(dln, diff, mask, dresid, dlin))
    SB_ROW_LAUNCH(blnrd_kernel, true, d.F, d, dln, istd, diff, mask, dresid, dlin);
  else
    SB_ROW_LAUNCH(blnrd_kernel, false, d.F, d, dln, istd, diff, mask, dresid, dlin);
  SB_CUDA_OK(cudaGetLastError());
  return SB_OK;
}

int launch_bad(cudaStream_t s, Dims3 d, View3 in, const void* bias, View3 mask, View3 lin1,
               View3 drop2, int activation, Rng rng) {
  const long long R = (long long)d.B * d.J;
  if (R == 0 || d.F == 0) return SB_OK;
  const int pvec = param_vec({bias}, d.F);
  if (pvec && all_dense3(d, in, mask, lin1, drop2)) {
    const unsigned long long ngroups = (unsigned long long)R * (d.F / 8);
    const unsigned long long work = (ngroups + (unsigned long long)kSmThreads * kFlatUnr - 1) / ((unsigned long long)kSmThreads * kFlatUnr);
    if (activation == SB_ACT_RELU) {
      auto k = bad_flat_kernel<SB_ACT_RELU>;
      SB_LAUNCH_OK(launch_k(k, persistent_blocks(k, kSmThreads, work), kSmThreads, 0, s, 
          ngroups, d.F / 8, (const uint4*)in.p, (const uint4*)bias, (uint2*)mask.p, (uint4*)lin1.p, (uint4*)drop2.p, rng));
    } else {
      auto k = bad_flat_kernel<SB_ACT_GELU>;
      SB_LAUNCH_OK(launch_k(k, persistent_blocks(k, kSmThreads, work), kSmThreads, 0, s, 
          ngroups, d.F / 8, (const uint4*)in.p, (const uint4*)bias, (uint2*)mask.p, (uint4*)lin1.p, (uint4*)drop2.p, rng));
    }
    SB_CUDA_OK(cudaGetLastError());
    return SB_OK;
  }
  const int spans = (d.F + kEwNV * 256 - 1) / (kEwNV * 256);
  const unsigned blocks = (unsigned)((R * spans + 3) / 4);
  if (pvec && all_vec(in, mask, lin1, drop2))
    SB_LAUNCH_OK(launch_k(bad_kernel<true>, blocks, kRowThreads, 0, s, d, spans, in, bias, mask, lin1, drop2, activation, rng, pvec));
  else
    SB_LAUNCH_OK(launch_k(bad_kernel<false>, blocks, kRowThreads, 0, s, d, spans, in, bias, mask, lin1, drop2, activation, rng, pvec));
  SB_CUDA_OK(cudaGetLastError());
  return SB_OK;
}

int launch_bei(cudaStream_t s, Dims3 d, View3 a, View3 b, View3 out) {
  const long long R = (long long)d.B * d.J;
  if (R == 0 || d.F == 0) return SB_OK;
  // same dense memory order in all three (any order): flat add
  const bool same = a.vec && b.vec && out.vec && a.sB == b.sB && a.sB == out.sB && a.sJ == b.sJ && a.sJ == out.sJ &&
                    ((a.sJ == d.F && a.sB == (long long)d.J * d.F) || (a.sB == d.F && a.sJ == (long long)d.B * d.F) ||
                     d.B == 1 || d.J == 1);
  if (same && dense3(d, a) ) {
    const unsigned long long ngroups = (unsigned long long)R * (d.F / 8);
    const unsigned long long work = (ngroups + (unsigned long long)kSmThreads * kFlatUnr - 1) / ((unsigned long long)kSmThreads * kFlatUnr);
    SB_LAUNCH_OK(launch_k(add_flat_kernel, persistent_blocks(add_flat_kernel, kSmThreads, work), kSmThreads, 0, s, 
        ngroups, (const uint4*)a.p, (const uint4*)b.p, (uint4*)out.p));
    SB_CUDA_OK(cudaGetLastError());
    return SB_OK;
  }
  const int spans = (d.F + kEwNV * 256 - 1) / (kEwNV * 256);
  const unsigned blocks = (unsigned)((R * spans + 3) / 4);
  if (all_vec(a, b, out)) SB_LAUNCH_OK(launch_k(bei_kernel<true>, blocks, kRowThreads, 0, s, d, spans, a, b, out));
  else SB_LAUNCH_OK(launch_k(bei_kernel<false>, blocks, kRowThreads, 0, s, d, spans, a, b, out));
  SB_CUDA_OK(cudaGetLastError());
  return SB_OK;
}

int launch_aib(cudaStream_t s, Dims5 d, View5 in, const void* bias, long long bsN, long long bsP,
               long long bsH, View5 out) {
  const long long R = (long long)d.N * d.P * d.H * d.B;
  if (R == 0 || d.J == 0) return SB_OK;
  // dense [N,P,H,B,J] in logical order on both sides and a dense bias: rows of B*J elements plus one scalar
  const long long BJ = (long long)d.B * d.J;
  const bool dense = in.vec && out.vec && d.J % 8 == 0 && in.sJ == 1 && out.sJ == 1 && in.sB == d.J && out.sB == d.J &&
                     in.sH == BJ && out.sH == BJ && in.sP == BJ * d.H && out.sP == BJ * d.H &&
                     in.sN == BJ * d.H * d.P && out.sN == BJ * d.H * d.P && bsH == 1 && bsP == d.H &&
                     bsN == (long long)d.H * d.P;
  if (dense) {
    const unsigned long long ngroups = (unsigned long long)R * (d.J / 8);
    const unsigned long long work = (ngroups + (unsigned long long)kSmThreads * kFlatUnr - 1) / ((unsigned long long)kSmThreads * kFlatUnr);
    SB_LAUNCH_OK(launch_k(rowbias_flat_kernel, persistent_blocks(rowbias_flat_kernel, kSmThreads, work), kSmThreads, 0, s, 
        ngroups, (unsigned)(BJ / 8), (const uint4*)in.p, (const sb_half*)bias, (uint4*)out.p));
    SB_CUDA_OK(cudaGetLastError());
    return SB_OK;
  }
  const int spans = (d.J + kEwNV * 256 - 1) / (kEwNV * 256);
  const unsigned blocks = (unsigned)((R * spans + 3) / 4);
  if (all_vec(in, out)) SB_LAUNCH_OK(launch_k(aib_kernel<true>, blocks, kRowThreads, 0, s, d, spans, in, bias, bsN, bsP, bsH, out));
  else SB_LAUNCH_OK(launch_k(aib_kernel<false>, blocks, kRowThreads, 0, s, d, spans, in, bias, bsN, bsP, bsH, out));
  SB_CUDA_OK(cudaGetLastError());
  return SB_OK;
}

int launch_baib(cudaStream_t s, Dims5 d, View5 in, void* dbias, long long bsN, long long bsP,
                long long bsH) {
  const long long R = (long long)d.N * d.P * d.H;
  if (R == 0) return SB_OK;
  const long long BJ = (long long)d.B * d.J;
  if (in.vec && in.sJ == 1 && in.sB == d.J && in.sH == BJ && in.sP == BJ * d.H && in.sN == BJ * d.H * d.P &&
      bsH == 1 && bsP == d.H && bsN == (long long)d.H * d.P && R < 0x7fffffffLL && BJ / 8 < 0x7fffffffLL) {
    const unsigned blocks = persistent_blocks(rowsum_flat_kernel, kSmThreads, (unsigned long long)((R + 7) / 8));
    SB_LAUNCH_OK(launch_k(rowsum_flat_kernel, blocks, kSmThreads, 0, s, (unsigned)R, (unsigned)(BJ / 8), (const uint4*)in.p, (sb_half*)dbias));
    SB_CUDA_OK(cudaGetLastError());
    return SB_OK;
  }
  if (all_vec(in)) SB_LAUNCH_OK(launch_k(baib_kernel<true>, (unsigned)R, kColThreads, 0, s, d, in, dbias, bsN, bsP, bsH));
  else SB_LAUNCH_OK(launch_k(baib_kernel<false>, (unsigned)R, kColThreads, 0, s, d, in, dbias, bsN, bsP, bsH));
  SB_CUDA_OK(cudaGetLastError());
  return SB_OK;
}

int launch_bsb(cudaStream_t s, void* ws, Dims3 d, View3 dy, View3 ln, const void* gamma,
               View3 dln, void* dgamma, void* dbeta) {
  BsbOp op{dy, ln, dln, gamma, param_vec({gamma}, d.F)};
  ColOut<2> outs{{dgamma, dbeta}};
  return launch_colreduce(s, ws, d, op, outs, op.pvec && all_vec(dy, ln, dln));
}

int launch_ebsb(cudaStream_t s, void* ws, Dims3 d, View3 ln1, const void* gamma1, View3 dresid2,
                View3 dlin1_linw1, View3 dlin2, View3 dln1, void* dgamma1, void* dbeta1,
                void* dlinb2) {
  EbsbOp op{ln1, dresid2, dlin1_linw1, dlin2, dln1, gamma1, param_vec({gamma1}, d.F)};
  ColOut<3> outs{{dgamma1, dbeta1, dlinb2}};
  return launch_colreduce(s, ws, d, op, outs, op.pvec && all_vec(ln1, dresid2, dlin1_linw1, dlin2, dln1));
}

int launch_bdrlb(cudaStream_t s, void* ws, Dims3 d, View3 ddrop2, View3 mask, View3 lin1,
                 View3 dlin1, void* dbias, int activation) {
  BdrlbOp op{ddrop2, mask, lin1, dlin1, activation};
  ColOut<1> outs{{dbias}};
  return launch_colreduce(s, ws, d, op, outs, all_vec(ddrop2, mask, lin1, dlin1));
}

int launch_baob(cudaStream_t s, void* ws, Dims3 d, View3 datt, void* dbo) {
  BaobOp op{datt};
  ColOut<1> outs{{dbo}};
  return launch_colreduce(s, ws, d, op, outs, all_vec(datt));
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the attention-output-bias gradient.
//
// Some hosts cannot hand this library a workspace: a plugin that is only ever given
// its inputs and outputs, a runtime whose device heap is owned by another component
// and locked after start-up, a caller that is not allowed to touch the CUDA
// allocator from the thread it runs on.  For them the fp32 partial sums and the
// ticket counters live in a fixed device array that is part of the library image:
// every GPU that loads the library carries these bytes until the process exits.
// ---------------------------------------------------------------------------
namespace {

constexpr size_t kStaticPartialBytes = 1u << 20;                              // 1 MiB of partial sums
constexpr size_t kStaticScratchBytes = kWsCounterBytes + kStaticPartialBytes;  // + 4 KiB of counters
constexpr int kStaticMaxFeatures = 16384;
constexpr int kMaxDevices = 64;

static __device__ __align__(256) unsigned char sb_static_scratch[kStaticScratchBytes];

// In host code `sb_static_scratch` is only a handle for the runtime, never a device pointer;
// the address each device sees is asked for once, with that device current, and remembered.
void* g_static_scratch_ptr[kMaxDevices] = {};
std::mutex g_static_scratch_mutex;

int static_scratch_for_current_device(void** out) {
  int dev = 0;
  SB_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return fail(SB_ERR_UNSUPPORTED, "device ordinal beyond the per-device scratch table");
  std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
  if (!g_static_scratch_ptr[dev]) {
    void* ptr = nullptr;
    SB_CUDA_OK(cudaGetSymbolAddress(&ptr, sb_static_scratch));
    if (!ptr) return fail(SB_ERR_CUDA, "cudaGetSymbolAddress returned a null address for the built-in scratch");
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return SB_OK;
}

}  // namespace
}  // namespace sb

extern "C" int sb_backward_attn_out_bias_noalloc(void* stream, const sb_tensor* datt, const sb_tensor* dbo) {
  using namespace sb;
  if (!datt || !dbo) return fail(SB_ERR_ARG, "baob (no-alloc): null tensor");
  if (datt->ndim != 3 || dbo->ndim != 1) return fail(SB_ERR_ARG, "baob (no-alloc): datt must have rank 3 and dbo rank 1");
  for (int i = 0; i < 3; ++i)
    if (datt->size[i] < 0 || datt->size[i] > 0x7fffffffLL) return fail(SB_ERR_ARG, "baob (no-alloc): extent out of range");
  const long long B = datt->size[0], J = datt->size[1], F = datt->size[2];
  if (dbo->size[0] != F) return fail(SB_ERR_ARG, "baob (no-alloc): extent mismatch between operands");
  if (F > kStaticMaxFeatures)
    return fail(SB_ERR_UNSUPPORTED, "baob (no-alloc): feature extent " + std::to_string(F) +
                                        " exceeds the built-in scratch limit of " + std::to_string(kStaticMaxFeatures) +
                                        "; use sb_backward_attn_out_bias with a caller workspace");
  if (F > 1 && dbo->stride[0] != 1) return fail(SB_ERR_UNSUPPORTED, "baob (no-alloc): dbo must be contiguous");
  if (B * J * F == 0) return SB_OK;
  if (!datt->ptr || !dbo->ptr) return fail(SB_ERR_ARG, "baob (no-alloc): null data pointer");

  void* scratch = nullptr;
  SB_TRY(static_scratch_for_current_device(&scratch));
  cudaStream_t s = (cudaStream_t)stream;

  View3 v;
  v.p = datt->ptr; v.sB = datt->stride[0]; v.sJ = datt->stride[1]; v.sF = datt->stride[2];
  v.vec = (v.sF == 1 && F % 8 == 0 && (reinterpret_cast<uintptr_t>(v.p) & 15u) == 0 &&
           (B <= 1 || v.sB % 8 == 0) && (J <= 1 || v.sJ % 8 == 0)) ? 1 : 0;
  const Dims3 d{(int)B, (int)J, (int)F};
  const int slices = (int)((F + 255) / 256);
  const long long R = B * J, Fp = (long long)slices * 256;
  if (R > 0x7fffffffLL)   // the kernel indexes tokens with 32-bit arithmetic
    return fail(SB_ERR_UNSUPPORTED, "baob (no-alloc): more than 2^31-1 tokens (B*J) are not supported");
  long long P = ((long long)usable_sms(device_facts().sms) * 4 + slices - 1) / slices;
  const long long cap = (long long)(kStaticPartialBytes / (Fp * sizeof(float)));  // >= 16 for F <= 16384
  if (P > cap) P = cap;
  if (P > (R + 7) / 8) P = (R + 7) / 8;
  if (P < 1) P = 1;
  const int rpc = (int)((R + P - 1) / P);
  P = (R + rpc - 1) / rpc;
  // The array keeps whatever the previous call left in it.  Partial sums are fully rewritten
  // before they are read; the ticket counters must start at zero, so clear them on the stream.
  SB_CUDA_OK(cudaMemsetAsync(scratch, 0, kWsCounterBytes, s));
  unsigned* counters = reinterpret_cast<unsigned*>(scratch);
  float* partial = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + kWsCounterBytes);
  BaobOp op{v};
  ColOut<1> outs{{dbo->ptr}};
  dim3 grid(slices, (unsigned)P);
  if (v.vec) colreduce_kernel<BaobOp, true><<<grid, kColThreads, 0, s>>>(op, d, rpc, partial, counters, outs);
  else colreduce_kernel<BaobOp, false><<<grid, kColThreads, 0, s>>>(op, d, rpc, partial, counters, outs);
  SB_CUDA_OK(cudaGetLastError());
  return SB_OK;
}
