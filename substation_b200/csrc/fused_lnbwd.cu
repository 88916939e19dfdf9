// LayerNorm operators that stream whole token rows.
//
// Backward, fused: the LayerNorm scale/bias gradients, the LayerNorm backward-data with dropout, and the bias
// gradients that are plain sums over tokens of tensors this pass touches anyway, in ONE pass over the data.
//   mode A  = backward_scale_bias + backward_layernorm_residual_dropout
//             (pytorch_module/block_bsb_ebsb.cuh:171-216, block_blnrd.cuh:71-129)
//   mode B  = extended_backward_scale_bias + backward_layernorm_residual_dropout
//             + backward_attn_out_bias
//             (block_bsb_ebsb.cuh:368-420, block_blnrd.cuh:195-259, block_baob.cuh:75-97)
// Both need sums over features (per token) AND sums over tokens (per feature).
// Mapping: a CTA has 4 row groups of 128 threads; the 128 threads of a group span one token (8 features each,
// up to 1024 features).  Per-token sums: warp shuffles, then the group's 4 warps exchange through shared
// memory behind a group-local named barrier.  Per-feature sums: each thread accumulates its 8 features in
// registers over all of its tokens; at the end the 4 groups are added in order, the CTA writes one fp32
// partial row per quantity, and a second small kernel adds the partial rows in order (deterministic).
// Two kernels share that mapping: lnbwd_ring_kernel takes its input rows from a shared-memory ring that a
// producer warp fills with bulk copies (see ring.cuh; rows of 16-byte multiples), lnbwd_kernel loads them
// straight from global memory (any feature count that is a multiple of 8).
//
// Forward: bias + dropout + residual + LayerNorm (pytorch_module/block_bdrln.cuh:105-180, :275-352) with the same
// ring, one warp per token: bdrln_ring_kernel.

#include <algorithm>
#include <cstdlib>

#include "ops.h"
#include "ring.cuh"

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
      s[r] = sb_h2f(reinterpret_cast<const sb_half*>(p.istd.p)[b * p.istd.sB + j * p.istd.sJ]);
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

// ---------------------------------------------------------------------------------------------------------
// The same pass with its inputs staged through a shared-memory ring.  Thread layout: warps 0-15 = four row groups
// (as above), warp 16 = producer.  The tensors must be dense token-major ([tokens][F] with nothing between rows),
// so that kGroups consecutive tokens are one contiguous piece of every tensor: a ring stage holds such a block of
// four tokens, fetched with ONE bulk copy per tensor (8 KB at 1024 features; the copy engine keeps few requests
// in flight, so requests of one row each leave most of the bandwidth unused).  Block sequence of a CTA: blocks
// blockIdx.x + i * gridDim.x; block i lives in stage i % NS and group g works on its g-th token.  Stage layout:
//   mode A: DY, LN, DIFF (4 x 2F bytes each), mask (4 x F bytes);   mode B: LN1, DRESID2, DLIN1_LINW1, DLIN2, DIFF, mask.
// The per-feature accumulators go through the ring's memory once the ring is drained.
// ---------------------------------------------------------------------------------------------------------
constexpr int kRingThreads = kThreads + 32;

template <int MODE>
struct RingCfg {
  static constexpr int NQ = MODE == 0 ? 2 : 4;
  static constexpr int NIN = MODE == 0 ? 3 : 5;                 // fp16 input rows per token (incl. DIFF)
  static constexpr int kColredBytes = kGroups * NQ * kMaxF * 4;
  static constexpr int kBudget = 232448 - 1024;                 // ring bytes available (barriers and sums follow)
};

// one lane polls, the warp follows (fewer pollers on the barrier unit than one per thread)
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, int code, int lane) {
  int ok = 1;
  if (lane == 0) ok = ring::mbar_wait(bar, parity, code) ? 1 : 0;
  return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

template <int MODE>
__global__ void __launch_bounds__(kRingThreads, 1)
lnbwd_ring_kernel(LnBwdParams p, int nstages, int stage_bytes) {
  using C = RingCfg<MODE>;
  constexpr int NQ = C::NQ;
  constexpr int NIN = C::NIN;
  extern __shared__ __align__(128) uint8_t smem[];
  // layout: ring (reused for the column sums [kGroups][NQ][1024] at the end) | red | barriers
  uint8_t* ring_gen = smem;
  const uint32_t ring_s = ring::smem_u32(ring_gen);
  const int ring_bytes = max(nstages * stage_bytes, C::kColredBytes);
  float* red = reinterpret_cast<float*>(ring_gen + ring_bytes);                       // [kGroups][2][4][2]
  const uint32_t bars = ring::smem_u32(red) + kGroups * 2 * 4 * 2 * 4;                 // full[NS], empty[NS]
  const uint32_t bar_full = bars, bar_empty = bars + 8 * nstages;

  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int F = p.d.F;
  const unsigned R = (unsigned)p.d.B * (unsigned)p.d.J;
  const unsigned nblocks = (R + kGroups - 1) / kGroups;
  const unsigned G = gridDim.x;
  const unsigned n_i = blockIdx.x < nblocks ? (nblocks - blockIdx.x + G - 1) / G : 0;   // blocks of this CTA
  const uint32_t row_bytes = 2u * (uint32_t)F;
  const uint32_t tensor_bytes = kGroups * row_bytes;       // one tensor's part of a stage

  if (tid == 0) {
    for (int s = 0; s < nstages; ++s) {
      ring::mbar_init(bar_full + 8 * s, 1);
      ring::mbar_init(bar_empty + 8 * s, kThreads / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  grid_dependency_sync();

  if (warp == kThreads / 32) {
    // ---------------- producer: one elected lane issues the copies of block after block ----------------
    if (lane == 0) {
      for (unsigned i = 0; i < n_i; ++i) {
        const int s = (int)(i % (unsigned)nstages);
        const uint32_t ph = (i / (unsigned)nstages) & 1u;
        if (!ring::mbar_wait(bar_empty + 8 * s, ph ^ 1u, 11)) break;
        const unsigned long long row0 = (unsigned long long)(blockIdx.x + i * G) * kGroups;
        const uint32_t nrows = (uint32_t)min((unsigned long long)kGroups, R - row0);
        const uint32_t full = bar_full + 8 * s;
        const uint32_t dst = ring_s + (uint32_t)s * (uint32_t)stage_bytes;
        const uint32_t nb = nrows * row_bytes;
        ring::mbar_expect_tx(full, NIN * nb + nrows * (uint32_t)F);
        auto rows_of = [&](const View3& v) { return reinterpret_cast<const sb_half*>(v.p) + row0 * F; };
        if (MODE == 0) {
          ring::bulk_load(dst, rows_of(p.y), nb, full);
          ring::bulk_load(dst + tensor_bytes, rows_of(p.n), nb, full);
        } else {
          ring::bulk_load(dst, rows_of(p.n), nb, full);
          ring::bulk_load(dst + tensor_bytes, rows_of(p.r2), nb, full);
          ring::bulk_load(dst + 2 * tensor_bytes, rows_of(p.w), nb, full);
          ring::bulk_load(dst + 3 * tensor_bytes, rows_of(p.l2), nb, full);
        }
        ring::bulk_load(dst + (NIN - 1) * tensor_bytes, rows_of(p.diff), nb, full);
        ring::bulk_load(dst + NIN * tensor_bytes, reinterpret_cast<const uint8_t*>(p.mask.p) + row0 * F, nrows * (uint32_t)F, full);
      }
    }
    __syncwarp();
  } else {
    // ---------------- consumers: group g takes the g-th token of every block ----------------
    const int group = tid / kGroupThreads, t = tid % kGroupThreads;
    const int warp_in_group = t >> 5;
    const int f = t * 8;
    const bool has_f = f < F;
    const float invn = 1.f / (float)F;
    float gm[8];
    if (has_f) unpack8(load8h_raw(p.gamma, 0, 1, 1, f, F), gm);
    float acc[NQ][8];
#pragma unroll
    for (int q = 0; q < NQ; ++q)
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[q][e] = 0.f;
    const sb_half* istd = reinterpret_cast<const sb_half*>(p.istd.p);
    auto istd_of = [&](unsigned i) {
      const unsigned long long row = (unsigned long long)(blockIdx.x + i * G) * kGroups + group;
      if (row >= R) return sb_f2h(0.f);
      return istd[(long long)(row / (unsigned)p.d.J) * p.istd.sB + (long long)(row % (unsigned)p.d.J) * p.istd.sJ];
    };
    sb_half s_next = n_i > 0 ? istd_of(0) : sb_f2h(0.f);
    for (unsigned i = 0; i < n_i; ++i) {
      const int s = (int)(i % (unsigned)nstages);
      const uint32_t ph = (i / (unsigned)nstages) & 1u;
      const unsigned long long row = (unsigned long long)(blockIdx.x + i * G) * kGroups + group;
      const bool active = has_f && row < R;
      const float sd = sb_h2f(s_next);
      if (i + 1 < n_i) s_next = istd_of(i + 1);          // in flight while this token is worked on
      if (!warp_wait(bar_full + 8 * s, ph, 12, lane)) break;
      const uint8_t* st = ring_gen + (size_t)s * stage_bytes;
      uint4 in[NIN];
      uint2 mk = make_uint2(0, 0);
      if (active) {
#pragma unroll
        for (int k = 0; k < NIN; ++k)
          in[k] = *reinterpret_cast<const uint4*>(st + (size_t)k * tensor_bytes + (size_t)group * row_bytes + (size_t)t * 16);
        mk = *reinterpret_cast<const uint2*>(st + (size_t)NIN * tensor_bytes + (size_t)group * F + (size_t)t * 8);
      }
      __syncwarp();
      if (lane == 0) ring::mbar_arrive(bar_empty + 8 * s);             // this warp has its pieces in registers
      float g[8], d8[8];
      float sg = 0.f, sgd = 0.f;
      if (active) {
        float a[8], n8[8];
        unpack8(in[NIN - 1], d8);
        if (MODE == 0) {
          unpack8(in[0], a);
          unpack8(in[1], n8);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            g[e] = a[e] * gm[e];
            acc[0][e] = fmaf(a[e], n8[e], acc[0][e]);
            acc[1][e] += a[e];
          }
        } else {
          float r2[8], w8[8], l28[8];
          unpack8(in[0], n8);
          unpack8(in[1], r2);
          unpack8(in[2], w8);
          unpack8(in[3], l28);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            a[e] = r2[e] + w8[e];
            g[e] = a[e] * gm[e];
            acc[0][e] = fmaf(a[e], n8[e], acc[0][e]);
            acc[1][e] += a[e];
            acc[2][e] += l28[e];
          }
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          sg += g[e];
          sgd = fmaf(g[e], d8[e], sgd);
        }
      }
      sg = warp_sum(sg);
      sgd = warp_sum(sgd);
      float* rg = red + ((group * 2 + (i & 1)) * 4) * 2;
      if (lane == 0) {
        rg[warp_in_group * 2] = sg;
        rg[warp_in_group * 2 + 1] = sgd;
      }
      group_barrier(group);
      sg = rg[0] + rg[2] + rg[4] + rg[6];
      sgd = rg[1] + rg[3] + rg[5] + rg[7];
      if (active) {
        const float c1 = sg * sd * invn, c2 = sgd * sd * sd * sd * invn;
        float o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = fmaf(g[e], sd, -c1) - d8[e] * c2;
        const uint4 dres = pack8(o);
        const uint4 dl = mask_apply(dres, mk);
        const long long off = (long long)row * F;
        if (p.dln.p) store8h_raw(p.dln.p, off, 1, 1, f, F, pack8(g));
        store8h_raw(p.dresid.p, off, 1, 1, f, F, dres);
        store8h_raw(p.dlin.p, off, 1, 1, f, F, dl);
        if (MODE == 1) {
          float dv[8];
          unpack8(dl, dv);  // the fp16 values just stored: the bias gradient sums exactly them
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[3][e] += dv[e];
        }
      }
    }
    __syncwarp();
    // every consumer is done with the ring before its memory takes the accumulators (a named barrier over the
    // 512 consumer threads; the producer warp is not part of it)
    asm volatile("bar.sync 8, %0;" ::"n"(kThreads) : "memory");
    float* colred = reinterpret_cast<float*>(smem);
#pragma unroll
    for (int q = 0; q < NQ; ++q)
#pragma unroll
      for (int e = 0; e < 8; ++e) colred[(group * NQ + q) * kMaxF + f + e] = acc[q][e];
  }
  __syncthreads();
  const float* colred = reinterpret_cast<const float*>(smem);
  for (int i = tid; i < NQ * kMaxF; i += kRingThreads) {
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
    reinterpret_cast<sb_half*>(outs[q])[f] = sb_f2h(total);
  }
}

// ---------------------------------------------------------------------------------------------------------
// Forward: bias + dropout + residual + LayerNorm out of the same kind of ring (dense token-major tensors, blocks of
// four consecutive tokens, one bulk copy per tensor and block).  Warps 0-27 consume, one warp per token: block i of
// the CTA lives in stage i % NS and belongs to the warp set i % 7 (warps 4 * set .. 4 * set + 3, one token each), so
// the seven blocks a CTA gets at 4096 tokens on 148 SMs are one round (sixteen warps took two: 18.3 against 16.5 us).
// Warp 28 produces.  A stage holds IN and RESID (4 x 2F bytes each) and, when the mask is an input, the mask rows
// (4 x F bytes).  NV = 128-bit pieces per lane and row (F <= 256 * NV).
// ---------------------------------------------------------------------------------------------------------
constexpr int kFwdWarps = 28;
constexpr int kFwdThreads = (kFwdWarps + 1) * 32;
constexpr int kFwdRows = 4;                      // tokens per stage

struct BdrlnParams {
  Dims3 d;
  View3 in, resid, mask, lin, diff, ln, out;
  View2 istd;
  const void *bias, *gamma, *beta;
  Rng rng;
};

template <int NV>
__global__ void __launch_bounds__(kFwdThreads, 1)
bdrln_ring_kernel(BdrlnParams p, int nstages, int stage_bytes) {
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t ring_s = ring::smem_u32(smem);
  const uint32_t bars = ring_s + (uint32_t)nstages * (uint32_t)stage_bytes;   // full[NS], empty[NS]
  const uint32_t bar_full = bars, bar_empty = bars + 8 * nstages;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int F = p.d.F;
  const unsigned R = (unsigned)p.d.B * (unsigned)p.d.J;
  const unsigned nblocks = (R + kFwdRows - 1) / kFwdRows;
  const unsigned G = gridDim.x;
  const unsigned n_i = blockIdx.x < nblocks ? (nblocks - blockIdx.x + G - 1) / G : 0;
  const uint32_t row_bytes = 2u * (uint32_t)F;
  const uint32_t tensor_bytes = kFwdRows * row_bytes;
  const bool mask_in = !p.rng.philox;

  if (tid == 0) {
    for (int s = 0; s < nstages; ++s) {
      ring::mbar_init(bar_full + 8 * s, 1);
      ring::mbar_init(bar_empty + 8 * s, kFwdRows);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  grid_dependency_sync();

  if (warp == kFwdWarps) {
    if (lane == 0) {
      for (unsigned i = 0; i < n_i; ++i) {
        const int s = (int)(i % (unsigned)nstages);
        const uint32_t ph = (i / (unsigned)nstages) & 1u;
        if (!ring::mbar_wait(bar_empty + 8 * s, ph ^ 1u, 13)) break;
        const unsigned long long row0 = (unsigned long long)(blockIdx.x + i * G) * kFwdRows;
        const uint32_t nrows = (uint32_t)min((unsigned long long)kFwdRows, R - row0);
        const uint32_t full = bar_full + 8 * s;
        const uint32_t dst = ring_s + (uint32_t)s * (uint32_t)stage_bytes;
        const uint32_t nb = nrows * row_bytes;
        ring::mbar_expect_tx(full, 2 * nb + (mask_in ? nrows * (uint32_t)F : 0u));
        ring::bulk_load(dst, reinterpret_cast<const sb_half*>(p.in.p) + row0 * F, nb, full);
        ring::bulk_load(dst + tensor_bytes, reinterpret_cast<const sb_half*>(p.resid.p) + row0 * F, nb, full);
        if (mask_in)
          ring::bulk_load(dst + 2 * tensor_bytes, reinterpret_cast<const uint8_t*>(p.mask.p) + row0 * F, nrows * (uint32_t)F, full);
      }
    }
    __syncwarp();
    return;
  }
  const float invF = 1.f / (float)F;
  const int set = warp >> 2, rsel = warp & 3;          // which blocks, which token of a block
  for (unsigned i = set; i < n_i; i += kFwdWarps / kFwdRows) {
    const int s = (int)(i % (unsigned)nstages);
    const uint32_t ph = (i / (unsigned)nstages) & 1u;
    const unsigned long long row = (unsigned long long)(blockIdx.x + i * G) * kFwdRows + rsel;
    if (!warp_wait(bar_full + 8 * s, ph, 14, lane)) break;
    const bool valid = row < R;
    const long long b = (long long)(row / (unsigned)p.d.J), j = (long long)(row % (unsigned)p.d.J);
    const long long off = (long long)row * F;
    const uint8_t* st = smem + (size_t)s * stage_bytes + (size_t)rsel * row_bytes;          // this token's IN row
    const uint8_t* st_m = smem + (size_t)s * stage_bytes + 2 * (size_t)tensor_bytes + (size_t)rsel * F;
    float r[NV][8];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int piece = lane + kWarp * k;
      const int f = piece * 8;
      if (valid && f < F) {
        uint2 mk;
        if (mask_in) {
          mk = *reinterpret_cast<const uint2*>(st_m + (size_t)piece * 8);
        } else {
          uint32_t mm[8];
          philox_keep8(p.rng, ((unsigned long long)row * F + f) >> 3, mm);
          mk = mask_pack(mm);
          store8m_raw(p.mask.p, off, 1, 1, f, F, mk);
        }
        float x[8], bb[8], rs[8];
        unpack8(*reinterpret_cast<const uint4*>(st + (size_t)piece * 16), x);
        unpack8(load8h_raw(p.bias, 0, 1, 1, f, F), bb);
        unpack8(*reinterpret_cast<const uint4*>(st + tensor_bytes + (size_t)piece * 16), rs);
#pragma unroll
        for (int e = 0; e < 8; ++e) x[e] += bb[e];
        if (p.lin.p) store8h_raw(p.lin.p, off, 1, 1, f, F, pack8(x));
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          r[k][e] = (mask_keep(mk, e) ? x[e] : 0.f) + rs[e];
          sum += r[k][e];
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) r[k][e] = 0.f;
      }
    }
    __syncwarp();
    if (lane == 0) ring::mbar_arrive(bar_empty + 8 * s);     // the row has been read: the stage may be refilled
    if (!valid) continue;
    const float mean = warp_sum(sum) * invF;
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int f = (lane + kWarp * k) * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        r[k][e] = (f < F) ? r[k][e] - mean : 0.f;
        sq = fmaf(r[k][e], r[k][e], sq);
      }
    }
    const float rstd = rsqrtf(warp_sum(sq) * invF + kLnEps);
    if (lane == 0) reinterpret_cast<sb_half*>(p.istd.p)[b * p.istd.sB + j * p.istd.sJ] = sb_f2h(rstd);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int f = (lane + kWarp * k) * 8;
      if (f >= F) continue;
      float gm[8], bt[8], n[8], o[8];
      unpack8(load8h_raw(p.gamma, 0, 1, 1, f, F), gm);
      unpack8(load8h_raw(p.beta, 0, 1, 1, f, F), bt);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        n[e] = r[k][e] * rstd;
        o[e] = fmaf(n[e], gm[e], bt[e]);
      }
      store8h_raw(p.diff.p, off, 1, 1, f, F, pack8(r[k]));
      store8h_raw(p.ln.p, off, 1, 1, f, F, pack8(n));
      store8h_raw(p.out.p, off, 1, 1, f, F, pack8(o));
    }
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

bool ring_enabled() {
  static const bool on = [] {
    const char* e = getenv("SUBSTATION_B200_LN_RING");
    return !(e && e[0] == '0');
  }();
  return on;
}

// The ring kernels fetch blocks of consecutive tokens with one bulk copy per tensor: every tensor must be dense
// token-major ([tokens][F], unit feature stride, nothing between rows) and rows must be 16-byte multiples from a
// 16-byte-aligned base (for the byte mask that means F % 16 == 0).
bool dense_rows(const Dims3& d, const View3& v) {
  return v.sF == 1 && (d.J <= 1 || v.sJ == d.F) && (d.B <= 1 || v.sB == (long long)d.J * d.F) &&
         (reinterpret_cast<uintptr_t>(v.p) & 15u) == 0;
}
bool ring_ok(const Dims3& d, std::initializer_list<const View3*> views, bool with_mask) {
  if (!ring_enabled() || d.F % 8 != 0 || (with_mask && d.F % 16 != 0)) return false;
  for (const View3* v : views)
    if (v->p && !dense_rows(d, *v)) return false;
  return true;
}

template <int MODE>
int launch(cudaStream_t s, void* ws, const LnBwdParams& p0, void* const outs[4]) {
  constexpr int NQ = MODE == 0 ? 2 : 4;
  LnBwdParams p = p0;
  const long long R = (long long)p.d.B * p.d.J;
  const int sms = usable_sms(device_facts().sms);
  const bool use_ring = MODE == 0 ? ring_ok(p.d, {&p.y, &p.n, &p.diff, &p.mask, &p.dln, &p.dresid, &p.dlin}, true)
                                  : ring_ok(p.d, {&p.n, &p.r2, &p.w, &p.l2, &p.diff, &p.mask, &p.dln, &p.dresid, &p.dlin}, true);
  const int per_cta = use_ring ? kGroups : kGroups * kRows;
  const int P = (int)std::max<long long>(1, std::min<long long>(sms, (R + per_cta - 1) / per_cta));
  if ((size_t)NQ * P * kMaxF * sizeof(float) > kWsBytes - kWsCounterBytes)
    return fail(SB_ERR_UNSUPPORTED, "fused LayerNorm backward: workspace too small");
  p.partial = reinterpret_cast<float*>(reinterpret_cast<char*>(ws) + kWsCounterBytes);
  if (use_ring) {
    using C = RingCfg<MODE>;
    const int stage_bytes = (kGroups * (C::NIN * 2 * p.d.F + p.d.F) + 127) / 128 * 128;
    const int nstages = std::max(2, std::min(16, C::kBudget / stage_bytes));
    const size_t smem = (size_t)std::max(nstages * stage_bytes, C::kColredBytes) + 256 + 16 * (size_t)nstages + 64;
    // the attribute is set once to the most any launch may ask for (launches differ in their ring size)
    SB_CUDA_OK(ensure_dynamic_smem(reinterpret_cast<const void*>(lnbwd_ring_kernel<MODE>), 232448));
    SB_LAUNCH_OK(launch_k(lnbwd_ring_kernel<MODE>, P, kRingThreads, smem, s, p, nstages, stage_bytes));
  } else {
    const size_t smem = (size_t)kGroups * NQ * kMaxF * sizeof(float);
    SB_CUDA_OK(ensure_dynamic_smem(reinterpret_cast<const void*>(lnbwd_kernel<MODE>), (int)smem));
    SB_LAUNCH_OK(launch_k(lnbwd_kernel<MODE>, P, kThreads, smem, s, p));
  }
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

// Ring-fed forward LayerNorm; SB_ERR_UNSUPPORTED (nothing launched) when the views do not qualify, the caller then
// runs the register-resident kernel.
int launch_bdrln_ring(cudaStream_t s, Dims3 d, View3 in, const void* bias, View3 resid, const void* gamma,
                      const void* beta, View3 mask, View3 lin, View3 diff, View2 istd, View3 ln, View3 out, Rng rng) {
  const long long R = (long long)d.B * d.J;
  if (!ring_enabled() || d.F % 8 != 0 || d.F > 2048 || R > 0x3fffffffLL || R < 1)
    return fail(SB_ERR_UNSUPPORTED, "ring LayerNorm: shape not covered");
  if (!ring_ok(d, {&in, &resid, &lin, &diff, &ln, &out}, false) || !dense_rows(d, mask) || (!rng.philox && d.F % 16 != 0))
    return fail(SB_ERR_UNSUPPORTED, "ring LayerNorm needs dense token-major tensors with 16-byte-multiple rows");
  for (const void* q : {bias, gamma, beta})
    if (reinterpret_cast<uintptr_t>(q) & 15u) return fail(SB_ERR_UNSUPPORTED, "ring LayerNorm needs aligned parameter vectors");
  BdrlnParams p{};
  p.d = d; p.in = in; p.resid = resid; p.mask = mask; p.lin = lin; p.diff = diff; p.ln = ln; p.out = out;
  p.istd = istd; p.bias = bias; p.gamma = gamma; p.beta = beta; p.rng = rng;
  const int stage_bytes = (kFwdRows * 5 * d.F + 127) / 128 * 128;
  const int nstages = std::max(2, std::min(16, (232448 - 1024) / stage_bytes));
  const size_t smem = (size_t)nstages * stage_bytes + 16 * (size_t)nstages + 64;
  const int P = (int)std::max<long long>(1, std::min<long long>(usable_sms(device_facts().sms), (R + kFwdRows - 1) / kFwdRows));
#define SB_BDRLN_RING(NV)                                                                                    \
  do {                                                                                                       \
    SB_CUDA_OK(ensure_dynamic_smem(reinterpret_cast<const void*>(bdrln_ring_kernel<NV>), 232448));           \
    SB_LAUNCH_OK(launch_k(bdrln_ring_kernel<NV>, P, kFwdThreads, smem, s, p, nstages, stage_bytes));         \
  } while (0)
  if (d.F <= 256) SB_BDRLN_RING(1);
  else if (d.F <= 512) SB_BDRLN_RING(2);
  else if (d.F <= 1024) SB_BDRLN_RING(4);
  else SB_BDRLN_RING(8);
#undef SB_BDRLN_RING
  SB_CUDA_OK(cudaGetLastError());
  return SB_OK;
}

int ring_device_error(cudaStream_t s, int* code) {
  int v = 0;
  SB_CUDA_OK(cudaMemcpyFromSymbolAsync(&v, ring::g_ring_error, sizeof(int), 0, cudaMemcpyDeviceToHost, s));
  SB_CUDA_OK(cudaStreamSynchronize(s));
  *code = v;
  return SB_OK;
}
int ring_device_error_reset(cudaStream_t s) {
  const int zero = 0;
  SB_CUDA_OK(cudaStreamSynchronize(s));
  SB_CUDA_OK(cudaMemcpyToSymbol(ring::g_ring_error, &zero, sizeof(int), 0, cudaMemcpyHostToDevice));
  return SB_OK;
}

}  // namespace sb
