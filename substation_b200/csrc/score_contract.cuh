// Contractions of a score tensor S[h,b,j,k] with head-size-64 projections (included by gemm.cu;
// shares its TMA / tcgen05 helpers):
//
//   rows:  R[p,h,b,j] = alpha * sum_k S[h,b,j,k] * X[p,h,b,k]
//          (gamma and dX1QKT of pytorch_module/encoder.cu:123-125, 263-265)
//   cols:  C[p,h,b,k] = alpha * sum_j S[h,b,j,k] * Y[p,h,b,j]
//          (dX2gamma and dX2QKT of pytorch_module/encoder.cu:254-256, 267-269)
//
// either one, or both from a single pass over S.  These are HBM-bound: 2 L^2 bytes of S per
// (head, sample) against 4 * 64 * L of projections, so the kernel is organised around reading S
// exactly once.  One CTA owns a whole (head, sample): X and Y stay resident in shared memory, S
// streams through a ring of [128 j x 128 k] tiles, and each tile feeds both contractions, as a
// K-major A operand (M = j, K = k) for the rows and, unchanged in shared memory, as an MN-major A
// operand (M = k, K = j) for the columns.  Accumulators: two 64-column buffers for the rows of the
// current j block (so the epilogue of one block overlaps the next) and L/128 buffers of 64 columns
// for the columns, which accumulate over all j blocks.
// Requirements: head size 64, L a multiple of 128 and at most 512, S dense as [H,B,J,K].

#pragma once

namespace scon {

constexpr int kMaxStages = 6;
constexpr int kStageBytes = 32768;  // [128 j x 128 k] fp16 as two 128-byte-swizzled boxes

struct Params {
  int L, nt;              // sequence length, L / 128
  int units;              // H * B
  int has_r, has_c;
  int x_mn, x_swap, y_mn, y_swap, s_swap;
  int nstages;
  int nbuf;               // 1 or 2 sets of (X, Y, column accumulators): with 2, the next unit loads while this one computes
  float alpha;
  sb_half* out_r; long long r_sU, r_sRow, r_sP;   // strides of R over (unit, j, p)
  sb_half* out_c; long long c_sU, c_sRow, c_sP;   // strides of C over (unit, k, p)
};

// 64 fp32 accumulator columns of this thread's row -> alpha * value as fp16 at ptr[p * sP]
__device__ __forceinline__ void store_row64(sb_half* ptr, long long sP, const uint32_t* r, float alpha) {
  if (sP == 1 && (reinterpret_cast<uintptr_t>(ptr) & 15u) == 0) {
#pragma unroll
    for (int v = 0; v < 8; ++v) {
      float f[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]) * alpha;
      reinterpret_cast<uint4*>(ptr)[v] = pack8(f);
    }
  } else {
#pragma unroll
    for (int e = 0; e < 64; ++e) ptr[e * sP] = sb_f2h(__uint_as_float(r[e]) * alpha);
  }
}

__global__ void __launch_bounds__(kTcThreads, 1)
score_contract_kernel(const __grid_constant__ CUtensorMap tmS, const __grid_constant__ CUtensorMap tmX,
                      const __grid_constant__ CUtensorMap tmY, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const int L = p.L, nt = p.nt, NS = p.nstages;
  const uint32_t proj_bytes = (uint32_t)L * 128u;  // one projection of one unit: 64 x L fp16
  const uint32_t nbuf = (uint32_t)p.nbuf;
  const uint32_t sx = base;
  const uint32_t sy = sx + (p.has_r ? nbuf * proj_bytes : 0u);
  const uint32_t ring = sy + (p.has_c ? nbuf * proj_bytes : 0u);
  const uint32_t bars = ring + (uint32_t)NS * kStageBytes;
  const uint32_t bar_xyf = bars, bar_xye = bars + 16, bar_cf = bars + 32, bar_ce = bars + 48;   // two of each
  const uint32_t bar_rf = bars + 64, bar_re = bars + 80, bar_sf = bars + 96, bar_se = bar_sf + 8 * kMaxStages;
  uint8_t* gen_base = smem_raw + (base - raw);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + (bars - base) + 96 + 16 * kMaxStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_xyf + 8 * i, 1);
      mbar_init(bar_xye + 8 * i, 1);
      mbar_init(bar_cf + 8 * i, 1);
      mbar_init(bar_ce + 8 * i, 4);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_rf + 8 * i, 1);
      mbar_init(bar_re + 8 * i, 4);
    }
    for (int s = 0; s < NS; ++s) {
      mbar_init(bar_sf + 8 * s, 1);
      mbar_init(bar_se + 8 * s, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmS) : "memory");
    if (p.has_r) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmX) : "memory");
    if (p.has_c) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmY) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  const uint32_t tmem_c = tmem_base + 128u;  // column accumulators start after the two row buffers
  grid_dependency_sync();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    uint32_t un = 0, sit = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x, ++un) {
      const uint32_t xb = un % nbuf, xph = (un / nbuf) & 1u;
      const uint32_t xyf = bar_xyf + 8 * xb;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_xye + 8 * xb, xph ^ 1u, 1));
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(xyf, (uint32_t)(p.has_r + p.has_c) * proj_bytes);
        for (int blk = 0; blk < L / 64; ++blk) {
          const int k0 = blk * 64;
          if (p.has_r) {
            const uint32_t dst = sx + xb * proj_bytes + blk * 8192;
            if (!p.x_mn) { if (p.x_swap) tma_load_3d(dst, &tmX, xyf, k0, u, 0); else tma_load_3d(dst, &tmX, xyf, k0, 0, u); }
            else { if (p.x_swap) tma_load_3d(dst, &tmX, xyf, 0, u, k0); else tma_load_3d(dst, &tmX, xyf, 0, k0, u); }
          }
          if (p.has_c) {
            const uint32_t dst = sy + xb * proj_bytes + blk * 8192;
            if (!p.y_mn) { if (p.y_swap) tma_load_3d(dst, &tmY, xyf, k0, u, 0); else tma_load_3d(dst, &tmY, xyf, k0, 0, u); }
            else { if (p.y_swap) tma_load_3d(dst, &tmY, xyf, 0, u, k0); else tma_load_3d(dst, &tmY, xyf, 0, k0, u); }
          }
        }
      }
      __syncwarp();
      for (int jt = 0; jt < nt && ok; ++jt) {
        for (int kc = 0; kc < nt; ++kc, ++sit) {
          const int s = (int)(sit % (uint32_t)NS);
          const uint32_t ph = (sit / (uint32_t)NS) & 1u;
          ok = __all_sync(0xffffffffu, mbar_wait(bar_se + 8 * s, ph ^ 1u, 1));
          if (!ok) break;
          if (lane == 0) {
            const uint32_t full = bar_sf + 8 * s, dst = ring + s * kStageBytes;
            mbar_expect_tx(full, kStageBytes);
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const int k0 = kc * 128 + i * 64, j0 = jt * 128;
              if (p.s_swap) tma_load_3d(dst + i * 16384, &tmS, full, k0, u, j0);
              else tma_load_3d(dst + i * 16384, &tmS, full, k0, j0, u);
            }
          }
          __syncwarp();
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    const uint32_t x_lbo = p.x_mn ? 8192u : 16u, x_step = p.x_mn ? 2048u : 32u;
    const uint32_t y_lbo = p.y_mn ? 8192u : 16u, y_step = p.y_mn ? 2048u : 32u;
    const uint32_t idesc_r = (1u << 4) | SB_IDESC_AB_FMT | ((uint32_t)(p.x_mn ? 1 : 0) << 16) | ((64u >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
    const uint32_t idesc_c = (1u << 4) | SB_IDESC_AB_FMT | (1u << 15) | ((uint32_t)(p.y_mn ? 1 : 0) << 16) | ((64u >> 3) << 17) |
                             ((uint32_t)(kBM >> 4) << 24);
    uint32_t un = 0, sit = 0, rn = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x, ++un) {
      const uint32_t xb = un % nbuf, xph = (un / nbuf) & 1u;
      const uint32_t sxb = sx + xb * proj_bytes, syb = sy + xb * proj_bytes;
      const uint32_t tmem_cb = tmem_c + xb * (uint32_t)nt * 64u;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_xyf + 8 * xb, xph, 2));
      if (!ok) break;
      if (p.has_c) {  // the column accumulators of this set must have been read out by its previous unit
        ok = __all_sync(0xffffffffu, mbar_wait(bar_ce + 8 * xb, xph ^ 1u, 4));
        if (!ok) break;
      }
      for (int jt = 0; jt < nt && ok; ++jt) {
        const uint32_t rb = rn & 1u;
        if (p.has_r) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar_re + 8 * rb, ((rn >> 1) & 1u) ^ 1u, 4));
          if (!ok) break;
        }
        for (int kc = 0; kc < nt; ++kc, ++sit) {
          const int s = (int)(sit % (uint32_t)NS);
          const uint32_t ph = (sit / (uint32_t)NS) & 1u;
          ok = __all_sync(0xffffffffu, mbar_wait(bar_sf + 8 * s, ph, 2));
          if (!ok) break;
          tc_fence_after();
          if (lane == 0) {
            const uint32_t st = ring + s * kStageBytes;
            if (p.has_r) {
#pragma unroll
              for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                  const uint64_t da = make_desc(st + i * 16384 + k * 32, 16u, 1024u);
                  const uint64_t db = make_desc(sxb + (kc * 2 + i) * 8192 + k * x_step, x_lbo, 1024u);
                  umma_f16(tmem_base + rb * 64, da, db, idesc_r, (kc | i | k) != 0 ? 1u : 0u);
                }
            }
            if (p.has_c) {
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                // the same tile as an MN-major operand: M = k index (two 64-wide blocks 16 KiB apart), K = j
                const uint64_t da = make_desc(st + k * 2048, 16384u, 1024u);
                const uint64_t db = make_desc(syb + (jt * 2 + (k >> 2)) * 8192 + (k & 3) * y_step, y_lbo, 1024u);
                umma_f16(tmem_cb + kc * 64, da, db, idesc_c, (jt | k) != 0 ? 1u : 0u);
              }
            }
            umma_commit(bar_se + 8 * s);
          }
          __syncwarp();
        }
        if (p.has_r && ok) {
          if (lane == 0) umma_commit(bar_rf + 8 * rb);
          __syncwarp();
          ++rn;
        }
      }
      if (ok && lane == 0) {
        if (p.has_c) umma_commit(bar_cf + 8 * xb);
        umma_commit(bar_xye + 8 * xb);  // X and Y may be replaced once every MMA of the unit has completed
      }
      __syncwarp();
    }
  } else {
    // ---------------- epilogue warps: thread = one accumulator row ----------------
    const int q = warp & 3;
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    uint32_t un = 0, rn = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < p.units && ok; u += gridDim.x, ++un) {
      if (p.has_r) {
        for (int jt = 0; jt < nt; ++jt, ++rn) {
          const uint32_t rb = rn & 1u;
          ok = __all_sync(0xffffffffu, mbar_wait(bar_rf + 8 * rb, (rn >> 1) & 1u, 3));
          if (!ok) break;
          tc_fence_after();
          uint32_t r[64];
          tmem_ld32_nowait(tmem_base + rb * 64 + lane_off, r);
          tmem_ld32_nowait(tmem_base + rb * 64 + 32 + lane_off, r + 32);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_re + 8 * rb);
          const long long row = (long long)jt * 128 + q * 32 + lane;
          store_row64(p.out_r + (long long)u * p.r_sU + row * p.r_sRow, p.r_sP, r, p.alpha);
        }
        if (!ok) break;
      }
      if (p.has_c) {
        const uint32_t xb = un % nbuf, xph = (un / nbuf) & 1u;
        const uint32_t tmem_cb = tmem_c + xb * (uint32_t)nt * 64u;
        ok = __all_sync(0xffffffffu, mbar_wait(bar_cf + 8 * xb, xph, 3));
        if (!ok) break;
        tc_fence_after();
        for (int kc = 0; kc < nt; ++kc) {
          uint32_t r[64];
          tmem_ld32_nowait(tmem_cb + kc * 64 + lane_off, r);
          tmem_ld32_nowait(tmem_cb + kc * 64 + 32 + lane_off, r + 32);
          tmem_ld_wait();
          if (kc == nt - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_ce + 8 * xb);
          }
          const long long row = (long long)kc * 128 + q * 32 + lane;
          store_row64(p.out_c + (long long)u * p.c_sU + row * p.c_sRow, p.c_sP, r, p.alpha);
        }
      }
    }
  }
  if (*reinterpret_cast<volatile int*>(&g_tc_error) != 0) {
    // a wait ran out somewhere: give copies still in flight time to land before the CTA retires
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace scon
