// Split-K form of the paired-CTA contraction kernel for outputs of few tiles and long K (included by gemm.cu
// after gemm_pair.cuh; the weight gradient of the attention output projection is 16 tiles with K = all tokens).
//
// One cluster of 2 SK CTAs per 256 x 256 output tile: SK CTA pairs (2 to 4), pair i taking the i-th part of K
// through the same TMA ring and tcgen05.mma.cta_group::2 main loop as the plain kernel.  The partial accumulators
// never go to global memory: every CTA copies its 128 x 256 fp32 part from tensor memory into its own shared memory
// (the operand ring is free by then), the cluster synchronises, and the SK CTAs that hold one row half each add up a
// contiguous share of it, reading their peers through distributed shared memory, in the fixed order pair 0..SK-1.
// One launch, no workspace, deterministic.
// Requirements: C with unit stride along N, rows 8-byte aligned (N and the row pitch multiples of 4), one batch.

#pragma once

namespace pair {

constexpr int kPartialPitch = kBN * 4 + 16;      // bytes per row of the fp32 partial in shared memory: the 16 spare
                                                 // bytes spread the 32 rows a warp writes over all banks

__device__ __forceinline__ float4 ld_cluster_f4(uint32_t cluster_addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(cluster_addr) : "memory");
  return v;
}

// SK = CTA pairs per cluster (2 or 4), each taking 1/SK of K
template <int EW, int SK>
__global__ void __cluster_dims__(2 * SK, 1, 1) __launch_bounds__(Cfg<EW>::kThreads, 1)
gemm_tc_pair_splitk_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                           const TcParams p) {
  using C = Cfg<EW>;
  constexpr int S = C::kStages;
  constexpr int kTileBytes = C::kTileBytes;
  static_assert(128 * kPartialPitch <= kTileBytes, "the fp32 partial must fit into the operand ring");
  static_assert(EW == 8, "the reduction is laid out for eight epilogue warps");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const uint32_t bars = tiles + kTileBytes + C::kStageOut;  // full[S], empty[S], acc_full
  const uint32_t bar_full = bars, bar_empty = bars + 8 * S, bar_accf = bars + 16 * S;
  uint8_t* gen_base = smem_raw + (tiles - raw);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + kTileBytes + C::kStageOut + 16 * S + 32);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const uint32_t half = rank & 1u;               // which 128 rows of the tile (and which half of B) this CTA stages
  const uint32_t pi = rank >> 1;                 // pair index = K quarter
  const uint32_t leader = rank & ~1u;            // the even CTA of the pair issues the MMAs
  const long long t = blockIdx.x / (2 * SK);
  const int KT = (int)((p.K + kBK - 1) / kBK);
  const int kb_begin = min(KT, (int)pi * p.kt_per_split), kb_end = min(KT, kb_begin + p.kt_per_split);
  const int n_tile = (int)(t % p.tiles_n) * kBN;
  const int m_tile = (int)((t / p.tiles_n) % p.tiles_m) * 256;
  const int bt = (int)(t / ((long long)p.tiles_n * p.tiles_m));

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_accf, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kBN) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();   // every CTA's barriers are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  grid_dependency_sync();

  if (warp == 0) {
    // ---------------- TMA producer: this pair's quarter of K ----------------
    const uint32_t leader_full = map_to_rank(bar_full, leader);
    const int n0 = n_tile + (int)half * 128, m0 = m_tile + (int)half * 128;
    uint32_t it = 0;
    for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
      const int s = it % S;
      const uint32_t ph = (it / S) & 1u;
      if (!__all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, ph ^ 1u, 1))) break;
      if (lane == 0) {
        const uint32_t full = leader_full + 8 * s;
        if (half == 0) mbar_expect_tx(bar_full + 8 * s, 2u * (uint32_t)kStageBytes);
        const uint32_t sa = tiles + s * kStageBytes, sb_ = sa + kABytes;
        const int k0 = kb * kBK;
        if (!p.a_mn) {
          if (p.a_swap) tma_load_3d_pair(sa, &tmA, full, k0, bt, m0);
          else tma_load_3d_pair(sa, &tmA, full, k0, m0, bt);
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (p.a_swap) tma_load_3d_pair(sa + h * 8192, &tmA, full, m0 + 64 * h, bt, k0);
            else tma_load_3d_pair(sa + h * 8192, &tmA, full, m0 + 64 * h, k0, bt);
          }
        }
        if (!p.b_mn) {
          if (p.b_swap) tma_load_3d_pair(sb_, &tmB, full, k0, bt, n0);
          else tma_load_3d_pair(sb_, &tmB, full, k0, n0, bt);
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (p.b_swap) tma_load_3d_pair(sb_ + h * 8192, &tmB, full, n0 + 64 * h, bt, k0);
            else tma_load_3d_pair(sb_ + h * 8192, &tmB, full, n0 + 64 * h, k0, bt);
          }
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    if (half == 0 && lane == 0) {
      // ---------------- MMA issuer (even CTA of the pair) ----------------
      const uint32_t idesc = (1u << 4) | SB_IDESC_AB_FMT | ((uint32_t)(p.a_mn ? 1 : 0) << 15) |
                             ((uint32_t)(p.b_mn ? 1 : 0) << 16) | ((uint32_t)(kBN >> 3) << 17) |
                             ((uint32_t)(256 >> 4) << 24);
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
      const uint32_t a_step = p.a_mn ? 2048u : 32u, b_step = p.b_mn ? 2048u : 32u;
      const uint32_t peer_empty = map_to_rank(bar_empty, leader + 1), peer_accf = map_to_rank(bar_accf, leader + 1);
      const uint64_t da_base = make_desc(tiles, a_lbo, 1024u), db_base = make_desc(tiles + kABytes, b_lbo, 1024u);
      const uint64_t a_inc = a_step >> 4, b_inc = b_step >> 4, stage_inc = (uint64_t)kStageBytes >> 4;
      uint32_t it = 0;
      bool ok = true;
      for (int kb = kb_begin; kb < kb_end; ++kb, ++it) {
        const uint32_t s = it % S;
        const uint32_t ph = (it / S) & 1u;
        ok = mbar_wait(bar_full + 8 * s, ph, 2);
        if (!ok) break;
        tc_fence_after();
        const uint64_t da = da_base + s * stage_inc, db = db_base + s * stage_inc;
#pragma unroll
        for (int k = 0; k < kBK / 16; ++k)
          umma_f16_pair(tmem_base, da + k * a_inc, db + k * b_inc, idesc, (it > 0 || k > 0) ? 1u : 0u);
        umma_commit_pair(bar_empty + 8 * s);
        umma_commit_pair(peer_empty + 8 * s);
      }
      if (ok) {
        umma_commit_pair(bar_accf);
        umma_commit_pair(peer_accf);
      }
    }
    __syncwarp();
  } else {
    // ---------------- this CTA's 128 x 256 partial: tensor memory -> shared memory (fp32) ----------------
    const int q = warp & 3;                        // the 32-lane quadrant of tensor memory this warp may read
    const int col0 = ((warp - 2) >> 2) * 128;      // its 128 of the 256 columns
    const bool ok = __all_sync(0xffffffffu, mbar_wait(bar_accf, 0u, 3));
    tc_fence_after();
    if (ok) {
      const uint32_t tsrc = tmem_base + ((uint32_t)(q * 32) << 16);
      uint8_t* prow = gen_base + (q * 32 + lane) * kPartialPitch;
#pragma unroll 1
      for (int c = col0; c < col0 + 128; c += 64) {
        uint32_t r[64];
        tmem_ld32_nowait(tsrc + (uint32_t)c, r);
        tmem_ld32_nowait(tsrc + (uint32_t)(c + 32), r + 32);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 16; ++v)
          *reinterpret_cast<uint4*>(prow + (c + 4 * v) * 4) = make_uint4(r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
      }
    }
  }
  tc_fence_before();
  cluster_sync_all();   // all eight partials are in shared memory (release / acquire at cluster scope)
  if (warp >= 2 && *reinterpret_cast<volatile int*>(&g_tc_error) == 0) {
    // ---------------- reduction: this CTA's share of its row half ----------------
    const int tid = threadIdx.x - 64;              // 0 .. 255
    uint32_t src[SK];
#pragma unroll
    for (int j = 0; j < SK; ++j) src[j] = map_to_rank(tiles, half + 2u * (uint32_t)j);
    sb_half* cbase = reinterpret_cast<sb_half*>(p.C) + (long long)bt * p.sCb;
    // the row half's 128 x 64 pieces of four columns are dealt out to the SK CTAs that hold it, a contiguous range
    // each; a thread asks for the SK parts of four pieces before it adds any, so that 4 SK remote loads are in flight
    constexpr int kItems = 128 * (kBN / 4), kPer = (kItems + SK - 1) / SK, kBatch = 4;
    const int first = (int)pi * kPer, last = min(kItems, first + kPer);
    for (int base = first + tid; base < last; base += 256 * kBatch) {
      float4 v[kBatch][SK];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int item = min(base + u * 256, last - 1);       // past the end: a valid address, result unused
        const uint32_t off = (uint32_t)((item / (kBN / 4)) * kPartialPitch + (item % (kBN / 4)) * 16);
#pragma unroll
        for (int j = 0; j < SK; ++j) v[u][j] = ld_cluster_f4(src[j] + off);
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int item = base + u * 256;
        if (item >= last) break;
        const int row = item / (kBN / 4), col = (item % (kBN / 4)) * 4;
        float4 acc = v[u][0];
#pragma unroll
        for (int j = 1; j < SK; ++j) {
          acc.x += v[u][j].x; acc.y += v[u][j].y; acc.z += v[u][j].z; acc.w += v[u][j].w;
        }
        const long long m = (long long)m_tile + half * 128 + row, n = (long long)n_tile + col;
        if (m < p.M && n < p.N) {
          const sb_half2 lo = sb_f2h2(acc.x * p.alpha, acc.y * p.alpha);
          const sb_half2 hi = sb_f2h2(acc.z * p.alpha, acc.w * p.alpha);
          uint2 o;
          o.x = *reinterpret_cast<const uint32_t*>(&lo);
          o.y = *reinterpret_cast<const uint32_t*>(&hi);
          *reinterpret_cast<uint2*>(cbase + m * p.sCm + n) = o;
        }
      }
    }
  }
  if (*reinterpret_cast<volatile int*>(&g_tc_error) != 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  cluster_sync_all();   // no CTA leaves (or frees tensor memory) while a peer may still read its shared memory
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kBN) : "memory");
  }
}

}  // namespace pair
