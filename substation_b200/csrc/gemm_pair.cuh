// Paired-CTA variant of the tcgen05 contraction kernel (included by gemm.cu).
//
// Two CTAs on neighbouring SMs form a cluster and compute one 256 x 256 output
// tile with tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and
// its own 128 rows (= half) of B, the tensor cores of both SMs read both halves
// of B, and each CTA's tensor memory receives its 128 x 256 part of the
// accumulator.  Per CTA and 64-wide K block that is 32 KiB of operands for
// 128 x 256 x 64 multiply-adds, against 48 KiB for the single-CTA kernel, with
// every CTA still fetching only its own tiles.
//
// Roles per CTA: warp 0 TMA producer, warp 1 tensor-memory allocation (+ MMA
// issue in the leader CTA, rank 0), warps 2-5 epilogue.  Barriers:
//   full[s]      leader only; the leader's producer arms it with the bytes of BOTH
//                CTAs, the peer's bulk loads complete on it too;
//   empty[s]     one per CTA; the leader's MMA thread commits to its own and to
//                the peer's when the stage has been read;
//   acc_full[b]  one per CTA (leader commits to both); acc_empty[b] leader only,
//                8 arrivals (4 epilogue warps of each CTA).
// Remote barrier addresses come from mapa.  Waits are bounded like in the
// single-CTA kernel.

#pragma once

namespace pair {

constexpr int kBN = 256;
constexpr int kHalfBBytes = 128 * kBK * 2;                 // this CTA's half of B per K block
constexpr int kStageBytes = kABytes + kHalfBBytes;         // 32 KiB
constexpr int kTmemCols = 512;                             // two 256-column accumulators

// EW epilogue warps per CTA: 4 (one per 32-lane quadrant of tensor memory, each draining all 256 columns of its
// rows) or 8 (two per quadrant, 128 columns each: the drain of a tile, which nothing overlaps when a cluster has
// a single tile, takes half as long).  Each epilogue warp owns two 4 KiB staging buffers, so the eight-warp
// form keeps five operand stages instead of six.
template <int EW>
struct Cfg {
  static constexpr int kThreads = 64 + 32 * EW;
  static constexpr int kStages = EW == 8 ? 5 : 6;
  static constexpr int kTileBytes = kStages * kStageBytes;
  static constexpr int kStageOut = EW * 2 * 4096;
  static constexpr int kSmemBytes = kTileBytes + kStageOut + 1024 + 256;
};

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// bulk tensor load of this CTA's tile whose completion bytes are counted on a barrier of the leader
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster,
                                                 int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                              uint32_t accumulate) {
  const uint32_t z = 0;
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
      " tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(z) : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar_cluster) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster) : "memory");
}

// Persistent: cluster c works on pair tiles c, c + (#clusters), ...; n fastest, then m (256 rows), then batch.
// EPI: 0 plain, else EpiParams::kind (extra outputs through tmC2 / tmC3, TMA-store mode only).
template <int EPI, int EW>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Cfg<EW>::kThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmC2,
                    const __grid_constant__ CUtensorMap tmC3, const TcParams p) {
  using C = Cfg<EW>;
  constexpr int S = C::kStages;
  constexpr int kTileBytes = C::kTileBytes;
  constexpr int kChunks = (kBN / 64) * 4 / EW;       // 64-column chunks each epilogue warp drains per tile
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const uint32_t stage_out = tiles + kTileBytes;
  const uint32_t bars = stage_out + C::kStageOut;  // full[S], empty[S], acc_full[2], acc_empty[2]
  const uint32_t bar_full = bars, bar_empty = bars + 8 * S;
  const uint32_t bar_accf = bars + 16 * S, bar_acce = bars + 16 * S + 16;
  uint8_t* gen_base = smem_raw + (tiles - raw);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + kTileBytes + C::kStageOut + 16 * S + 32);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();          // 0 = leader
  const unsigned cluster_id = blockIdx.x >> 1, nclusters = gridDim.x >> 1;
  const int KT = (int)((p.K + kBK - 1) / kBK);

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_accf + 8 * b, 1);
      mbar_init(bar_acce + 8 * b, 2 * EW);  // the epilogue warps of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    if (p.c_mode == 2) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmC) : "memory");
    if (EPI != 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmC2) : "memory");
    if (EPI == 3) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmC3) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  cluster_sync_all();   // barriers of both CTAs are initialised before anyone signals them
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);
  grid_dependency_sync();

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    const uint32_t leader_full = map_to_rank(bar_full, 0);
    uint32_t it = 0;
    bool ok = true;
    for (long long t = cluster_id; t < p.tiles && ok; t += nclusters) {
      const int n0 = (int)(t % p.tiles_n) * kBN + (int)rank * 128;       // this CTA's half of B
      const int m0 = (int)((t / p.tiles_n) % p.tiles_m) * 256 + (int)rank * 128;
      const int bt = (int)(t / ((long long)p.tiles_n * p.tiles_m));
      for (int kb = 0; kb < KT; ++kb, ++it) {
        const int s = it % S;
        const uint32_t ph = (it / S) & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, ph ^ 1u, 1));
        if (!ok) break;
        if (lane == 0) {
          const uint32_t full = leader_full + 8 * s;
          if (rank == 0) mbar_expect_tx(bar_full + 8 * s, 2u * (uint32_t)kStageBytes);
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
    }
  } else if (warp == 1) {
    if (rank == 0) {
      // ---------------- MMA issuer (leader CTA only; lane 0 issues) ----------------
      // instruction descriptor: fp32 accumulate, fp16 operands, majors, N = 256, M = 256 across the pair
      const uint32_t idesc = (1u << 4) | SB_IDESC_AB_FMT | ((uint32_t)(p.a_mn ? 1 : 0) << 15) |
                             ((uint32_t)(p.b_mn ? 1 : 0) << 16) | ((uint32_t)(kBN >> 3) << 17) |
                             ((uint32_t)(256 >> 4) << 24);
      const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
      const uint32_t a_step = p.a_mn ? 2048u : 32u, b_step = p.b_mn ? 2048u : 32u;
      const uint32_t peer_empty = map_to_rank(bar_empty, 1), peer_accf = map_to_rank(bar_accf, 1);
      // One thread runs the whole issue loop (no warp-wide votes on its path), and the shared-memory
      // descriptors are a base plus an address increment: the MMA issue rate of this thread is what
      // bounds the kernel once the operands arrive in time.
      if (lane == 0) {
        const uint64_t da_base = make_desc(tiles, a_lbo, 1024u), db_base = make_desc(tiles + kABytes, b_lbo, 1024u);
        const uint64_t a_inc = a_step >> 4, b_inc = b_step >> 4, stage_inc = (uint64_t)kStageBytes >> 4;
        uint32_t it = 0, lt = 0;
        bool ok = true;
        for (long long t = cluster_id; t < p.tiles && ok; t += nclusters, ++lt) {
          const uint32_t buf = lt & 1u, aph = (lt >> 1) & 1u;
          ok = mbar_wait(bar_acce + 8 * buf, aph ^ 1u, 4);
          if (!ok) break;
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + buf * kBN;
          for (int kb = 0; kb < KT; ++kb, ++it) {
            const uint32_t s = it % S;
            const uint32_t ph = (it / S) & 1u;
            ok = mbar_wait(bar_full + 8 * s, ph, 2);
            if (!ok) break;
            tc_fence_after();
            const uint64_t da = da_base + s * stage_inc, db = db_base + s * stage_inc;
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k)
              umma_f16_pair(tmem_d, da + k * a_inc, db + k * b_inc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            // the stage is free in both CTAs once these MMAs have read it
            umma_commit_pair(bar_empty + 8 * s);
            umma_commit_pair(peer_empty + 8 * s);
          }
          if (ok) {
            umma_commit_pair(bar_accf + 8 * buf);
            umma_commit_pair(peer_accf + 8 * buf);
          }
        }
      }
      __syncwarp();
    }
  } else {
    // ---------------- epilogue (both CTAs; each stores its own 128 rows) ----------------
    const int q = warp & 3;                    // the 32-lane quadrant of tensor memory this warp may read
    const int c_first = ((warp - 2) >> 2) * kChunks;   // its share of the tile's four 64-column chunks
    const uint32_t leader_acce = map_to_rank(bar_acce, 0);
    const uint32_t my_stage = stage_out + (uint32_t)(warp - 2) * 8192u;
    uint8_t* my_stage_gen = gen_base + kTileBytes + (warp - 2) * 8192;
    uint32_t lt = 0, nstore = 0;
    bool ok = true;
    for (long long t = cluster_id; t < p.tiles && ok; t += nclusters, ++lt) {
      const int n0 = (int)(t % p.tiles_n) * kBN;
      const int m0 = (int)((t / p.tiles_n) % p.tiles_m) * 256 + (int)rank * 128;
      const long long bt = t / ((long long)p.tiles_n * p.tiles_m);
      const uint32_t buf = lt & 1u, aph = (lt >> 1) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_accf + 8 * buf, aph, 3));
      if (!ok) break;
      tc_fence_after();
      const long long m = (long long)m0 + q * 32 + lane;
      const uint32_t tsrc = tmem_base + buf * kBN + ((uint32_t)(q * 32) << 16);
      if (p.c_mode == 2) {
#pragma unroll 1
        for (int c = c_first; c < c_first + kChunks; ++c) {
          uint32_t r[64];
          tmem_ld32_nowait(tsrc + (uint32_t)(c * 64), r);
          tmem_ld32_nowait(tsrc + (uint32_t)(c * 64 + 32), r + 32);
          tmem_ld_wait();
          if (c == c_first + kChunks - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_acce + 8 * buf);
          }
          const int nc = n0 + c * 64, mc = m0 + q * 32;
          const bool in_range = nc < p.N && mc < p.M;
          // stage 8 x 16 bytes of this thread's row and store the warp's 32 x 64 block through `map`
          auto put = [&](const CUtensorMap* map, const uint4* v8) {
            const uint32_t sbuf = nstore & 1u;
            // the store issued two blocks ago must have finished reading this buffer
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
            uint8_t* row = my_stage_gen + sbuf * 4096 + lane * 128;
#pragma unroll
            for (int v = 0; v < 8; ++v) *reinterpret_cast<uint4*>(row + ((v ^ (lane & 7)) << 4)) = v8[v];
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0 && in_range) {
              if (p.c_swap) tma_store_3d(map, my_stage + sbuf * 4096, nc, (int)bt, mc);
              else tma_store_3d(map, my_stage + sbuf * 4096, nc, mc, (int)bt);
            }
            if (lane == 0) asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            ++nstore;
          };
          // side inputs of the fused work: requested before the arithmetic on the accumulator
          uint4 side[8];
          uint2 mk[8];
          const bool row_ok = m < p.M && nc < p.N;
          if (EPI == 1 || EPI == 3) {
            if (p.epi.vec_along_m) {
              const sb_half2 b2 = sb_h2h2(m < p.M ? p.epi.vec[m] : sb_f2h(0.f));
              const uint32_t w = *reinterpret_cast<const uint32_t*>(&b2);
#pragma unroll
              for (int v = 0; v < 8; ++v) side[v] = make_uint4(w, w, w, w);
            } else if (nc < p.N) {
#pragma unroll
              for (int v = 0; v < 8; ++v) side[v] = *reinterpret_cast<const uint4*>(p.epi.vec + nc + 8 * v);
            }
          }
          if (EPI == 2 && row_ok) {
            const sb_half* rp = p.epi.resid + m * p.sCm + nc;
#pragma unroll
            for (int v = 0; v < 8; ++v) side[v] = *reinterpret_cast<const uint4*>(rp + 8 * v);
          }
          if (EPI == 3 && !p.epi.rng.philox && row_ok) {
            const uint8_t* kp = p.epi.mask + m * p.sCm + nc;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const uint4 t4 = *reinterpret_cast<const uint4*>(kp + 16 * v);
              mk[2 * v] = make_uint2(t4.x, t4.y);
              mk[2 * v + 1] = make_uint2(t4.z, t4.w);
            }
          }
          uint4 o1[8];
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]) * p.alpha;
            o1[v] = pack8(f);
          }
          if (EPI == 0 || !p.epi.skip_c) put(&tmC, o1);
          if (EPI == 1 || EPI == 2) {
#pragma unroll
            for (int v = 0; v < 8; ++v) o1[v] = hadd8(o1[v], side[v]);
            put(&tmC2, o1);
          }
          if (EPI == 3) {
#pragma unroll
            for (int v = 0; v < 8; ++v) o1[v] = hadd8(o1[v], side[v]);   // the biased pre-activation
            put(&tmC2, o1);
            if (p.epi.rng.philox) {
              // keep flags of the logical elements (m, nc + 8v ..): C is dense in logical order, so the
              // element index is the memory offset
#pragma unroll
              for (int v = 0; v < 8; ++v) {
                uint32_t mm[8];
                philox_keep8(p.epi.rng, (unsigned long long)(m * p.sCm + nc + 8 * v) >> 3, mm);
                mk[v] = mask_pack(mm);
              }
              if (row_ok) {
                uint8_t* kp = p.epi.mask + m * p.sCm + nc;
#pragma unroll
                for (int v = 0; v < 4; ++v)
                  *reinterpret_cast<uint4*>(kp + 16 * v) = make_uint4(mk[2 * v].x, mk[2 * v].y, mk[2 * v + 1].x, mk[2 * v + 1].y);
              }
            }
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              uint4 a;
              if (p.epi.activation == SB_ACT_RELU) {
                const sb_half2* h = reinterpret_cast<const sb_half2*>(&o1[v]);
                sb_half2* qq = reinterpret_cast<sb_half2*>(&a);
                const sb_half2 zero = sb_f2h2_dup(0.f);
#pragma unroll
                for (int i = 0; i < 4; ++i) qq[i] = __hmax2(h[i], zero);
              } else {
                float x[8];
                unpack8(o1[v], x);
#pragma unroll
                for (int e = 0; e < 8; ++e) x[e] = act_fwd(x[e], SB_ACT_GELU);
                a = pack8(x);
              }
              o1[v] = mask_apply(a, mk[v]);
            }
            put(&tmC3, o1);
          }
        }
      } else {
        sb_half* crow = reinterpret_cast<sb_half*>(p.C) + bt * p.sCb + m * p.sCm;
#pragma unroll 1
        for (int c = 2 * c_first; c < 2 * (c_first + kChunks); ++c) {
          uint32_t r[32];
          tmem_ld32_nowait(tsrc + (uint32_t)(c * 32), r);
          tmem_ld_wait();
          if (c == 2 * (c_first + kChunks) - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(leader_acce + 8 * buf);
          }
          if (m < p.M) {
            const long long nb = (long long)n0 + c * 32;
            if (p.c_mode == 1) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                if (nb + v * 8 < p.N) {
                  float f[8];
#pragma unroll
                  for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]) * p.alpha;
                  *reinterpret_cast<uint4*>(crow + nb + v * 8) = pack8(f);
                }
              }
            } else {
#pragma unroll
              for (int e = 0; e < 32; ++e)
                if (nb + e < p.N) crow[(nb + e) * p.sCn] = sb_f2h(__uint_as_float(r[e]) * p.alpha);
            }
          }
        }
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __syncwarp();
  }
  if (*reinterpret_cast<volatile int*>(&g_tc_error) != 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(1000);
  }
  tc_fence_before();
  cluster_sync_all();   // neither CTA may leave (or free tensor memory) while its peer can still reach it
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols) : "memory");
  }
}

}  // namespace pair
