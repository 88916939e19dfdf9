// Fused attention-score kernels (included by gemm.cu; shares its TMA / tcgen05 helpers).
//
// Forward:  BETA = scale * Q K^T,  ALPHA = softmax_k(BETA),  ATTN_DROP = mask * ALPHA
//           (QKT contraction + Softmax of pytorch_module/encoder.cu:116-120 in one kernel)
// Backward: DATTN_DROP = DGAMMA^T V,  DBETA = ALPHA * (da - sum_k da * ALPHA), da = mask * DATTN_DROP
//           (dX1gamma contraction + BackwardSoftmax of pytorch_module/encoder.cu:250-260)
//
// One CTA owns 128 query rows of one (head, sample) and ALL keys (at most 512): the 128 x L score
// tile is produced by tcgen05.mma into tensor memory (L fp32 columns), where thread r of the four
// epilogue warps owns row r.  Row maximum, row sum and the normalisation are therefore plain
// per-thread loops over TMEM columns, with no shuffles and no second trip through HBM for the
// scores: the forward kernel never reads BETA back, the backward kernel never reads DATTN_DROP
// back.  Outputs leave through 128-byte-swizzled staging rows and TMA stores.
// Requirements: head size 64, sequence length a multiple of 64 and at most 512, score tensors
// dense as [H,B,J,K]; otherwise the caller runs the separate operators.

#pragma once

namespace attn {

constexpr int kMaxL = 512;
constexpr int kStageBytes = kABytes + kMaxL * 128;  // 128 x 64 queries + up to 512 x 64 keys, fp16
constexpr int kStages = 2;
constexpr int kStagingPerWarp = 4 * 4096;           // four 32-row x 128-byte buffers
constexpr int kSmemBytes = kStages * kStageBytes + 4 * kStagingPerWarp + 1024 + 256;

struct Params {
  int L;                 // sequence length (rows and columns of a score tile)
  int tiles_j;           // ceil(L / 128)
  int b_bytes;           // bytes the key/value boxes of one tile deliver (out-of-range rows included)
  long long tiles;       // tiles_j * batch
  int a_mn, b_mn, a_swap, b_swap;
  int swap_o;            // dims 1,2 of the output tensor maps exchanged
  float scale;           // forward: BETA = scale * acc.  backward: 1 (DATTN_DROP = acc)
  Rng rng;               // forward: dropout source
  uint8_t* mask;         // [batch][L][L] bytes
  const __half* alpha;   // backward: softmax output [batch][L][L]
};

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
        "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
        "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Write 64 fp16 values (this thread's part of a row) into a swizzled staging row.
__device__ __forceinline__ void stage_row64(uint8_t* row, int lane, const uint4 v[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) *reinterpret_cast<uint4*>(row + ((i ^ (lane & 7)) << 4)) = v[i];
}

// BWD = false: forward (maps: Q, K; outputs BETA, ALPHA, ATTN_DROP)
// BWD = true : backward (maps: DGAMMA, V; outputs DATTN_DROP, DBETA; the third map is unused)
template <bool BWD>
__global__ void __launch_bounds__(kTcThreads, 1)
attn_scores_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmO0, const __grid_constant__ CUtensorMap tmO1,
                   const __grid_constant__ CUtensorMap tmO2, const Params p) {
  constexpr int S = kStages;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const uint32_t staging = tiles + S * kStageBytes;
  const uint32_t bars = staging + 4 * kStagingPerWarp;  // full[S], empty[S], tmem_full, tmem_empty
  const uint32_t bar_full = bars, bar_empty = bars + 8 * S, bar_tfull = bars + 16 * S, bar_tempty = bars + 16 * S + 8;
  uint8_t* gen_base = smem_raw + (tiles - raw);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + S * kStageBytes + 4 * kStagingPerWarp + 16 * S + 16);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = p.L;
  const int nchunk = (L + 255) / 256;  // MMA column chunks of up to 256 keys

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    mbar_init(bar_tfull, 1);
    mbar_init(bar_tempty, 4);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmO0) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmO1) : "memory");
    if (!BWD) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmO2) : "memory");
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
  grid_dependency_sync();

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    uint32_t it = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++it) {
      const int j0 = (int)(t % p.tiles_j) * 128;
      const int bt = (int)(t / p.tiles_j);
      const int s = it % S;
      const uint32_t ph = (it / S) & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, ph ^ 1u, 1));
      if (!ok) break;
      if (lane == 0) {
        const uint32_t full = bar_full + 8 * s;
        mbar_expect_tx(full, (uint32_t)(kABytes + p.b_bytes));
        const uint32_t sa = tiles + s * kStageBytes, sb_ = sa + kABytes;
        if (!p.a_mn) {
          if (p.a_swap) tma_load_3d(sa, &tmA, full, 0, bt, j0);
          else tma_load_3d(sa, &tmA, full, 0, j0, bt);
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (p.a_swap) tma_load_3d(sa + h * 8192, &tmA, full, j0 + 64 * h, bt, 0);
            else tma_load_3d(sa + h * 8192, &tmA, full, j0 + 64 * h, 0, bt);
          }
        }
        if (!p.b_mn) {
          // boxes of 64 x min(256, L) key rows
          for (int c = 0; c < nchunk; ++c) {
            if (p.b_swap) tma_load_3d(sb_ + c * 32768, &tmB, full, 0, bt, c * 256);
            else tma_load_3d(sb_ + c * 32768, &tmB, full, 0, c * 256, bt);
          }
        } else {
          for (int h = 0; h < L / 64; ++h) {
            if (p.b_swap) tma_load_3d(sb_ + h * 8192, &tmB, full, 64 * h, bt, 0);
            else tma_load_3d(sb_ + h * 8192, &tmB, full, 64 * h, 0, bt);
          }
        }
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
    const uint32_t a_step = p.a_mn ? 2048u : 32u, b_step = p.b_mn ? 2048u : 32u;
    uint32_t it = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++it) {
      const int s = it % S;
      const uint32_t ph = (it / S) & 1u;
      // tensor memory holds one tile: the previous tile must have been read out completely
      ok = __all_sync(0xffffffffu, mbar_wait(bar_tempty, (it & 1u) ^ 1u, 4));
      if (!ok) break;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_full + 8 * s, ph, 2));
      if (!ok) break;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t sa = tiles + s * kStageBytes, sb_ = sa + kABytes;
        for (int c = 0; c < nchunk; ++c) {
          const int width = min(256, L - c * 256);
          const uint32_t idesc = (1u << 4) | ((uint32_t)(p.a_mn ? 1 : 0) << 15) | ((uint32_t)(p.b_mn ? 1 : 0) << 16) |
                                 ((uint32_t)(width >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = make_desc(sa + k * a_step, a_lbo, 1024u);
            const uint64_t db = make_desc(sb_ + c * 32768 + k * b_step, b_lbo, 1024u);
            umma_f16(tmem_base + c * 256, da, db, idesc, k > 0 ? 1u : 0u);
          }
        }
        umma_commit(bar_empty + 8 * s);
        umma_commit(bar_tfull);
      }
      __syncwarp();
    }
  } else {
    // ---------------- softmax / epilogue: thread = one query row ----------------
    const int q = warp & 3;
    const uint32_t my_stage = staging + (uint32_t)(warp - 2) * kStagingPerWarp;
    uint8_t* my_stage_gen = gen_base + S * kStageBytes + (warp - 2) * kStagingPerWarp;
    const float c2 = p.scale * 1.4426950408889634f;
    uint32_t it = 0, ngroup = 0;
    bool ok = true;
    for (long long t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++it) {
      const int j0 = (int)(t % p.tiles_j) * 128;
      const long long bt = t / p.tiles_j;
      ok = __all_sync(0xffffffffu, mbar_wait(bar_tfull, it & 1u, 3));
      if (!ok) break;
      tc_fence_after();
      const int jr = j0 + q * 32;                    // first row of this warp
      const int j = jr + lane;                       // this thread's row
      const bool row_ok = j < L;
      const uint32_t trow = tmem_base + ((uint32_t)(q * 32) << 16);
      const long long row_off = (bt * L + (row_ok ? j : 0)) * (long long)L;   // element offset of the row
      const int nc64 = L / 64;

      if (!BWD) {
        // pass 1: row maximum of t = acc * scale * log2(e)
        float mx = -INFINITY;
        for (int c = 0; c < nc64; ++c) {
          uint32_t r[64];
          tmem_ld32_nowait(trow + c * 64, r);
          tmem_ld32_nowait(trow + c * 64 + 32, r + 32);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 64; ++e) mx = fmaxf(mx, __uint_as_float(r[e]) * c2);
        }
        // pass 2: e = 2^(t - max) back into tensor memory, row sum, BETA out
        float sum = 0.f;
        for (int c = 0; c < nc64; ++c) {
          uint32_t r[64];
          tmem_ld32_nowait(trow + c * 64, r);
          tmem_ld32_nowait(trow + c * 64 + 32, r + 32);
          tmem_ld_wait();
          uint4 beta[8];
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const float a = __uint_as_float(r[v * 8 + e]);
              f[e] = a * p.scale;
              const float ex = exp2f(fmaf(a, c2, -mx));
              sum += ex;
              r[v * 8 + e] = __float_as_uint(ex);
            }
            beta[v] = pack8(f);
          }
          tmem_st32(trow + c * 64, r);
          tmem_st32(trow + c * 64 + 32, r + 32);
          const uint32_t sbuf = ngroup & 1u;
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          __syncwarp();
          stage_row64(my_stage_gen + sbuf * 4096 + lane * 128, lane, beta);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            if (jr < L) {
              if (p.swap_o) tma_store_3d(&tmO0, my_stage + sbuf * 4096, c * 64, (int)bt, jr);
              else tma_store_3d(&tmO0, my_stage + sbuf * 4096, c * 64, jr, (int)bt);
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          ++ngroup;
        }
        tmem_st_wait();
        const float inv = 1.f / sum;
        // pass 3: ALPHA = e / sum, ATTN_DROP = mask * ALPHA
        for (int c = 0; c < nc64; ++c) {
          uint4 mraw[4];
          if (!p.rng.philox && row_ok) {
            const uint4* mp = reinterpret_cast<const uint4*>(p.mask + row_off + c * 64);
#pragma unroll
            for (int i = 0; i < 4; ++i) mraw[i] = mp[i];
          }
          uint32_t r[64];
          tmem_ld32_nowait(trow + c * 64, r);
          tmem_ld32_nowait(trow + c * 64 + 32, r + 32);
          tmem_ld_wait();
          if (c == nc64 - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty);
          }
          if (p.rng.philox) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              uint32_t mm[8];
              philox_keep8(p.rng, (unsigned long long)(row_off + c * 64 + v * 8) >> 3, mm);
              const uint2 pk = mask_pack(mm);
              reinterpret_cast<uint32_t*>(mraw)[2 * v] = pk.x;
              reinterpret_cast<uint32_t*>(mraw)[2 * v + 1] = pk.y;
            }
            if (row_ok) {
              uint4* mp = reinterpret_cast<uint4*>(p.mask + row_off + c * 64);
#pragma unroll
              for (int i = 0; i < 4; ++i) mp[i] = mraw[i];
            }
          }
          uint4 al[8], dr[8];
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            float f[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]) * inv;
            al[v] = pack8(f);
            const uint2 mk = make_uint2(reinterpret_cast<const uint32_t*>(mraw)[2 * v],
                                        reinterpret_cast<const uint32_t*>(mraw)[2 * v + 1]);
            dr[v] = mask_apply(al[v], mk);
          }
          const uint32_t sbuf = ngroup & 1u;
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          __syncwarp();
          stage_row64(my_stage_gen + sbuf * 4096 + lane * 128, lane, al);
          stage_row64(my_stage_gen + (2 + sbuf) * 4096 + lane * 128, lane, dr);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            if (jr < L) {
              if (p.swap_o) {
                tma_store_3d(&tmO1, my_stage + sbuf * 4096, c * 64, (int)bt, jr);
                tma_store_3d(&tmO2, my_stage + (2 + sbuf) * 4096, c * 64, (int)bt, jr);
              } else {
                tma_store_3d(&tmO1, my_stage + sbuf * 4096, c * 64, jr, (int)bt);
                tma_store_3d(&tmO2, my_stage + (2 + sbuf) * 4096, c * 64, jr, (int)bt);
              }
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          ++ngroup;
        }
      } else {
        // backward pass 1: da = mask * acc (kept in tensor memory), s = sum da * alpha, DATTN_DROP out
        float ssum = 0.f;
        for (int c = 0; c < nc64; ++c) {
          uint4 mraw[4], araw[8];
          if (row_ok) {
            const uint4* mp = reinterpret_cast<const uint4*>(p.mask + row_off + c * 64);
            const uint4* ap = reinterpret_cast<const uint4*>(p.alpha + row_off + c * 64);
#pragma unroll
            for (int i = 0; i < 4; ++i) mraw[i] = mp[i];
#pragma unroll
            for (int i = 0; i < 8; ++i) araw[i] = ap[i];
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) mraw[i] = make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int i = 0; i < 8; ++i) araw[i] = make_uint4(0, 0, 0, 0);
          }
          uint32_t r[64];
          tmem_ld32_nowait(trow + c * 64, r);
          tmem_ld32_nowait(trow + c * 64 + 32, r + 32);
          tmem_ld_wait();
          uint4 dad[8];
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            float f[8], a8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]);
            dad[v] = pack8(f);   // DATTN_DROP as stored (fp16)
            const uint2 mk = make_uint2(reinterpret_cast<const uint32_t*>(mraw)[2 * v],
                                        reinterpret_cast<const uint32_t*>(mraw)[2 * v + 1]);
            // continue from the fp16 value, as the separate softmax-backward operator would
            unpack8(mask_apply(dad[v], mk), f);
            unpack8(araw[v], a8);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              ssum = fmaf(f[e], a8[e], ssum);
              r[v * 8 + e] = __float_as_uint(f[e]);
            }
          }
          tmem_st32(trow + c * 64, r);
          tmem_st32(trow + c * 64 + 32, r + 32);
          const uint32_t sbuf = ngroup & 1u;
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          __syncwarp();
          stage_row64(my_stage_gen + sbuf * 4096 + lane * 128, lane, dad);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            if (jr < L) {
              if (p.swap_o) tma_store_3d(&tmO0, my_stage + sbuf * 4096, c * 64, (int)bt, jr);
              else tma_store_3d(&tmO0, my_stage + sbuf * 4096, c * 64, jr, (int)bt);
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          ++ngroup;
        }
        tmem_st_wait();
        // backward pass 2: DBETA = alpha * (da - s)
        for (int c = 0; c < nc64; ++c) {
          uint4 araw[8];
          if (row_ok) {
            const uint4* ap = reinterpret_cast<const uint4*>(p.alpha + row_off + c * 64);
#pragma unroll
            for (int i = 0; i < 8; ++i) araw[i] = ap[i];
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) araw[i] = make_uint4(0, 0, 0, 0);
          }
          uint32_t r[64];
          tmem_ld32_nowait(trow + c * 64, r);
          tmem_ld32_nowait(trow + c * 64 + 32, r + 32);
          tmem_ld_wait();
          if (c == nc64 - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_tempty);
          }
          uint4 db[8];
#pragma unroll
          for (int v = 0; v < 8; ++v) {
            float f[8], a8[8];
            unpack8(araw[v], a8);
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = a8[e] * (__uint_as_float(r[v * 8 + e]) - ssum);
            db[v] = pack8(f);
          }
          const uint32_t sbuf = ngroup & 1u;
          if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
          __syncwarp();
          stage_row64(my_stage_gen + sbuf * 4096 + lane * 128, lane, db);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            if (jr < L) {
              if (p.swap_o) tma_store_3d(&tmO1, my_stage + sbuf * 4096, c * 64, (int)bt, jr);
              else tma_store_3d(&tmO1, my_stage + sbuf * 4096, c * 64, jr, (int)bt);
            }
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          }
          ++ngroup;
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
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace attn
