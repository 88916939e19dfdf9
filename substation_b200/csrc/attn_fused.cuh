// Fused attention-score kernels (included by gemm.cu; shares its TMA / tcgen05 helpers).
//
// Forward:  BETA = scale * Q K^T,  ALPHA = softmax_k(BETA),  ATTN_DROP = mask * ALPHA
//           (QKT contraction + Softmax of pytorch_module/encoder.cu:116-120 in one kernel)
// Backward: DATTN_DROP = DGAMMA^T V,  DBETA = ALPHA * (da - sum_k da * ALPHA), da = mask * DATTN_DROP
//           (dX1gamma contraction + BackwardSoftmax of pytorch_module/encoder.cu:250-260)
//
// One CTA owns 128 query rows of one (head, sample) and ALL keys (at most 512): the 128 x L score
// tile is produced by tcgen05.mma into tensor memory (L fp32 columns).  Eight epilogue warps read it
// back: two per 32-lane quadrant of tensor memory, thread = one query row, the two warps of a
// quadrant taking alternate 64-key chunks and exchanging their partial row maximum / row sums
// through shared memory.  The forward softmax is an online one: the first pass exponentiates every
// 32-key piece against the row maximum seen so far (rescaling the running sum when it rises) and
// leaves the exponentials in tensor memory, the second brings each piece to the final maximum while
// it normalises and writes; a separate maximum pass over the tile is not needed.  The scores never make a second trip through HBM: the forward kernel
// does not read BETA back, the backward kernel does not read DATTN_DROP back (it keeps
// (mask*dattn_drop, alpha) as an fp16 pair per tensor-memory word between its two passes).
// Inputs that stream per row (the dropout mask, ALPHA in the backward kernel) arrive through
// per-warp TMA slots, outputs leave through swizzled staging rows and TMA stores, so every HBM
// access is a full 64- or 128-byte row segment.
// Requirements: head size 64, sequence length a multiple of 64 and at most 512, score tensors
// dense as [H,B,J,K], scale > 0; otherwise the caller runs the separate operators.

#pragma once

namespace attn {

constexpr int kMaxL = 512;
constexpr int kNW = 2;                               // epilogue warps per tensor-memory quadrant
constexpr int kEpiWarps = 4 * kNW;
constexpr int kThreads = 64 + 32 * kEpiWarps;        // producer warp, MMA warp, epilogue warps
constexpr int kOperandBytes = kABytes + kMaxL * 128; // 128 x 64 queries + up to 512 x 64 keys, fp16
constexpr int kRedBytes = 2 * 2 * kNW * 128 * 4;     // partial row maxima and row sums, two sets used by alternate tiles
constexpr int kRefBytes = 8 * kEpiWarps * 32 * 4;    // forward: the maximum each 32-column piece of a row was scaled by

template <bool BWD>
struct Cfg {
  // Shared memory left after the operands is split between output staging and input slots where the kernel
  // stalls most: the forward kernel issues two stores per chunk and reads 2 KiB of mask, the backward kernel reads
  // 6 KiB (ALPHA and mask) per chunk and issues one store; a second input slot bought the backward kernel 4.5 us
  // of 51, the second staging buffer it gave up cost 1 us.
  static constexpr int kOutBufs = BWD ? 1 : 3;       // staging buffers (32 rows x 128 B) per warp
  static constexpr int kInSlot = BWD ? 6144 : 2048;  // ALPHA rows (4 KiB) + mask rows (2 KiB) | mask rows
  static constexpr int kSlots = 2;                   // input chunks in flight per warp
  static constexpr int kStaging = kEpiWarps * kOutBufs * 4096;
  static constexpr int kSmemBytes = kOperandBytes + kStaging + kEpiWarps * kInSlot * kSlots + kRedBytes + (BWD ? 0 : kRefBytes) + 1024 + 256;
};

struct Params {
  int L;                 // sequence length (rows and columns of a score tile)
  int tiles_j;           // ceil(L / 128)
  int b_bytes;           // bytes the key/value boxes of one tile deliver (out-of-range rows included)
  int tiles;             // tiles_j * batch
  int a_mn, b_mn, a_swap, b_swap;
  int swap_o;            // dims 1,2 of the score tensor maps exchanged
  float scale;           // forward: BETA = scale * acc.  backward: unused (DATTN_DROP = acc)
  Rng rng;               // forward: dropout source
  uint8_t* mask;         // [batch][L][L] bytes (written directly when the mask is generated here)
  int prefetch;          // producer warp asks for the row inputs of the next tile to be brought into L2
  int skip_o0;           // the first score output (BETA forward, DATTN_DROP backward) is not wanted: never stored
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

// Wait for the outstanding tensor-memory loads; the registers are operands so that no use of them
// can be scheduled above the wait.
__device__ __forceinline__ void tmem_ld_wait32(uint32_t* r) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :: "memory");
}

// Walk this warp's 64-column chunks (c = first, first + kNW, ... < end) in 32-column halves, keeping
// the tensor-memory load of the next half in flight while f(c, half, r) works on the current one.
template <class F>
__device__ __forceinline__ void sweep(uint32_t trow, int first, int end, F&& f) {
  if (first >= end) return;
  uint32_t ra[32], rb[32];
  tmem_ld32_nowait(trow + first * 64, ra);
  for (int c = first; c < end; c += kNW) {
    tmem_ld_wait32(ra);
    tmem_ld32_nowait(trow + c * 64 + 32, rb);
    f(c, 0, ra);
    tmem_ld_wait32(rb);
    if (c + kNW < end) tmem_ld32_nowait(trow + (c + kNW) * 64, ra);
    f(c, 1, rb);
  }
}

// The same walk, one 256-column half of tensor memory at a time (the MMAs fill and the last pass
// releases the halves separately): pre(half) runs before the first read of a half, post(half) after
// the last.
template <class Pre, class Post, class F>
__device__ __forceinline__ void sweep_halves(uint32_t trow, int h, int nc64, Pre&& pre, Post&& post, F&& f) {
  for (int hf = 0; hf * 4 < nc64; ++hf) {
    pre(hf);
    sweep(trow, hf * 4 + h, min(nc64, hf * 4 + 4), f);
    post(hf);
  }
}

// Barrier among the epilogue warps with a bounded wait (one arrival per warp).
__device__ __forceinline__ bool epi_barrier(uint32_t bar, uint32_t& uses, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
  const bool ok = mbar_wait(bar, uses & 1u, 6);
  ++uses;
  return __all_sync(0xffffffffu, ok);
}

// 2^x for x <= 0 on the special-function unit (results below 2^-126 flush to zero)
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Ask for a box to be brought into L2 (no shared-memory destination, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* map, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(map), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }

// BWD = false: forward  (maps: Q, K; score maps: BETA, ALPHA, ATTN_DROP; tmI unused)
// BWD = true : backward (maps: DGAMMA, V; score maps: DATTN_DROP, DBETA, -; tmI = ALPHA)
// tmM: the mask as a byte tensor (read when it is an input).
template <bool BWD>
__global__ void __launch_bounds__(kThreads, 1)
attn_scores_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                   const __grid_constant__ CUtensorMap tmO0, const __grid_constant__ CUtensorMap tmO1,
                   const __grid_constant__ CUtensorMap tmO2, const __grid_constant__ CUtensorMap tmI,
                   const __grid_constant__ CUtensorMap tmM, const Params p) {
  using C = Cfg<BWD>;
  constexpr int NB = C::kOutBufs;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t operands = (raw + 1023u) & ~1023u;
  const uint32_t staging = operands + kOperandBytes;
  const uint32_t inslots = staging + C::kStaging;
  const uint32_t red = inslots + kEpiWarps * C::kInSlot * C::kSlots;
  const uint32_t refs = red + kRedBytes;                    // forward only
  const uint32_t bars = refs + (BWD ? 0 : kRefBytes);  // full, empty, tmem_full, tmem_empty, tmem_full[2], tmem_empty[2], in_full[kEpiWarps], epilogue barrier, tmem slot
  const uint32_t bar_full = bars, bar_empty = bars + 8, bar_tfull = bars + 16, bar_tempty = bars + 32, bar_in = bars + 48;
  const uint32_t bar_epi = bar_in + 8 * kEpiWarps * C::kSlots;
  uint8_t* gen_base = smem_raw + (operands - raw);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + (bars - operands) + 64 + 8 * kEpiWarps * C::kSlots);
  float* red_gen = reinterpret_cast<float*>(gen_base + (red - operands));
  float* ref_gen = reinterpret_cast<float*>(gen_base + (refs - operands));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int L = p.L;
  const int nchunk = (L + 255) / 256;  // MMA column chunks of up to 256 keys
  const bool mask_in = BWD || !p.rng.philox;

  if (threadIdx.x == 0) {
    mbar_init(bar_full, 1);
    mbar_init(bar_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_tfull + 8 * i, 1);
      mbar_init(bar_tempty + 8 * i, kEpiWarps);
    }
    for (int w = 0; w < kEpiWarps * C::kSlots; ++w) mbar_init(bar_in + 8 * w, 1);
    mbar_init(bar_epi, kEpiWarps);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmA) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmB) : "memory");
    if (!p.skip_o0) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmO0) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmO1) : "memory");
    if (!BWD) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmO2) : "memory");
    if (BWD) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmI) : "memory");
    if (mask_in) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmM) : "memory");
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
    // ---------------- TMA producer: the operands of one tile at a time ----------------
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++it) {
      const int j0 = (int)(t % p.tiles_j) * 128;
      const int bt = (int)(t / p.tiles_j);
      ok = __all_sync(0xffffffffu, mbar_wait(bar_empty, (it & 1u) ^ 1u, 1));
      if (!ok) break;
      if (lane == 0) {
        mbar_expect_tx(bar_full, (uint32_t)(kABytes + p.b_bytes));
        const uint32_t sa = operands, sb_ = sa + kABytes;
        if (!p.a_mn) {
          if (p.a_swap) tma_load_3d(sa, &tmA, bar_full, 0, bt, j0);
          else tma_load_3d(sa, &tmA, bar_full, 0, j0, bt);
        } else {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (p.a_swap) tma_load_3d(sa + h * 8192, &tmA, bar_full, j0 + 64 * h, bt, 0);
            else tma_load_3d(sa + h * 8192, &tmA, bar_full, j0 + 64 * h, 0, bt);
          }
        }
        if (!p.b_mn) {
          for (int c = 0; c < nchunk; ++c) {  // boxes of 64 x min(256, L) key rows
            if (p.b_swap) tma_load_3d(sb_ + c * 32768, &tmB, bar_full, 0, bt, c * 256);
            else tma_load_3d(sb_ + c * 32768, &tmB, bar_full, 0, c * 256, bt);
          }
        } else {
          for (int h = 0; h < L / 64; ++h) {
            if (p.b_swap) tma_load_3d(sb_ + h * 8192, &tmB, bar_full, 64 * h, bt, 0);
            else tma_load_3d(sb_ + h * 8192, &tmB, bar_full, 64 * h, 0, bt);
          }
        }
      }
      __syncwarp();
      // The epilogue warps are still busy with the previous tile: bring this tile's row inputs (mask,
      // and ALPHA in the backward kernel) into L2 now, so that their slot fetches find them there.
      if (mask_in && p.prefetch) {
        const int nbox = (min(128, L - j0) / 32) * (L / 64);
        for (int b = lane; b < nbox; b += 32) {
          const int jr = j0 + (b / (L / 64)) * 32, c0 = (b % (L / 64)) * 64;
          if (p.swap_o) {
            if (BWD) tma_prefetch_3d(&tmI, c0, bt, jr);
            tma_prefetch_3d(&tmM, c0, bt, jr);
          } else {
            if (BWD) tma_prefetch_3d(&tmI, c0, jr, bt);
            tma_prefetch_3d(&tmM, c0, jr, bt);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    const uint32_t a_lbo = p.a_mn ? 8192u : 16u, b_lbo = p.b_mn ? 8192u : 16u;
    const uint32_t a_step = p.a_mn ? 2048u : 32u, b_step = p.b_mn ? 2048u : 32u;
    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < p.tiles && ok; t += gridDim.x, ++it) {
      // tensor memory holds one tile, in two halves of 256 columns that are filled (and, by the last
      // epilogue pass of the previous tile, released) separately: the MMAs of the first half run
      // while the previous tile's second half is still being read
      for (int c = 0; c < nchunk && ok; ++c) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_tempty + 8 * c, (it & 1u) ^ 1u, 4));
        if (!ok) break;
        if (c == 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar_full, it & 1u, 2));
          if (!ok) break;
        }
        tc_fence_after();
        if (lane == 0) {
          const uint32_t sa = operands, sb_ = sa + kABytes;
          const int width = min(256, L - c * 256);
          const uint32_t idesc = (1u << 4) | SB_IDESC_AB_FMT | ((uint32_t)(p.a_mn ? 1 : 0) << 15) | ((uint32_t)(p.b_mn ? 1 : 0) << 16) |
                                 ((uint32_t)(width >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t da = make_desc(sa + k * a_step, a_lbo, 1024u);
            const uint64_t db = make_desc(sb_ + c * 32768 + k * b_step, b_lbo, 1024u);
            umma_f16(tmem_base + c * 256, da, db, idesc, k > 0 ? 1u : 0u);
          }
          umma_commit(bar_tfull + 8 * c);
          if (c == nchunk - 1) umma_commit(bar_empty);   // the operand buffer may be refilled for the next tile
        }
        __syncwarp();
      }
    }
  } else {
    // ---------------- softmax / epilogue warps: thread = one query row ----------------
    const int ew = warp - 2;
    const int q = warp & 3;               // tensor-memory quadrant this warp may access
    const int h = ew >> 2;                // which of the quadrant's warps: chunks h, h + kNW, ...
    const int rt = q * 32 + lane;         // row within the tile
    const int nc64 = L / 64;
    const uint32_t my_stage = staging + (uint32_t)ew * NB * 4096;
    uint8_t* my_stage_gen = gen_base + (my_stage - operands);
    constexpr int NSL = C::kSlots;
    const uint32_t my_in = inslots + (uint32_t)ew * C::kInSlot * NSL;      // this warp's NSL slots, back to back
    const uint8_t* my_in_gen0 = gen_base + (my_in - operands);
    const uint32_t my_bar0 = bar_in + 8 * ew * NSL;
    const float c2 = p.scale * 1.4426950408889634f;
    const uint32_t trow = tmem_base + ((uint32_t)(q * 32) << 16);
    const int G = gridDim.x;

    auto tile_has_rows = [&](int t) { return (t % p.tiles_j) * 128 + q * 32 < L; };
    // fetch the row inputs of chunk c of tile t into this warp's slot (lane 0)
    auto fetch_in = [&](int t, int c, uint32_t slot) {
      const int jr = (t % p.tiles_j) * 128 + q * 32;
      const int bt = t / p.tiles_j;
      const uint32_t bar = my_bar0 + 8 * slot, dst = my_in + slot * (uint32_t)C::kInSlot;
      mbar_expect_tx(bar, (uint32_t)C::kInSlot);
      if (BWD) {
        if (p.swap_o) tma_load_3d(dst, &tmI, bar, c * 64, bt, jr);
        else tma_load_3d(dst, &tmI, bar, c * 64, jr, bt);
      }
      const uint32_t md = dst + (BWD ? 4096u : 0u);
      if (p.swap_o) tma_load_3d(md, &tmM, bar, c * 64, bt, jr);
      else tma_load_3d(md, &tmM, bar, c * 64, jr, bt);
    };
    // successor of (t, c) in this warp's sequence of input chunks
    auto next_in = [&](int& t, int& c) {
      c += kNW;
      if (c < nc64) return true;
      c = h;
      for (t += G; t < p.tiles; t += G)
        if (tile_has_rows(t)) return true;
      return false;
    };
    uint32_t n_in = 0;    // input chunks consumed (slot = n_in % NSL, phase = (n_in / NSL) & 1)
    uint32_t n_out = 0;   // staging buffers filled (buffer = n_out % NB)
    uint32_t n_bar = 0;   // uses of the epilogue barrier
    // lane 0 keeps the cursor of the next chunk to fetch: NSL chunks are requested up front, and every chunk taken
    // out of its slot lets the one NSL positions further in
    int ft = blockIdx.x, fc = h;
    bool fmore = false;
    uint32_t n_f = 0;
    if (mask_in && h < nc64 && lane == 0) {
      while (ft < p.tiles && !tile_has_rows(ft)) ft += G;
      fmore = ft < p.tiles;
      for (int i = 0; i < NSL && fmore; ++i) {
        fetch_in(ft, fc, n_f % NSL);
        ++n_f;
        fmore = next_in(ft, fc);
      }
    }
    auto refill = [&]() {                  // lane 0, after the slot just read is free again
      if (fmore) {
        fetch_in(ft, fc, n_f % NSL);
        ++n_f;
        fmore = next_in(ft, fc);
      }
    };

    // staging: 16-byte piece i (0..7) of this thread's row in buffer b
    auto stage_ptr = [&](uint32_t b, int i) {
      return reinterpret_cast<uint4*>(my_stage_gen + b * 4096 + lane * 128 + ((i ^ (lane & 7)) << 4));
    };
    auto store_rows = [&](const CUtensorMap* map, uint32_t b, int c, int jr, int bt) {
      if (p.swap_o) tma_store_3d(map, my_stage + b * 4096, c * 64, bt, jr);
      else tma_store_3d(map, my_stage + b * 4096, c * 64, jr, bt);
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    };

    uint32_t it = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < p.tiles && ok; t += G, ++it) {
      const int j0 = (t % p.tiles_j) * 128;
      const int bt = t / p.tiles_j;
      const int jr = j0 + q * 32;                          // first row of this warp
      const bool rows = jr < L && h < nc64;                // warp-uniform: this warp has work in the tile
      const long long row_off = ((long long)bt * L + (jr + lane)) * (long long)L;
      // first reads of a half wait for its MMAs; the last pass hands the halves back one by one
      auto wait_half = [&](int hf) {
        ok = __all_sync(0xffffffffu, mbar_wait(bar_tfull + 8 * hf, it & 1u, 3)) && ok;
        tc_fence_after();
      };
      auto release_half = [&](int hf) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_tempty + 8 * hf);
      };
      auto no_op = [](int) {};

      if (!BWD) {
        // pass 1 (online softmax): e = 2^(t - m) back into tensor memory, where m is the row maximum SO FAR (over
        // the pieces this warp has seen); when a piece raises m, the running sum is rescaled.  The m each 32-column
        // piece was scaled by is kept (shared memory, one float per thread and piece) so that the last pass can
        // bring every piece to the final maximum.  BETA out unless it is not wanted.  (scale > 0.)
        float mrun = -INFINITY, sum = 0.f;
        float* my_ref = ref_gen + (ew * 32 + lane);
        if (rows)
          sweep_halves(trow, h, nc64, wait_half, no_op, [&](int c, int hh, uint32_t* r) {
            const uint32_t b = n_out % NB;
            if (hh == 0 && !p.skip_o0) {
              if (lane == 0) bulk_wait_read<NB - 1>();
              __syncwarp();
            }
            float mx = mrun;
#pragma unroll
            for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(r[e]));
            if (mx > mrun) {
              sum *= ex2_approx((mrun - mx) * c2);      // 0 for the first piece (mrun = -inf, sum = 0)
              mrun = mx;
            }
            my_ref[((c / kNW) * 2 + hh) * (kEpiWarps * 32)] = mrun;
            const float mxs = mrun * c2;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float a = __uint_as_float(r[v * 8 + e]);
                f[e] = a * p.scale;
                const float ex = ex2_approx(fmaf(a, c2, -mxs));
                sum += ex;
                r[v * 8 + e] = __float_as_uint(ex);
              }
              if (!p.skip_o0) *stage_ptr(b, hh * 4 + v) = pack8(f);
            }
            tmem_st32(trow + c * 64 + hh * 32, r);
            if (hh == 1 && !p.skip_o0) {
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0) store_rows(&tmO0, b, c, jr, bt);
              ++n_out;
            }
          });
        tmem_st_wait();
        // the warps of a quadrant combine their (maximum, sum) pairs; alternate tiles use alternate slots, so a
        // warp already in the next tile never overwrites what a slower one still reads
        float* rset = red_gen + (it & 1u) * (2 * kNW * 128);
        rset[h * 128 + rt] = mrun;
        rset[(kNW + h) * 128 + rt] = sum;
        ok = epi_barrier(bar_epi, n_bar, lane) && ok;
        float mfin = -INFINITY;
#pragma unroll
        for (int w = 0; w < kNW; ++w) mfin = fmaxf(mfin, rset[w * 128 + rt]);
        sum = 0.f;
#pragma unroll
        for (int w = 0; w < kNW; ++w) {
          const float mw_ = rset[w * 128 + rt];
          if (mw_ > -INFINITY) sum = fmaf(rset[(kNW + w) * 128 + rt], ex2_approx((mw_ - mfin) * c2), sum);
        }
        const float inv = 1.f / sum;
        // pass 2: ALPHA = e * 2^(m_piece - m_final) / sum, ATTN_DROP = mask * ALPHA
        uint32_t mall[16];  // the mask bytes of this thread's row for one 64-column chunk
        if (rows)
          sweep_halves(trow, h, nc64, no_op, release_half, [&](int c, int hh, uint32_t* r) {
            // mask bytes of this thread's 32 columns, as 8 words
            uint32_t mw[8];
            if (!p.rng.philox) {
              if (hh == 0) {
                // take the whole chunk out of the slot at once, so that the next fetch starts early
                const uint32_t slot = n_in % NSL;
                const uint8_t* my_in_gen = my_in_gen0 + slot * C::kInSlot;
                ok = ok && __all_sync(0xffffffffu, mbar_wait(my_bar0 + 8 * slot, (n_in / NSL) & 1u, 5));
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  uint4 m = make_uint4(0, 0, 0, 0);
                  if (ok) m = *reinterpret_cast<const uint4*>(my_in_gen + lane * 64 + ((i ^ ((lane >> 1) & 3)) << 4));
                  mall[4 * i] = m.x; mall[4 * i + 1] = m.y; mall[4 * i + 2] = m.z; mall[4 * i + 3] = m.w;
                }
                ++n_in;
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0 && ok) refill();
              }
#pragma unroll
              for (int i = 0; i < 8; ++i) mw[i] = mall[hh * 8 + i];
            } else {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint32_t mm[8];
                philox_keep8(p.rng, (unsigned long long)(row_off + c * 64 + hh * 32 + v * 8) >> 3, mm);
                const uint2 pk = mask_pack(mm);
                mw[2 * v] = pk.x;
                mw[2 * v + 1] = pk.y;
              }
              uint4* mp = reinterpret_cast<uint4*>(p.mask + row_off + c * 64 + hh * 32);
              mp[0] = make_uint4(mw[0], mw[1], mw[2], mw[3]);
              mp[1] = make_uint4(mw[4], mw[5], mw[6], mw[7]);
            }
            const uint32_t b0 = n_out % NB, b1 = (n_out + 1) % NB;
            if (hh == 0) {
              if (lane == 0) bulk_wait_read<NB - 2>();
              __syncwarp();
            }
            // bring this piece from the maximum it was scaled by to the row's final one, and normalise
            const float fac = ex2_approx((my_ref[((c / kNW) * 2 + hh) * (kEpiWarps * 32)] - mfin) * c2) * inv;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]) * fac;
              const uint4 al = pack8(f);
              *stage_ptr(b0, hh * 4 + v) = al;
              *stage_ptr(b1, hh * 4 + v) = mask_apply(al, make_uint2(mw[2 * v], mw[2 * v + 1]));
            }
            if (hh == 1) {
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0) {
                store_rows(&tmO1, b0, c, jr, bt);
                store_rows(&tmO2, b1, c, jr, bt);
              }
              n_out += 2;
            }
          });
      } else {
        // backward pass 1: DATTN_DROP out; (da, alpha) with da = mask * DATTN_DROP kept as an fp16
        // pair per tensor-memory word; partial s = sum da * alpha
        float ssum = 0.f;
        uint4 aall[8];      // ALPHA of this thread's row for one 64-column chunk
        uint32_t mall[16];  // and its mask bytes
        if (rows)
          sweep_halves(trow, h, nc64, wait_half, no_op, [&](int c, int hh, uint32_t* r) {
            if (hh == 0) {
              // take the whole chunk (ALPHA and mask rows) out of the slot, then refill it at once
              const uint32_t slot = n_in % NSL;
              const uint8_t* my_in_gen = my_in_gen0 + slot * C::kInSlot;
              ok = ok && __all_sync(0xffffffffu, mbar_wait(my_bar0 + 8 * slot, (n_in / NSL) & 1u, 5));
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                aall[i] = make_uint4(0, 0, 0, 0);
                if (ok) aall[i] = *reinterpret_cast<const uint4*>(my_in_gen + lane * 128 + ((i ^ (lane & 7)) << 4));
              }
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                uint4 m = make_uint4(0, 0, 0, 0);
                if (ok) m = *reinterpret_cast<const uint4*>(my_in_gen + 4096 + lane * 64 + ((i ^ ((lane >> 1) & 3)) << 4));
                mall[4 * i] = m.x; mall[4 * i + 1] = m.y; mall[4 * i + 2] = m.z; mall[4 * i + 3] = m.w;
              }
              ++n_in;
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0 && ok) refill();
            }
            uint4 araw[4];
            uint32_t mw[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) araw[i] = aall[hh * 4 + i];
#pragma unroll
            for (int i = 0; i < 8; ++i) mw[i] = mall[hh * 8 + i];
            const uint32_t b = n_out % NB;
            if (hh == 0 && !p.skip_o0) {
              if (lane == 0) bulk_wait_read<NB - 1>();
              __syncwarp();
            }
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8], a8[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(r[v * 8 + e]);
              const uint4 dad = pack8(f);   // DATTN_DROP as stored (fp16)
              if (!p.skip_o0) *stage_ptr(b, hh * 4 + v) = dad;
              // continue from the fp16 value, as the separate softmax-backward operator would
              const uint4 da = mask_apply(dad, make_uint2(mw[2 * v], mw[2 * v + 1]));
              unpack8(da, f);
              unpack8(araw[v], a8);
#pragma unroll
              for (int e = 0; e < 8; ++e) ssum = fmaf(f[e], a8[e], ssum);
              const uint32_t dw[4] = {da.x, da.y, da.z, da.w}, aw[4] = {araw[v].x, araw[v].y, araw[v].z, araw[v].w};
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                r[v * 8 + 2 * k] = __byte_perm(dw[k], aw[k], 0x5410);      // (da, alpha) of the even element
                r[v * 8 + 2 * k + 1] = __byte_perm(dw[k], aw[k], 0x7632);  // ... of the odd element
              }
            }
            tmem_st32(trow + c * 64 + hh * 32, r);
            if (hh == 1 && !p.skip_o0) {
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0) store_rows(&tmO0, b, c, jr, bt);
              ++n_out;
            }
          });
        tmem_st_wait();
        float* rset = red_gen + (it & 1u) * (2 * kNW * 128);   // alternate tiles, alternate slots (see forward)
        rset[h * 128 + rt] = ssum;
        ok = epi_barrier(bar_epi, n_bar, lane) && ok;
        ssum = 0.f;
#pragma unroll
        for (int w = 0; w < kNW; ++w) ssum += rset[w * 128 + rt];
        // backward pass 2: DBETA = alpha * (da - s)
        if (rows)
          sweep_halves(trow, h, nc64, no_op, release_half, [&](int c, int hh, uint32_t* r) {
            const uint32_t b = n_out % NB;
            if (hh == 0) {
              if (lane == 0) bulk_wait_read<NB - 1>();
              __syncwarp();
            }
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              float f[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float2 da_al = sb_h22f2(*reinterpret_cast<const sb_half2*>(&r[v * 8 + e]));
                f[e] = da_al.y * (da_al.x - ssum);
              }
              *stage_ptr(b, hh * 4 + v) = pack8(f);
            }
            if (hh == 1) {
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              __syncwarp();
              if (lane == 0) store_rows(&tmO1, b, c, jr, bt);
              ++n_out;
            }
          });
      }
      // a warp without rows in this tile reads nothing: it hands both halves back here
      if (!rows)
        for (int hf = 0; hf * 4 < nc64; ++hf) release_half(hf);
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    __syncwarp();
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

}  // namespace attn
