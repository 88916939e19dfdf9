// Tensor-pipe peak probe (included by gemm.cu; shares its tcgen05 helpers).
//
// What the paired-CTA contraction kernel could reach if nothing but the MMAs cost time: every cluster of two
// CTAs fills two shared-memory stages with fp16 (or bf16) values once, then its leader thread issues
// tcgen05.mma.cta_group::2 (256 x 256 x 16 per instruction, the instruction the contraction kernel uses) back to
// back on those resident operands, alternating between the two accumulators in tensor memory.  No loads, no
// epilogue.  The host times the launch with CUDA events; FLOPs = clusters * k_blocks * 4 * 2 * 256 * 256 * 16.
// Plays the role of the reference's tensor-core microbenchmark (tc_profiling/microbenchmark/tensorcores.cu:16-40).

#pragma once

namespace probe {

constexpr int kThreads = 128;
constexpr int kStages = 2;
constexpr int kSmemBytes = kStages * pair::kStageBytes + 1024 + 64;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
mma_peak_kernel(int k_blocks, int bf16) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t tiles = (raw + 1023u) & ~1023u;
  const uint32_t bars = tiles + kStages * pair::kStageBytes;   // two batch barriers, then the tensor-memory slot
  uint8_t* gen_base = smem_raw + (tiles - raw);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(gen_base + kStages * pair::kStageBytes + 32);
  const int warp = threadIdx.x >> 5;
  const uint32_t rank = pair::cluster_rank();

  // operands: values in [-1, 1) from a hash of the position (real bit patterns, so the multipliers toggle)
  for (int i = threadIdx.x; i < kStages * pair::kStageBytes / 2; i += kThreads) {
    uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u;
    h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
    const float v = (float)(int)(h & 0xffffu) * (1.f / 32768.f) - 1.f;
    if (bf16) reinterpret_cast<__nv_bfloat16*>(gen_base)[i] = __float2bfloat16_rn(v);
    else reinterpret_cast<__half*>(gen_base)[i] = __float2half_rn(v);
  }
  if (threadIdx.x == 0) {
    mbar_init(bars, 1);
    mbar_init(bars + 8, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 ::"r"(smem_u32(tmem_slot)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  pair::cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

  if (rank == 0 && threadIdx.x == 0) {
    const uint32_t fmt = bf16 ? ((1u << 7) | (1u << 10)) : 0u;   // A and B element type
    const uint32_t idesc = (1u << 4) | fmt | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
    const uint64_t da_base = make_desc(tiles, 16u, 1024u), db_base = make_desc(tiles + kABytes, 16u, 1024u);
    const uint64_t stage_inc = (uint64_t)pair::kStageBytes >> 4;
    // batches of 16 K blocks (64 instructions): batch b commits to barrier b & 1 and the thread waits for batch
    // b - 1 before it issues batch b + 1, so the queue never drains and never grows without bound
    constexpr int kBatch = 16;
    const int batches = (k_blocks + kBatch - 1) / kBatch;
    bool ok = true;
    for (int b = 0; b < batches && ok; ++b) {
      const int n = min(kBatch, k_blocks - b * kBatch);
      for (int kb = 0; kb < n; ++kb) {
        const uint64_t da = da_base + (uint64_t)(kb & 1) * stage_inc, db = db_base + (uint64_t)(kb & 1) * stage_inc;
        const uint32_t tmem_d = tmem_base + (uint32_t)(b & 1) * 256u;
#pragma unroll
        for (int k = 0; k < 4; ++k) pair::umma_f16_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, (b > 1 || kb > 0 || k > 0) ? 1u : 0u);
      }
      pair::umma_commit_pair(bars + 8 * (b & 1));
      if (b > 0) ok = mbar_wait(bars + 8 * ((b - 1) & 1), ((b - 1) >> 1) & 1u, 7);
    }
    // a wait that ran out has recorded code 7 where sb_device_error finds it
    if (ok && batches > 0) mbar_wait(bars + 8 * ((batches - 1) & 1), ((batches - 1) >> 1) & 1u, 7);
  }
  __syncthreads();
  tc_fence_before();
  pair::cluster_sync_all();   // the leader has seen every MMA complete before either CTA lets go of its memory
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace probe
