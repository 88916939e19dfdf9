// Internal launch interface of the fused operators (views already validated).
#pragma once

#include "common.cuh"

namespace sb {

struct Dims3 { int B, J, F; };
struct Dims4 { int H, B, J, K; };
struct Dims5 { int N, P, H, B, J; };

// Workspace layout: [0, kWsCounterBytes) ticket counters (must start at zero; every
// kernel that uses them leaves them at zero), then fp32 partial sums.
constexpr size_t kWsCounterBytes = 4096;
constexpr size_t kWsBytes = 8u << 20;

int launch_aib(cudaStream_t s, Dims5 d, View5 in, const void* bias, long long bsN, long long bsP,
               long long bsH, View5 out);
int launch_softmax_fwd(cudaStream_t s, Dims4 d, View4 beta, View4 alpha, View4 mask, View4 drop,
                       float scale, Rng rng);
int launch_softmax_bwd(cudaStream_t s, Dims4 d, View4 alpha, View4 mask, View4 dattn_drop,
                       View4 dbeta);
int launch_bdrln(cudaStream_t s, Dims3 d, View3 in, const void* bias, View3 resid,
                 const void* gamma, const void* beta, View3 mask, View3 lin, View3 diff,
                 View2 istd, View3 ln, View3 out, Rng rng);
int launch_bad(cudaStream_t s, Dims3 d, View3 in, const void* bias, View3 mask, View3 lin1,
               View3 drop2, int activation, Rng rng);
int launch_blnrd(cudaStream_t s, Dims3 d, View3 dln, View2 istd, View3 diff, View3 mask,
                 View3 dresid, View3 dlin);
int launch_bei(cudaStream_t s, Dims3 d, View3 a, View3 b, View3 out);
int launch_baib(cudaStream_t s, Dims5 d, View5 in, void* dbias, long long bsN, long long bsP,
                long long bsH);
int launch_bsb(cudaStream_t s, void* ws, Dims3 d, View3 dy, View3 ln, const void* gamma,
               View3 dln, void* dgamma, void* dbeta);
int launch_ebsb(cudaStream_t s, void* ws, Dims3 d, View3 ln1, const void* gamma1, View3 dresid2,
                View3 dlin1_linw1, View3 dlin2, View3 dln1, void* dgamma1, void* dbeta1,
                void* dlinb2);
int launch_bdrlb(cudaStream_t s, void* ws, Dims3 d, View3 ddrop2, View3 mask, View3 lin1,
                 View3 dlin1, void* dbias, int activation);
int launch_baob(cudaStream_t s, void* ws, Dims3 d, View3 datt, void* dbo);

// Fused LayerNorm backward (scale/bias gradients + backward-data + dropout [+ bias gradients]);
// SB_ERR_UNSUPPORTED when a view is not feature-innermost or has more than 1024 features.
int launch_lnbwd_a(cudaStream_t s, void* ws, Dims3 d, View3 dy, View3 ln, const void* gamma, View2 istd, View3 diff,
                   View3 mask, View3 dln, View3 dresid, View3 dlin, void* dgamma, void* dbeta);
int launch_lnbwd_b(cudaStream_t s, void* ws, Dims3 d, View3 ln1, const void* gamma1, View3 dresid2, View3 dlw,
                   View3 dlin2, View2 istd, View3 diff, View3 mask, View3 dln1, View3 dresid1, View3 datt,
                   void* dgamma1, void* dbeta1, void* dlinb2, void* dbo);

// bias + dropout + residual + LayerNorm with the input rows staged through a shared-memory ring (bulk copies);
// SB_ERR_UNSUPPORTED, nothing launched, unless every view is feature-innermost with 16-byte-multiple rows.
int launch_bdrln_ring(cudaStream_t s, Dims3 d, View3 in, const void* bias, View3 resid, const void* gamma,
                      const void* beta, View3 mask, View3 lin, View3 diff, View2 istd, View3 ln, View3 out, Rng rng);
// Error flag of the ring kernels (a bounded wait ran out: codes 11-14), per device.
int ring_device_error(cudaStream_t s, int* code);
int ring_device_error_reset(cudaStream_t s);

// Fused attention scores.  qq/kk/dgamma/vv are [P,H,B,rows] projections passed as View4 whose
// (sH,sB,sJ,sK) fields hold the (P,H,B,row) strides; d = {H,B,J,K}.  SB_ERR_UNSUPPORTED when
// the shapes or layouts do not qualify.
int launch_attn_scores_fwd(cudaStream_t s, Dims4 d, int P, View4 qq, View4 kk, View4 beta, View4 alpha, View4 mask,
                           View4 drop, float scale, Rng rng);
int launch_attn_scores_bwd(cudaStream_t s, Dims4 d, int P, View4 dgamma, View4 vv, View4 alpha, View4 mask,
                           View4 dattn_drop, View4 dbeta);

// Score-tensor contractions with head-size-64 projections, S read once:
//   out_r[p,h,b,j] = alpha * sum_k scores[h,b,j,k] * x[p,h,b,k]   (x, out_r both null to skip)
//   out_c[p,h,b,k] = alpha * sum_j scores[h,b,j,k] * y[p,h,b,j]   (y, out_c both null to skip)
// Projections use the same View4 convention as above.  SB_ERR_UNSUPPORTED when not eligible.
int launch_score_contract(cudaStream_t s, Dims4 d, int P, View4 scores, const View4* x, const View4* out_r, const View4* y,
                          const View4* out_c, float alpha);

// Contractions -----------------------------------------------------------------
struct GemmProblem {
  long long batch, M, N, K;
  long long sAb, sAm, sAk;
  long long sBb, sBn, sBk;
  long long sCb, sCm, sCn;
  const void* A;
  const void* B;
  void* C;
  float alpha;
};
// Elementwise work fused behind the epilogue of a contraction (see EpiParams in gemm.cu).  out2 / out3 / resid /
// mask have C's shape and strides (mask: in bytes); vec is a dense vector over C's rows (vec_along_m) or columns.
struct GemmEpilogue {
  int kind;            // 1 bias -> out2; 2 residual -> out2; 3 bias + activation + dropout -> out2, out3
  int vec_along_m;
  const void* vec;
  const void* resid;
  void* mask;
  int activation;
  Rng rng;
  void* out2;
  void* out3;
  int skip_c;          // do not store C itself (only the fused outputs are wanted)
};
// The contraction with fused epilogue work; SB_ERR_UNSUPPORTED unless the problem runs on the paired-CTA
// kernel with TMA stores (large, single batch, unit-stride columns, N a multiple of 64).
int run_gemm_fused(cudaStream_t s, const GemmProblem& g, const GemmEpilogue& epi);

// Collapse an einsum over strided operands into one batched GEMM (error if it is not one).
int plan_einsum(const char* a_dims, const sb_tensor* a, const char* b_dims, const sb_tensor* b,
                const char* c_dims, const sb_tensor* c, float alpha, GemmProblem* out);
bool tcgen05_supported(const GemmProblem& g, std::string* why);
int launch_gemm_tcgen05(cudaStream_t s, const GemmProblem& g, void* ws, size_t ws_bytes);
int launch_gemm_simt(cudaStream_t s, const GemmProblem& g);
// ws (optional): scratch for fp32 split-K partials; without it few-tile problems are not split.
int run_gemm(cudaStream_t s, const GemmProblem& g, int impl, void* ws = nullptr, size_t ws_bytes = 0);
extern thread_local int g_last_gemm_impl;
// Number of SMs the persistent contraction kernels may occupy (0 = all).
void set_gemm_sm_budget(int n);
int gemm_sm_budget();
// SMs a persistent grid may count on: all of them, or the budget set through sb_set_sm_budget when a concurrent
// kernel (a collective) holds the rest.  A grid sized for SMs it cannot get runs its last CTAs as a second round.
inline int usable_sms(int sms) {
  const int b = gemm_sm_budget();
  return (b > 0 && b < sms) ? b : sms;
}
// Non-zero once a tcgen05 kernel on the current device reported a bounded wait running out (until reset).
int gemm_device_error(cudaStream_t s, int* code);
int gemm_device_error_reset(cudaStream_t s);
// MMA-only loop of the paired-CTA instruction on operands resident in shared memory (see peak_probe.cuh).
int run_mma_peak_probe(cudaStream_t s, int k_blocks, int bf16, double* flops);

}  // namespace sb
