/*
 * substation_b200 -- C ABI of the B200 encoder-layer library.
 *
 * This is the boundary a host binds (ctypes, cgo, JNI ...): plain C types, raw
 * device pointers, an opaque CUDA stream handle.  It replaces the four symbols
 * the reference exports from pytorch_module/encoder.cu:304-318 (init,
 * encoder_forward, encoder_backward, destroy) and adds one entry point per
 * fused operator and one for the tensor contractions, which is what the
 * reference's per-kernel harness (pytorch_module/benchmark.py) generates a
 * translation unit for.
 *
 * Differences from the reference ABI, all deliberate:
 *   - every function returns an sb_status instead of aborting the process
 *     (reference: CHECK -> abort, pytorch_module/all.cuh:7-13);
 *   - sizes, dropout probabilities and per-tensor dim orders are run-time
 *     arguments of sb_create, not macros in a generated header
 *     (reference: pytorch_module/encoder.py:213-376);
 *   - work is enqueued on the caller's stream, not on a private one
 *     (reference: pytorch_module/encoder.cu:78);
 *   - dropout masks are uint8 tensors that the caller either supplies
 *     (SB_MASK_EXPLICIT) or the kernels fill (SB_MASK_PHILOX).
 *
 * All tensors are fp16 except dropout masks (uint8, values 0/1).
 * Strides are in elements.  No function synchronises the stream.
 */
#ifndef SUBSTATION_B200_H
#define SUBSTATION_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SB_MAX_DIMS 5
#define SB_NUM_PARAMS 12
#define SB_NUM_FWD_INTERM 23
#define SB_NUM_BWD_INTERM 14

typedef enum sb_status {
  SB_OK = 0,
  SB_ERR_ARG = 1,         /* null pointer, bad enum, non-positive size */
  SB_ERR_LAYOUT = 2,      /* a dim-order string is not a permutation of the tensor's dims */
  SB_ERR_UNSUPPORTED = 3, /* valid request outside what the kernels cover (message says what) */
  SB_ERR_CUDA = 4,        /* a CUDA runtime/driver call failed (message carries its text) */
  SB_ERR_ALIGNMENT = 5,   /* pointer or stride not aligned as the selected kernel needs */
  SB_ERR_DEVICE = 6       /* a kernel reported a bounded wait running out */
} sb_status;

typedef enum sb_activation { SB_ACT_RELU = 0, SB_ACT_GELU = 1 } sb_activation;
typedef enum sb_mask_mode { SB_MASK_EXPLICIT = 0, SB_MASK_PHILOX = 1 } sb_mask_mode;
/* which contraction kernel sb_einsum uses */
typedef enum sb_gemm_impl {
  SB_GEMM_AUTO = 0,    /* tcgen05 when the operands qualify, else SIMT */
  SB_GEMM_TCGEN05 = 1, /* fail with SB_ERR_UNSUPPORTED when they do not */
  SB_GEMM_SIMT = 2
} sb_gemm_impl;

/* A strided view.  size/stride are listed in the operator's LOGICAL dim order
 * (given per function below); any permutation of memory order is expressed
 * through the strides. */
typedef struct sb_tensor {
  void* ptr;
  int32_t ndim;
  int64_t size[SB_MAX_DIMS];
  int64_t stride[SB_MAX_DIMS];
} sb_tensor;

/* Dropout source for the forward operators.  In SB_MASK_PHILOX mode the mask of
 * the element with logical linear index e is derived from Philox4x32-10 with
 * key = seed, counter = (e >> 3, offset); it does not depend on memory layout
 * or launch geometry.  Replaces GlobalRandomState (pytorch_module/blocks.cuh:48-51). */
typedef struct sb_dropout {
  float p;         /* drop probability in [0,1) */
  int32_t mode;    /* sb_mask_mode */
  uint64_t seed;
  uint64_t offset; /* distinguishes dropout sites / calls */
} sb_dropout;

const char* sb_status_string(int status);
/* Message of the most recent failure on the calling thread ("" if none). */
const char* sb_last_error(void);
/* Library version and the SM architecture it was built for, e.g. "0.1 sm_100a". */
const char* sb_version(void);

/* Scratch used by the operators that reduce over tokens (they write fp32
 * partial sums there).  The caller allocates sb_workspace_bytes() of device
 * memory, zero-fills it ONCE, and may reuse it for any sequence of calls on one
 * stream; two calls that run concurrently need two workspaces. */
size_t sb_workspace_bytes(void);

/* ------------------------------------------------------------------------- */
/* Fused operators.  "stream" is a cudaStream_t passed as void*.             */
/* ------------------------------------------------------------------------- */

/* out[n,p,h,b,j] = in[n,p,h,b,j] + bias[n,p,h]; n counts stacked projections.
 * Replaces AttentionInputBiases::run, pytorch_module/block_aib.cuh:64-155.
 * in/out: [N,P,H,B,J]; bias: [N,P,H]. */
int sb_attention_input_biases(void* stream, const sb_tensor* in, const sb_tensor* bias,
                              const sb_tensor* out);

/* alpha = softmax_k(scale*beta); drop = mask*alpha.  All [H,B,J,K].
 * Replaces Softmax::run, pytorch_module/block_softmax.cuh:127-188. */
int sb_softmax_dropout(void* stream, const sb_tensor* beta, const sb_tensor* alpha,
                       const sb_tensor* mask, const sb_tensor* drop, float scale,
                       const sb_dropout* dropout);

/* lin = in + bias; r = mask*lin + resid; LayerNorm over the last dim:
 * diff = r - mean, istd = rsqrt(var + 1e-5), ln = diff*istd, out = ln*gamma + beta.
 * in, resid, mask, lin, diff, ln, out: [B,J,I]; istd: [B,J]; bias/gamma/beta: [I].
 * lin may alias in (same strides), or be NULL when the caller does not need it (the layer's
 * backward pass never reads it): it is then not stored.  Replaces BiasDropoutResidualLinearNorm::run,
 * pytorch_module/block_bdrln.cuh:105-180 and :275-352. */
int sb_bias_dropout_residual_layernorm(void* stream, const sb_tensor* in, const sb_tensor* bias,
                                       const sb_tensor* resid, const sb_tensor* gamma,
                                       const sb_tensor* beta, const sb_tensor* mask,
                                       const sb_tensor* lin, const sb_tensor* diff,
                                       const sb_tensor* istd, const sb_tensor* ln,
                                       const sb_tensor* out, const sb_dropout* dropout);

/* lin1 = in + bias; drop2 = mask*act(lin1).  [B,J,U], bias [U].
 * Replaces BiasActivationDropout::run, pytorch_module/block_bad.cuh:83-145
 * (ReLU there; GELU is the tanh form of substation/transformer.py:11-14). */
int sb_bias_activation_dropout(void* stream, const sb_tensor* in, const sb_tensor* bias,
                               const sb_tensor* mask, const sb_tensor* lin1,
                               const sb_tensor* drop2, int activation,
                               const sb_dropout* dropout);

/* dln = dy*gamma; dgamma = sum_{b,j} dy*ln; dbeta = sum_{b,j} dy.
 * dy, ln, dln: [B,J,I]; gamma, dgamma, dbeta: [I].
 * Replaces BackwardScaleBias::run, pytorch_module/block_bsb_ebsb.cuh:171-216. */
int sb_backward_scale_bias(void* stream, void* workspace, const sb_tensor* dy,
                           const sb_tensor* ln, const sb_tensor* gamma, const sb_tensor* dln,
                           const sb_tensor* dgamma, const sb_tensor* dbeta);

/* LayerNorm backward-data from the stored diff and reciprocal std, then dropout:
 * dresid = g*s - sum(g)*s/n - diff*sum(g*diff)*s^3/n; dlin = mask*dresid.
 * dln, diff, mask, dresid, dlin: [B,J,I]; istd: [B,J].
 * Replaces BackwardLayerNormResidualDropout::run, pytorch_module/block_blnrd.cuh:71-129, :195-259. */
int sb_backward_layernorm_residual_dropout(void* stream, const sb_tensor* dln,
                                           const sb_tensor* istd, const sb_tensor* diff,
                                           const sb_tensor* mask, const sb_tensor* dresid,
                                           const sb_tensor* dlin);

/* dlin1 = act'(lin1)*(mask*ddrop2); dbias = sum_{b,j} dlin1.  [B,J,U], dbias [U].
 * Replaces BackwardDropoutReluLinearBias::run, pytorch_module/block_bdrlb.cuh:98-146. */
int sb_backward_dropout_activation_bias(void* stream, void* workspace, const sb_tensor* ddrop2,
                                        const sb_tensor* mask, const sb_tensor* lin1,
                                        const sb_tensor* dlin1, const sb_tensor* dbias,
                                        int activation);

/* dlinb2 = sum dlin2; g = dresid2 + dlin1_linw1; dln1 = g*gamma1;
 * dgamma1 = sum g*ln1; dbeta1 = sum g.  3-D tensors [B,J,I], vectors [I].
 * Replaces ExtendedBackwardScaleBias::run, pytorch_module/block_bsb_ebsb.cuh:368-420. */
int sb_extended_backward_scale_bias(void* stream, void* workspace, const sb_tensor* ln1,
                                    const sb_tensor* gamma1, const sb_tensor* dresid2,
                                    const sb_tensor* dlin1_linw1, const sb_tensor* dlin2,
                                    const sb_tensor* dln1, const sb_tensor* dgamma1,
                                    const sb_tensor* dbeta1, const sb_tensor* dlinb2);

/* sb_backward_scale_bias followed by sb_backward_layernorm_residual_dropout in one pass over
 * the data: 13 instead of 15 bytes per element and one launch less.  dln (dln1 in the extended
 * form below) is only an intermediate of the pair: pass NULL and it is not stored (11 bytes).
 * Needs feature-innermost views of at most 1024 features, otherwise SB_ERR_UNSUPPORTED and the
 * caller runs the two operators.  Replaces the pair pytorch_module/encoder.cu:160-175. */
int sb_backward_scale_bias_layernorm(void* stream, void* workspace, const sb_tensor* dy,
                                     const sb_tensor* ln, const sb_tensor* gamma, const sb_tensor* istd,
                                     const sb_tensor* diff, const sb_tensor* mask, const sb_tensor* dln,
                                     const sb_tensor* dresid, const sb_tensor* dlin,
                                     const sb_tensor* dgamma, const sb_tensor* dbeta);

/* sb_extended_backward_scale_bias + sb_backward_layernorm_residual_dropout +
 * sb_backward_attn_out_bias in one pass (17 instead of 21 bytes per element, two launches
 * less).  Same eligibility rule.  Replaces the triple pytorch_module/encoder.cu:202-232. */
int sb_extended_backward_scale_bias_layernorm(
    void* stream, void* workspace, const sb_tensor* ln1, const sb_tensor* gamma1, const sb_tensor* dresid2,
    const sb_tensor* dlin1_linw1, const sb_tensor* dlin2, const sb_tensor* istd, const sb_tensor* diff,
    const sb_tensor* mask, const sb_tensor* dln1, const sb_tensor* dresid1, const sb_tensor* datt,
    const sb_tensor* dgamma1, const sb_tensor* dbeta1, const sb_tensor* dlinb2, const sb_tensor* dbo);

/* dbo[i] = sum_{b,j} datt[b,j,i].
 * Replaces BackwardAttnOutBias::run, pytorch_module/block_baob.cuh:75-97. */
int sb_backward_attn_out_bias(void* stream, void* workspace, const sb_tensor* datt,
                              const sb_tensor* dbo);

/* The same sum as sb_backward_attn_out_bias for callers that cannot provide a
 * workspace or reach the CUDA allocator (a plugin handed only inputs and outputs,
 * a process whose device heap is sealed after start-up).  This entry point has
 * no counterpart in the reference.  It makes no allocation of any kind: the
 * fp32 partial sums live in a 1 MiB + 4 KiB device array built into the library
 * (every GPU that loads the library holds it until the process exits).
 * Limits and rules:
 *   - the feature extent (last dim of datt) may be at most 16384, larger ones are
 *     refused with SB_ERR_UNSUPPORTED, and so are more than 2^31-1 tokens (B*J);
 *   - the first call on each device looks up that device's copy of the array
 *     (the stream's device must be current); make that first call outside of any
 *     stream capture;
 *   - all calls on a device share the one array, so two calls that may overlap
 *     on the GPU (different streams) race; serialise them. */
int sb_backward_attn_out_bias_noalloc(void* stream, const sb_tensor* datt, const sb_tensor* dbo);

/* The score contraction and the softmax in one kernel: beta = scale * sum_p qq*kk,
 * alpha = softmax_k(beta), drop = mask*alpha.  qq, kk: [P,H,B,J] projections (any strides TMA
 * can address); beta, alpha, mask, drop: [H,B,J,K] and dense in that order.  The 128 x K score
 * tile lives in tensor memory between the tcgen05 MMAs and the per-row softmax, so beta is
 * written but never read back; pass beta = NULL and it is not written at all.  Needs P = 64,
 * J = K a multiple of 64 and at most 512; otherwise
 * SB_ERR_UNSUPPORTED and the caller runs sb_einsum + sb_softmax_dropout.
 * Replaces the pair pytorch_module/encoder.cu:115-121. */
int sb_attention_scores_softmax(void* stream, const sb_tensor* qq, const sb_tensor* kk,
                                const sb_tensor* beta, const sb_tensor* alpha, const sb_tensor* mask,
                                const sb_tensor* drop, float scale, const sb_dropout* dropout);

/* dattn_drop = sum_p dgamma*vv and sb_backward_softmax in one kernel (dattn_drop is written
 * but never read back; NULL: not written at all).  Same requirements.  Replaces pytorch_module/encoder.cu:250-252 + :258-261. */
int sb_attention_scores_softmax_backward(void* stream, const sb_tensor* dgamma, const sb_tensor* vv,
                                         const sb_tensor* alpha, const sb_tensor* mask,
                                         const sb_tensor* dattn_drop, const sb_tensor* dbeta);

/* Contractions of a score tensor with head-size-64 projections, reading the scores once:
 *   out_rows[p,h,b,j] = alpha * sum_k scores[h,b,j,k] * x[p,h,b,k]   (x and out_rows both NULL to skip)
 *   out_cols[p,h,b,k] = alpha * sum_j scores[h,b,j,k] * y[p,h,b,j]   (y and out_cols both NULL to skip)
 * One CTA per (head, sample) keeps x and y in shared memory and streams the scores through
 * tcgen05 MMAs for both results.  scores: [H,B,J,K] dense in that order; projections [P,H,B,J]
 * with any strides TMA can address.  Needs P = 64, J = K a multiple of 128 and at most 512;
 * otherwise SB_ERR_UNSUPPORTED and the caller runs sb_einsum.  Replaces the contractions
 * gamma (pytorch_module/encoder.cu:123-125), dX2gamma (:254-256) and the pair dX1QKT, dX2QKT
 * (:263-269), the pair as one launch. */
int sb_attention_score_contractions(void* stream, const sb_tensor* scores, const sb_tensor* x,
                                    const sb_tensor* out_rows, const sb_tensor* y, const sb_tensor* out_cols,
                                    float alpha);

/* dbeta = alpha*(da - sum_k da*alpha), da = mask*dattn_drop.  All [H,B,J,K].
 * Replaces BackwardSoftmax::run, pytorch_module/block_bs.cuh:100-156. */
int sb_backward_softmax(void* stream, const sb_tensor* alpha, const sb_tensor* mask,
                        const sb_tensor* dattn_drop, const sb_tensor* dbeta);

/* dbias[n,p,h] = sum_{b,j} d[n,p,h,b,j].
 * Replaces BackwardAttentionInputBiases::run, pytorch_module/block_baib.cuh:156-211. */
int sb_backward_attention_input_biases(void* stream, const sb_tensor* d, const sb_tensor* dbias);

/* dx = dxatt + dresid1.  [B,J,I].
 * Replaces BackwardEncoderInput::run, pytorch_module/block_bei.cuh:52-106. */
int sb_backward_encoder_input(void* stream, const sb_tensor* dxatt, const sb_tensor* dresid1,
                              const sb_tensor* dx);

/* C = alpha * einsum(A, B): a_dims/b_dims/c_dims name each operand's dims with
 * one letter per entry of its size/stride arrays (e.g. "phbk","phbj","hbjk").
 * Letters in all three are batch dims, letters in A and B only are summed.
 * Each of the four letter groups must collapse to one stride in every operand,
 * as in the reference (pytorch_module/einsumparser.h:29-37).
 * Replaces Einsum::run / Gemm::run, pytorch_module/gemm.cuh:52-147.
 * workspace (optional, may be NULL): device scratch for fp32 partial sums; with it a
 * contraction that has few output tiles and a long summed extent (the weight gradients)
 * is split along K over more SMs and reduced in a fixed order.  It need not be cleared. */
int sb_einsum(void* stream, const char* a_dims, const sb_tensor* a, const char* b_dims,
              const sb_tensor* b, const char* c_dims, const sb_tensor* c, float alpha,
              int impl, void* workspace, size_t workspace_bytes);
/* Which kernel the last sb_einsum on this thread ran: SB_GEMM_TCGEN05 or SB_GEMM_SIMT. */
int sb_einsum_last_impl(void);

/* Elementwise operators folded into the epilogue of a contraction: c is written as by sb_einsum, and the
 * operator that would read it next is applied to the rounded fp16 values on their way out, with the same
 * arithmetic as the separate kernel (results are bit-identical to sb_einsum followed by that operator):
 *   SB_EPI_BIAS              out2 = c + bias               (sb_attention_input_biases, pytorch_module/encoder.cu:105-113)
 *   SB_EPI_RESIDUAL          out2 = c + resid              (sb_backward_encoder_input, pytorch_module/encoder.cu:294-296)
 *   SB_EPI_BIAS_ACT_DROPOUT  out2 = c + bias, out3 = mask * act(out2)   (sb_bias_activation_dropout, :142-145)
 * resid, mask, out2, out3: dims, sizes and strides of c (mask in bytes).  bias: a dense vector over exactly the
 * indices c shares with only one of the operands, nested as in c.  With SB_MASK_PHILOX the mask is generated
 * and written; c must then be dense in the order logical_dims gives.  SB_ERR_UNSUPPORTED unless the
 * contraction runs on the paired-CTA tcgen05 kernel (single batch, M, N, K >= 256, unit-stride columns,
 * N a multiple of 64); the caller then runs the two calls separately. */
typedef enum sb_epilogue_kind { SB_EPI_BIAS = 1, SB_EPI_RESIDUAL = 2, SB_EPI_BIAS_ACT_DROPOUT = 3 } sb_epilogue_kind;
typedef struct sb_epilogue {
  int kind;
  const char* bias_dims;
  const sb_tensor* bias;
  const sb_tensor* resid;
  const sb_tensor* mask;
  const sb_tensor* out2;
  const sb_tensor* out3;
  int activation;
  const sb_dropout* dropout;
  const char* logical_dims;
  int discard_c; /* non-zero: c itself is not stored, only out2 / out3 (c still gives the geometry) */
} sb_epilogue;
int sb_einsum_fused(void* stream, const char* a_dims, const sb_tensor* a, const char* b_dims, const sb_tensor* b,
                    const char* c_dims, const sb_tensor* c, float alpha, const sb_epilogue* epilogue);
/* Every wait inside the tcgen05 kernels and the ring-fed LayerNorm kernels is bounded; when one runs
 * out the kernel records a code (tcgen05: 1 producer, 2 MMA issuer, 3 epilogue, ...; ring: 11-14),
 * drains and returns.
 * This reads that flag after synchronising `stream` (0 = no wait ran out since the
 * last reset).  The flag is per device (the device current when the call is made) and
 * sticky: while it is set, every later tcgen05 kernel on that device gives up its waits
 * at once, so its output is garbage.  sb_device_error_reset clears it (after
 * synchronising `stream`) once the caller has dealt with the failed pass.  The
 * reference has no counterpart: its CHECK macro aborts the process
 * (pytorch_module/all.cuh:7-13). */
int sb_device_error(void* stream, int* code);
int sb_device_error_reset(void* stream);
/* Measurement aid: one launch in which every cluster of two CTAs issues k_blocks * 4 tcgen05.mma instructions
 * (cta_group::2, 256 x 256 x 16, fp16 or bf16 operands, fp32 accumulation: the instruction of the contraction
 * kernels) on operands already resident in shared memory, with no loads and no epilogue.  *flops receives the
 * floating-point operations of the launch; the caller times it with events on `stream`.  The result is the
 * tensor-pipe rate these kernels could reach if nothing but the MMAs cost time.  Stands in for the reference's
 * tensor-core microbenchmark (tc_profiling/microbenchmark/tensorcores.cu:16-40). */
int sb_mma_peak_probe(void* stream, int k_blocks, int bf16, double* flops);
/* The contraction, attention and LayerNorm kernels are persistent: one CTA per SM (or a
 * fixed number per SM) walks the work.  When another kernel must run next to them (the NCCL
 * gradient allreduce of the data-parallel path), tell the library to size every such grid
 * for n_sms SMs only, so that no CTA waits behind the other kernel and then runs its share
 * as a second round (0 = use every SM, the default).  Process-wide.  No counterpart in the
 * reference, which has no multi-GPU path. */
int sb_set_sm_budget(int n_sms);

/* ------------------------------------------------------------------------- */
/* Whole layer                                                               */
/* ------------------------------------------------------------------------- */

typedef struct sb_encoder sb_encoder;

typedef struct sb_encoder_config {
  int32_t batch;      /* B */
  int32_t seq;        /* J = K */
  int32_t heads;      /* H */
  int32_t embed;      /* I; P = I/H, U = 4*I */
  int32_t activation; /* sb_activation */
  float p_softmax, p_resid1, p_activation, p_resid2;
  /* Dim order of every tensor, as in the reference's layout pickle
   * (config_selection/optimize.py:443-493): names[i] -> dims[i], for X, SB2, the 12
   * parameters, the 23 forward and the 14 backward intermediates. */
  int32_t n_tensors;
  const char* const* names;
  const char* const* dims;
} sb_encoder_config;

/* Replaces init() (pytorch_module/encoder.cu:304-306) and the code generation of
 * pytorch_module/encoder.py:165-405.  Allocates the handle's workspaces (token-reduction partials and
 * split-K partials: the only device allocations the library makes for a layer). */
int sb_encoder_create(const sb_encoder_config* cfg, sb_encoder** out);
/* Replaces destroy() (pytorch_module/encoder.cu:316-318). */
int sb_encoder_destroy(sb_encoder* enc);

/* Replaces encoder_forward (pytorch_module/encoder.cu:308-310).  params, fwd: arrays of
 * device pointers in the order of the config's parameter / forward-intermediate
 * lists (the same order the reference passes them, pytorch_module/encoder.py:88-93).
 * The four mask tensors inside fwd are read (explicit) or written (philox).
 * seed/offset: Philox key and base offset; the four dropout sites use offset+0..3. */
int sb_encoder_forward(sb_encoder* enc, void* stream, const void* x, const void* const* params,
                       void* const* fwd, void* y, int mask_mode, uint64_t seed,
                       uint64_t offset);
/* Replaces encoder_backward (pytorch_module/encoder.cu:312-314); argument groups in the
 * reference's order: dY, 12 parameter gradients, 14 backward intermediates, 12
 * parameters, 23 forward intermediates, X, dX (pytorch_module/encoder.py:124-130). */
int sb_encoder_backward(sb_encoder* enc, void* stream, const void* dy, void* const* dparams,
                        void* const* bwd, const void* const* params, void* const* fwd,
                        const void* x, void* dx);
/* Per-operator device time of the most recent forward+backward, measured with
 * CUDA events when timing was switched on; writes up to max (name, ms) pairs
 * and returns the count.  While timing is on every operator is also an NVTX range
 * of the same name on the calling thread (the ranges of pytorch_module/encoder.cu:32-53),
 * and passes are launched plainly rather than replayed as graphs. */
int sb_encoder_set_timing(sb_encoder* enc, int enabled);
int sb_encoder_get_timing(sb_encoder* enc, int max, const char** names, float* ms);
/* Number of operators the most recent forward / backward launched. */
/* A pass whose pointer arguments repeat (explicit masks, timing off) is captured once as a CUDA graph and
 * replayed with a single launch afterwards; 0 switches that off for the handle (default on; the environment
 * variable SUBSTATION_B200_GRAPHS=0 switches it off for the process). */
int sb_encoder_set_graphs(sb_encoder* enc, int enabled);
/* A CUDA event (cudaEvent_t, caller-owned; NULL to stop) that every backward pass records on its stream as soon
 * as the gradients of the feed-forward half and of both LayerNorms are final (LINW1, LINB1, LINW2, LINB2, S1,
 * B1, S2, B2, BO: in the parameter order these are everything from LINB1 on, plus S1, B1, BO), i.e. before
 * the attention half of the backward pass runs.  A data-parallel host waits for it on its communication
 * stream and starts the allreduce of that part of the gradient bucket while the pass continues. */
int sb_encoder_set_ffn_grads_event(sb_encoder* enc, void* event);
/* How many passes were captured as graphs and how many were replayed since the handle was created. */
int sb_encoder_graph_stats(sb_encoder* enc, long long* captures, long long* replays);
int sb_encoder_launch_count(sb_encoder* enc);
/* Kernels launched by the most recent forward plus the most recent backward (an operator may need
 * a second, finishing kernel, so this can exceed the two operator counts). */
int sb_encoder_kernel_count(sb_encoder* enc);
/* Fused multi-operator kernels (on by default) can be switched off to run the reference's
 * one-kernel-per-operator sequence. */
int sb_encoder_set_fusion(sb_encoder* enc, int enabled);
/* Nine tensors of the reference's pointer tables are written by the layer but read by nothing
 * afterwards once the fused operators run (pytorch_module/encoder.cu:158-299 lists what backward
 * reads): BETA, WKKWQQWVV, SB1_LINW1, LIN2 and the bias written back over ATT in the forward pass;
 * DATTN_DROP, DLN2, DLN1 and DXATT in the backward pass, 235 MB per step at B=8, L=512.  enabled = 1 (the
 * default) writes them all, as the reference does; 0 leaves them untouched wherever a fused
 * operator makes them unnecessary (their pointers must still be valid: an operator that declines
 * falls back to the separate kernels, which need them). */
int sb_encoder_set_dead_stores(sb_encoder* enc, int enabled);

#ifdef __cplusplus
}
#endif
#endif /* SUBSTATION_B200_H */
