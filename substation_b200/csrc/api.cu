// C ABI: argument validation, strided-view construction, per-operator entry
// points and the whole-layer handle (operator sequence of the encoder layer).

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "ops.h"

namespace sb {
thread_local long long g_kernel_launches = 0;

namespace {
thread_local std::string g_error;
}

bool pdl_enabled() {
  static const bool on = [] {
    const char* e = getenv("SUBSTATION_B200_PDL");
    return !(e && e[0] == '0');
  }();
  return on;
}

void set_error(const std::string& msg) { g_error = msg; }
int fail(int status, const std::string& msg) {
  g_error = msg;
  return status;
}

namespace {

bool aligned(const void* p, unsigned a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// vec flag: unit stride along `inner`, extent % 8 == 0, other strides % 8 == 0, base aligned.
int vec_flag(const sb_tensor* t, int inner, unsigned align) {
  if (t->stride[inner] != 1 || t->size[inner] % 8 != 0 || !aligned(t->ptr, align)) return 0;
  for (int i = 0; i < t->ndim; ++i)
    if (i != inner && t->size[i] > 1 && t->stride[i] % 8 != 0) return 0;
  return 1;
}

int check_tensor(const sb_tensor* t, int ndim, const char* what) {
  if (!t) return fail(SB_ERR_ARG, std::string(what) + ": null tensor");
  if (t->ndim != ndim)
    return fail(SB_ERR_ARG, std::string(what) + ": expected rank " + std::to_string(ndim) + ", got " +
                                std::to_string(t->ndim));
  long long n = 1;
  for (int i = 0; i < ndim; ++i) {
    if (t->size[i] < 0) return fail(SB_ERR_ARG, std::string(what) + ": negative extent");
    n *= t->size[i];
  }
  if (n > 0 && !t->ptr) return fail(SB_ERR_ARG, std::string(what) + ": null data pointer");
  return SB_OK;
}

int same_shape(const sb_tensor* a, const sb_tensor* b, const char* what) {
  for (int i = 0; i < a->ndim; ++i)
    if (a->size[i] != b->size[i]) return fail(SB_ERR_ARG, std::string(what) + ": extent mismatch between operands");
  return SB_OK;
}

int fits_int(const sb_tensor* t, const char* what) {
  for (int i = 0; i < t->ndim; ++i)
    if (t->size[i] > 0x7fffffffLL) return fail(SB_ERR_UNSUPPORTED, std::string(what) + ": extent exceeds 2^31-1");
  return SB_OK;
}

int to_view3(const sb_tensor* t, const sb_tensor* shape_ref, bool is_mask, const char* what, View3* v) {
  SB_TRY(check_tensor(t, 3, what));
  SB_TRY(fits_int(t, what));
  if (shape_ref) SB_TRY(same_shape(shape_ref, t, what));
  v->p = t->ptr; v->sB = t->stride[0]; v->sJ = t->stride[1]; v->sF = t->stride[2];
  v->vec = vec_flag(t, 2, is_mask ? 8 : 16);
  return SB_OK;
}
int to_view2(const sb_tensor* t, const sb_tensor* ref3, const char* what, View2* v) {
  SB_TRY(check_tensor(t, 2, what));
  if (t->size[0] != ref3->size[0] || t->size[1] != ref3->size[1])
    return fail(SB_ERR_ARG, std::string(what) + ": extent mismatch between operands");
  v->p = t->ptr; v->sB = t->stride[0]; v->sJ = t->stride[1];
  return SB_OK;
}
int to_view4(const sb_tensor* t, const sb_tensor* shape_ref, bool is_mask, const char* what, View4* v) {
  SB_TRY(check_tensor(t, 4, what));
  SB_TRY(fits_int(t, what));
  if (shape_ref) SB_TRY(same_shape(shape_ref, t, what));
  v->p = t->ptr; v->sH = t->stride[0]; v->sB = t->stride[1]; v->sJ = t->stride[2]; v->sK = t->stride[3];
  v->vec = vec_flag(t, 3, is_mask ? 8 : 16);
  return SB_OK;
}
int to_view5(const sb_tensor* t, const sb_tensor* shape_ref, const char* what, View5* v) {
  SB_TRY(check_tensor(t, 5, what));
  SB_TRY(fits_int(t, what));
  if (shape_ref) SB_TRY(same_shape(shape_ref, t, what));
  v->p = t->ptr; v->sN = t->stride[0]; v->sP = t->stride[1]; v->sH = t->stride[2];
  v->sB = t->stride[3]; v->sJ = t->stride[4];
  v->vec = vec_flag(t, 4, 16);
  return SB_OK;
}
// Per-feature vector [F]: must be contiguous.
int to_param(const sb_tensor* t, long long F, const char* what, void** p) {
  SB_TRY(check_tensor(t, 1, what));
  if (t->size[0] != F) return fail(SB_ERR_ARG, std::string(what) + ": extent mismatch between operands");
  if (F > 1 && t->stride[0] != 1) return fail(SB_ERR_UNSUPPORTED, std::string(what) + ": per-feature vectors must be contiguous");
  *p = t->ptr;
  return SB_OK;
}

int to_rng(const sb_dropout* d, Rng* r) {
  if (!d) return fail(SB_ERR_ARG, "dropout: null descriptor");
  if (!(d->p >= 0.f && d->p < 1.f)) return fail(SB_ERR_ARG, "dropout: probability must be in [0,1)");
  if (d->mode != SB_MASK_EXPLICIT && d->mode != SB_MASK_PHILOX) return fail(SB_ERR_ARG, "dropout: unknown mask mode");
  r->seed_lo = (uint32_t)d->seed; r->seed_hi = (uint32_t)(d->seed >> 32);
  r->off_lo = (uint32_t)d->offset; r->off_hi = (uint32_t)(d->offset >> 32);
  long thr = lrintf(d->p * 65536.f);
  if (thr < 0) thr = 0;
  if (thr > 65535) thr = 65535;
  r->thr = (uint32_t)thr;
  r->philox = d->mode == SB_MASK_PHILOX ? 1 : 0;
  return SB_OK;
}

Dims3 dims3(const sb_tensor* t) { return Dims3{(int)t->size[0], (int)t->size[1], (int)t->size[2]}; }
Dims4 dims4(const sb_tensor* t) { return Dims4{(int)t->size[0], (int)t->size[1], (int)t->size[2], (int)t->size[3]}; }
Dims5 dims5(const sb_tensor* t) {
  return Dims5{(int)t->size[0], (int)t->size[1], (int)t->size[2], (int)t->size[3], (int)t->size[4]};
}

int check_activation(int a) {
  if (a != SB_ACT_RELU && a != SB_ACT_GELU) return fail(SB_ERR_ARG, "unknown activation");
  return SB_OK;
}

}  // namespace
}  // namespace sb

using namespace sb;

// ---------------------------------------------------------------------------
// Miscellaneous
// ---------------------------------------------------------------------------
extern "C" const char* sb_status_string(int status) {
  switch (status) {
    case SB_OK: return "ok";
    case SB_ERR_ARG: return "invalid argument";
    case SB_ERR_LAYOUT: return "invalid layout";
    case SB_ERR_UNSUPPORTED: return "unsupported";
    case SB_ERR_CUDA: return "CUDA error";
    case SB_ERR_ALIGNMENT: return "misaligned operand";
    case SB_ERR_DEVICE: return "device-side wait ran out";
    default: return "unknown status";
  }
}
extern "C" const char* sb_last_error(void) { return g_error.c_str(); }
extern "C" const char* sb_version(void) { return "0.2 sm_100a " SB_DTYPE_NAME; }
extern "C" size_t sb_workspace_bytes(void) { return kWsBytes; }

// ---------------------------------------------------------------------------
// Fused operators
// ---------------------------------------------------------------------------
extern "C" int sb_attention_input_biases(void* stream, const sb_tensor* in, const sb_tensor* bias,
                                         const sb_tensor* out) {
  View5 vi, vo;
  SB_TRY(to_view5(in, nullptr, "aib.in", &vi));
  SB_TRY(to_view5(out, in, "aib.out", &vo));
  SB_TRY(check_tensor(bias, 3, "aib.bias"));
  for (int i = 0; i < 3; ++i)
    if (bias->size[i] != in->size[i]) return fail(SB_ERR_ARG, "aib.bias: extent mismatch between operands");
  return launch_aib((cudaStream_t)stream, dims5(in), vi, bias->ptr, bias->stride[0], bias->stride[1],
                    bias->stride[2], vo);
}

extern "C" int sb_softmax_dropout(void* stream, const sb_tensor* beta, const sb_tensor* alpha,
                                  const sb_tensor* mask, const sb_tensor* drop, float scale,
                                  const sb_dropout* dropout) {
  View4 vb, va, vm, vd;
  Rng rng;
  SB_TRY(to_view4(beta, nullptr, false, "softmax.beta", &vb));
  SB_TRY(to_view4(alpha, beta, false, "softmax.alpha", &va));
  SB_TRY(to_view4(mask, beta, true, "softmax.mask", &vm));
  SB_TRY(to_view4(drop, beta, false, "softmax.drop", &vd));
  SB_TRY(to_rng(dropout, &rng));
  return launch_softmax_fwd((cudaStream_t)stream, dims4(beta), vb, va, vm, vd, scale, rng);
}

namespace {
// [P,H,B,rows] projection as a View4 whose fields carry the (P,H,B,row) strides
int to_proj(const sb_tensor* t, const sb_tensor* scores, const char* what, View4* v, int* P) {
  SB_TRY(check_tensor(t, 4, what));
  SB_TRY(fits_int(t, what));
  if (t->size[1] != scores->size[0] || t->size[2] != scores->size[1] || t->size[3] != scores->size[2])
    return fail(SB_ERR_ARG, std::string(what) + ": extent mismatch between operands");
  v->p = t->ptr; v->sH = t->stride[0]; v->sB = t->stride[1]; v->sJ = t->stride[2]; v->sK = t->stride[3];
  v->vec = 0;
  *P = (int)t->size[0];
  return SB_OK;
}
}  // namespace

extern "C" int sb_attention_scores_softmax(void* stream, const sb_tensor* qq, const sb_tensor* kk,
                                           const sb_tensor* beta, const sb_tensor* alpha, const sb_tensor* mask,
                                           const sb_tensor* drop, float scale, const sb_dropout* dropout) {
  View4 vq, vk, vb, va, vm, vd;
  Rng rng;
  int P = 0, P2 = 0;
  SB_TRY(to_view4(alpha, nullptr, false, "scores.alpha", &va));
  if (beta) SB_TRY(to_view4(beta, alpha, false, "scores.beta", &vb));
  else { vb = va; vb.p = nullptr; }   // not wanted: never stored
  SB_TRY(to_view4(mask, alpha, true, "scores.mask", &vm));
  SB_TRY(to_view4(drop, alpha, false, "scores.drop", &vd));
  SB_TRY(to_proj(qq, alpha, "scores.qq", &vq, &P));
  SB_TRY(to_proj(kk, alpha, "scores.kk", &vk, &P2));
  if (P != P2) return fail(SB_ERR_ARG, "scores: head size differs between queries and keys");
  if (alpha->size[2] != alpha->size[3]) return fail(SB_ERR_UNSUPPORTED, "scores: self-attention only (J must equal K)");
  SB_TRY(to_rng(dropout, &rng));
  return launch_attn_scores_fwd((cudaStream_t)stream, dims4(alpha), P, vq, vk, vb, va, vm, vd, scale, rng);
}

extern "C" int sb_attention_scores_softmax_backward(void* stream, const sb_tensor* dgamma, const sb_tensor* vv,
                                                    const sb_tensor* alpha, const sb_tensor* mask,
                                                    const sb_tensor* dattn_drop, const sb_tensor* dbeta) {
  View4 vg, vvv, va, vm, vd, vo;
  int P = 0, P2 = 0;
  SB_TRY(to_view4(alpha, nullptr, false, "scores_bwd.alpha", &va));
  SB_TRY(to_view4(mask, alpha, true, "scores_bwd.mask", &vm));
  if (dattn_drop) SB_TRY(to_view4(dattn_drop, alpha, false, "scores_bwd.dattn_drop", &vd));
  else { vd = va; vd.p = nullptr; }   // not wanted: never stored
  SB_TRY(to_view4(dbeta, alpha, false, "scores_bwd.dbeta", &vo));
  SB_TRY(to_proj(dgamma, alpha, "scores_bwd.dgamma", &vg, &P));
  SB_TRY(to_proj(vv, alpha, "scores_bwd.vv", &vvv, &P2));
  if (P != P2) return fail(SB_ERR_ARG, "scores_bwd: head size differs between operands");
  if (alpha->size[2] != alpha->size[3]) return fail(SB_ERR_UNSUPPORTED, "scores_bwd: self-attention only");
  return launch_attn_scores_bwd((cudaStream_t)stream, dims4(alpha), P, vg, vvv, va, vm, vd, vo);
}

extern "C" int sb_attention_score_contractions(void* stream, const sb_tensor* scores, const sb_tensor* x,
                                               const sb_tensor* out_rows, const sb_tensor* y,
                                               const sb_tensor* out_cols, float alpha) {
  View4 vs, vx, vr, vy, vc;
  if ((x == nullptr) != (out_rows == nullptr) || (y == nullptr) != (out_cols == nullptr))
    return fail(SB_ERR_ARG, "score_contractions: an operand and its output are given together or not at all");
  SB_TRY(to_view4(scores, nullptr, false, "score_contractions.scores", &vs));
  if (scores->size[2] != scores->size[3]) return fail(SB_ERR_UNSUPPORTED, "score_contractions: self-attention only");
  int P = 64, Pi = 0;
  if (x) {
    SB_TRY(to_proj(x, scores, "score_contractions.x", &vx, &P));
    SB_TRY(to_proj(out_rows, scores, "score_contractions.out_rows", &vr, &Pi));
    if (P != Pi) return fail(SB_ERR_ARG, "score_contractions: head size differs between operands");
  }
  if (y) {
    SB_TRY(to_proj(y, scores, "score_contractions.y", &vy, &Pi));
    if (x && P != Pi) return fail(SB_ERR_ARG, "score_contractions: head size differs between operands");
    P = Pi;
    SB_TRY(to_proj(out_cols, scores, "score_contractions.out_cols", &vc, &Pi));
    if (P != Pi) return fail(SB_ERR_ARG, "score_contractions: head size differs between operands");
  }
  return launch_score_contract((cudaStream_t)stream, dims4(scores), P, vs, x ? &vx : nullptr, x ? &vr : nullptr,
                               y ? &vy : nullptr, y ? &vc : nullptr, alpha);
}

extern "C" int sb_backward_softmax(void* stream, const sb_tensor* alpha, const sb_tensor* mask,
                                   const sb_tensor* dattn_drop, const sb_tensor* dbeta) {
  View4 va, vm, vg, vo;
  SB_TRY(to_view4(alpha, nullptr, false, "bs.alpha", &va));
  SB_TRY(to_view4(mask, alpha, true, "bs.mask", &vm));
  SB_TRY(to_view4(dattn_drop, alpha, false, "bs.dattn_drop", &vg));
  SB_TRY(to_view4(dbeta, alpha, false, "bs.dbeta", &vo));
  return launch_softmax_bwd((cudaStream_t)stream, dims4(alpha), va, vm, vg, vo);
}

extern "C" int sb_bias_dropout_residual_layernorm(void* stream, const sb_tensor* in, const sb_tensor* bias,
                                                  const sb_tensor* resid, const sb_tensor* gamma,
                                                  const sb_tensor* beta, const sb_tensor* mask,
                                                  const sb_tensor* lin, const sb_tensor* diff,
                                                  const sb_tensor* istd, const sb_tensor* ln,
                                                  const sb_tensor* out, const sb_dropout* dropout) {
  View3 vin, vres, vmask, vlin, vdiff, vln, vout;
  View2 vistd;
  void *pb, *pg, *pbt;
  Rng rng;
  SB_TRY(to_view3(in, nullptr, false, "bdrln.in", &vin));
  SB_TRY(to_view3(resid, in, false, "bdrln.resid", &vres));
  SB_TRY(to_view3(mask, in, true, "bdrln.mask", &vmask));
  if (lin) SB_TRY(to_view3(lin, in, false, "bdrln.lin", &vlin));
  else { vlin = vin; vlin.p = nullptr; }   // not wanted: never stored
  SB_TRY(to_view3(diff, in, false, "bdrln.diff", &vdiff));
  SB_TRY(to_view3(ln, in, false, "bdrln.ln", &vln));
  SB_TRY(to_view3(out, in, false, "bdrln.out", &vout));
  SB_TRY(to_view2(istd, in, "bdrln.istd", &vistd));
  SB_TRY(to_param(bias, in->size[2], "bdrln.bias", &pb));
  SB_TRY(to_param(gamma, in->size[2], "bdrln.gamma", &pg));
  SB_TRY(to_param(beta, in->size[2], "bdrln.beta", &pbt));
  SB_TRY(to_rng(dropout, &rng));
  if (lin && lin->ptr == in->ptr && (vlin.sB != vin.sB || vlin.sJ != vin.sJ || vlin.sF != vin.sF))
    return fail(SB_ERR_ARG, "bdrln: lin aliases in but has different strides");
  return launch_bdrln((cudaStream_t)stream, dims3(in), vin, pb, vres, pg, pbt, vmask, vlin, vdiff, vistd,
                      vln, vout, rng);
}

extern "C" int sb_bias_activation_dropout(void* stream, const sb_tensor* in, const sb_tensor* bias,
                                          const sb_tensor* mask, const sb_tensor* lin1,
                                          const sb_tensor* drop2, int activation,
                                          const sb_dropout* dropout) {
  View3 vin, vmask, vlin, vdrop;
  void* pb;
  Rng rng;
  SB_TRY(check_activation(activation));
  SB_TRY(to_view3(in, nullptr, false, "bad.in", &vin));
  SB_TRY(to_view3(mask, in, true, "bad.mask", &vmask));
  SB_TRY(to_view3(lin1, in, false, "bad.lin1", &vlin));
  SB_TRY(to_view3(drop2, in, false, "bad.drop2", &vdrop));
  SB_TRY(to_param(bias, in->size[2], "bad.bias", &pb));
  SB_TRY(to_rng(dropout, &rng));
  return launch_bad((cudaStream_t)stream, dims3(in), vin, pb, vmask, vlin, vdrop, activation, rng);
}

extern "C" int sb_backward_scale_bias(void* stream, void* workspace, const sb_tensor* dy, const sb_tensor* ln,
                                      const sb_tensor* gamma, const sb_tensor* dln, const sb_tensor* dgamma,
                                      const sb_tensor* dbeta) {
  View3 vdy, vln, vdln;
  void *pg, *pdg, *pdb;
  SB_TRY(to_view3(dy, nullptr, false, "bsb.dy", &vdy));
  SB_TRY(to_view3(ln, dy, false, "bsb.ln", &vln));
  SB_TRY(to_view3(dln, dy, false, "bsb.dln", &vdln));
  SB_TRY(to_param(gamma, dy->size[2], "bsb.gamma", &pg));
  SB_TRY(to_param(dgamma, dy->size[2], "bsb.dgamma", &pdg));
  SB_TRY(to_param(dbeta, dy->size[2], "bsb.dbeta", &pdb));
  return launch_bsb((cudaStream_t)stream, workspace, dims3(dy), vdy, vln, pg, vdln, pdg, pdb);
}

extern "C" int sb_backward_layernorm_residual_dropout(void* stream, const sb_tensor* dln, const sb_tensor* istd,
                                                      const sb_tensor* diff, const sb_tensor* mask,
                                                      const sb_tensor* dresid, const sb_tensor* dlin) {
  View3 vg, vd, vm, vr, vl;
  View2 vs;
  SB_TRY(to_view3(dln, nullptr, false, "blnrd.dln", &vg));
  SB_TRY(to_view3(diff, dln, false, "blnrd.diff", &vd));
  SB_TRY(to_view3(mask, dln, true, "blnrd.mask", &vm));
  SB_TRY(to_view3(dresid, dln, false, "blnrd.dresid", &vr));
  SB_TRY(to_view3(dlin, dln, false, "blnrd.dlin", &vl));
  SB_TRY(to_view2(istd, dln, "blnrd.istd", &vs));
  return launch_blnrd((cudaStream_t)stream, dims3(dln), vg, vs, vd, vm, vr, vl);
}

extern "C" int sb_backward_dropout_activation_bias(void* stream, void* workspace, const sb_tensor* ddrop2,
                                                   const sb_tensor* mask, const sb_tensor* lin1,
                                                   const sb_tensor* dlin1, const sb_tensor* dbias,
                                                   int activation) {
  View3 vg, vm, vx, vo;
  void* pdb;
  SB_TRY(check_activation(activation));
  SB_TRY(to_view3(ddrop2, nullptr, false, "bdrlb.ddrop2", &vg));
  SB_TRY(to_view3(mask, ddrop2, true, "bdrlb.mask", &vm));
  SB_TRY(to_view3(lin1, ddrop2, false, "bdrlb.lin1", &vx));
  SB_TRY(to_view3(dlin1, ddrop2, false, "bdrlb.dlin1", &vo));
  SB_TRY(to_param(dbias, ddrop2->size[2], "bdrlb.dbias", &pdb));
  return launch_bdrlb((cudaStream_t)stream, workspace, dims3(ddrop2), vg, vm, vx, vo, pdb, activation);
}

extern "C" int sb_extended_backward_scale_bias(void* stream, void* workspace, const sb_tensor* ln1,
                                               const sb_tensor* gamma1, const sb_tensor* dresid2,
                                               const sb_tensor* dlin1_linw1, const sb_tensor* dlin2,
                                               const sb_tensor* dln1, const sb_tensor* dgamma1,
                                               const sb_tensor* dbeta1, const sb_tensor* dlinb2) {
  View3 vn, vr, vw, vl2, vo;
  void *pg, *pdg, *pdb, *pdl;
  SB_TRY(to_view3(ln1, nullptr, false, "ebsb.ln1", &vn));
  SB_TRY(to_view3(dresid2, ln1, false, "ebsb.dresid2", &vr));
  SB_TRY(to_view3(dlin1_linw1, ln1, false, "ebsb.dlin1_linw1", &vw));
  SB_TRY(to_view3(dlin2, ln1, false, "ebsb.dlin2", &vl2));
  SB_TRY(to_view3(dln1, ln1, false, "ebsb.dln1", &vo));
  SB_TRY(to_param(gamma1, ln1->size[2], "ebsb.gamma1", &pg));
  SB_TRY(to_param(dgamma1, ln1->size[2], "ebsb.dgamma1", &pdg));
  SB_TRY(to_param(dbeta1, ln1->size[2], "ebsb.dbeta1", &pdb));
  SB_TRY(to_param(dlinb2, ln1->size[2], "ebsb.dlinb2", &pdl));
  return launch_ebsb((cudaStream_t)stream, workspace, dims3(ln1), vn, pg, vr, vw, vl2, vo, pdg, pdb, pdl);
}

extern "C" int sb_backward_scale_bias_layernorm(void* stream, void* workspace, const sb_tensor* dy,
                                                const sb_tensor* ln, const sb_tensor* gamma, const sb_tensor* istd,
                                                const sb_tensor* diff, const sb_tensor* mask, const sb_tensor* dln,
                                                const sb_tensor* dresid, const sb_tensor* dlin,
                                                const sb_tensor* dgamma, const sb_tensor* dbeta) {
  View3 vy, vn, vd, vm, vg, vr, vl;
  View2 vs;
  void *pg, *pdg, *pdb;
  SB_TRY(to_view3(dy, nullptr, false, "bsb+blnrd.dy", &vy));
  SB_TRY(to_view3(ln, dy, false, "bsb+blnrd.ln", &vn));
  SB_TRY(to_view3(diff, dy, false, "bsb+blnrd.diff", &vd));
  SB_TRY(to_view3(mask, dy, true, "bsb+blnrd.mask", &vm));
  if (dln) SB_TRY(to_view3(dln, dy, false, "bsb+blnrd.dln", &vg));
  else { vg = vy; vg.p = nullptr; }   // not wanted: never stored
  SB_TRY(to_view3(dresid, dy, false, "bsb+blnrd.dresid", &vr));
  SB_TRY(to_view3(dlin, dy, false, "bsb+blnrd.dlin", &vl));
  SB_TRY(to_view2(istd, dy, "bsb+blnrd.istd", &vs));
  SB_TRY(to_param(gamma, dy->size[2], "bsb+blnrd.gamma", &pg));
  SB_TRY(to_param(dgamma, dy->size[2], "bsb+blnrd.dgamma", &pdg));
  SB_TRY(to_param(dbeta, dy->size[2], "bsb+blnrd.dbeta", &pdb));
  return launch_lnbwd_a((cudaStream_t)stream, workspace, dims3(dy), vy, vn, pg, vs, vd, vm, vg, vr, vl, pdg, pdb);
}

extern "C" int sb_extended_backward_scale_bias_layernorm(
    void* stream, void* workspace, const sb_tensor* ln1, const sb_tensor* gamma1, const sb_tensor* dresid2,
    const sb_tensor* dlin1_linw1, const sb_tensor* dlin2, const sb_tensor* istd, const sb_tensor* diff,
    const sb_tensor* mask, const sb_tensor* dln1, const sb_tensor* dresid1, const sb_tensor* datt,
    const sb_tensor* dgamma1, const sb_tensor* dbeta1, const sb_tensor* dlinb2, const sb_tensor* dbo) {
  View3 vn, vr2, vw, vl2, vd, vm, vg, vr, va;
  View2 vs;
  void *pg, *p0, *p1, *p2, *p3;
  SB_TRY(to_view3(ln1, nullptr, false, "ebsb+blnrd.ln1", &vn));
  SB_TRY(to_view3(dresid2, ln1, false, "ebsb+blnrd.dresid2", &vr2));
  SB_TRY(to_view3(dlin1_linw1, ln1, false, "ebsb+blnrd.dlin1_linw1", &vw));
  SB_TRY(to_view3(dlin2, ln1, false, "ebsb+blnrd.dlin2", &vl2));
  SB_TRY(to_view3(diff, ln1, false, "ebsb+blnrd.diff", &vd));
  SB_TRY(to_view3(mask, ln1, true, "ebsb+blnrd.mask", &vm));
  if (dln1) SB_TRY(to_view3(dln1, ln1, false, "ebsb+blnrd.dln1", &vg));
  else { vg = vn; vg.p = nullptr; }   // not wanted: never stored
  SB_TRY(to_view3(dresid1, ln1, false, "ebsb+blnrd.dresid1", &vr));
  SB_TRY(to_view3(datt, ln1, false, "ebsb+blnrd.datt", &va));
  SB_TRY(to_view2(istd, ln1, "ebsb+blnrd.istd", &vs));
  SB_TRY(to_param(gamma1, ln1->size[2], "ebsb+blnrd.gamma1", &pg));
  SB_TRY(to_param(dgamma1, ln1->size[2], "ebsb+blnrd.dgamma1", &p0));
  SB_TRY(to_param(dbeta1, ln1->size[2], "ebsb+blnrd.dbeta1", &p1));
  SB_TRY(to_param(dlinb2, ln1->size[2], "ebsb+blnrd.dlinb2", &p2));
  SB_TRY(to_param(dbo, ln1->size[2], "ebsb+blnrd.dbo", &p3));
  return launch_lnbwd_b((cudaStream_t)stream, workspace, dims3(ln1), vn, pg, vr2, vw, vl2, vs, vd, vm, vg, vr, va,
                        p0, p1, p2, p3);
}

extern "C" int sb_backward_attn_out_bias(void* stream, void* workspace, const sb_tensor* datt,
                                         const sb_tensor* dbo) {
  View3 v;
  void* p;
  SB_TRY(to_view3(datt, nullptr, false, "baob.datt", &v));
  SB_TRY(to_param(dbo, datt->size[2], "baob.dbo", &p));
  return launch_baob((cudaStream_t)stream, workspace, dims3(datt), v, p);
}

extern "C" int sb_backward_attention_input_biases(void* stream, const sb_tensor* d, const sb_tensor* dbias) {
  View5 v;
  SB_TRY(to_view5(d, nullptr, "baib.d", &v));
  SB_TRY(check_tensor(dbias, 3, "baib.dbias"));
  for (int i = 0; i < 3; ++i)
    if (dbias->size[i] != d->size[i]) return fail(SB_ERR_ARG, "baib.dbias: extent mismatch between operands");
  return launch_baib((cudaStream_t)stream, dims5(d), v, dbias->ptr, dbias->stride[0], dbias->stride[1],
                     dbias->stride[2]);
}

extern "C" int sb_backward_encoder_input(void* stream, const sb_tensor* dxatt, const sb_tensor* dresid1,
                                         const sb_tensor* dx) {
  View3 a, b, o;
  SB_TRY(to_view3(dxatt, nullptr, false, "bei.dxatt", &a));
  SB_TRY(to_view3(dresid1, dxatt, false, "bei.dresid1", &b));
  SB_TRY(to_view3(dx, dxatt, false, "bei.dx", &o));
  return launch_bei((cudaStream_t)stream, dims3(dxatt), a, b, o);
}

extern "C" int sb_einsum(void* stream, const char* a_dims, const sb_tensor* a, const char* b_dims,
                         const sb_tensor* b, const char* c_dims, const sb_tensor* c, float alpha, int impl,
                         void* workspace, size_t workspace_bytes) {
  GemmProblem g;
  SB_TRY(plan_einsum(a_dims, a, b_dims, b, c_dims, c, alpha, &g));
  if (workspace && (reinterpret_cast<uintptr_t>(workspace) & 15u))
    return fail(SB_ERR_ALIGNMENT, "einsum: workspace must be 16-byte aligned");
  return run_gemm((cudaStream_t)stream, g, impl, workspace, workspace ? workspace_bytes : 0);
}
namespace {
bool same_geometry(const sb_tensor* t, const sb_tensor* c) {
  if (!t || !t->ptr || t->ndim != c->ndim) return false;
  for (int i = 0; i < c->ndim; ++i)
    if (t->size[i] != c->size[i] || t->stride[i] != c->stride[i]) return false;
  return true;
}
}  // namespace

extern "C" int sb_einsum_fused(void* stream, const char* a_dims, const sb_tensor* a, const char* b_dims,
                               const sb_tensor* b, const char* c_dims, const sb_tensor* c, float alpha,
                               const sb_epilogue* ep) {
  if (!ep) return fail(SB_ERR_ARG, "einsum_fused: null epilogue");
  GemmProblem g;
  SB_TRY(plan_einsum(a_dims, a, b_dims, b, c_dims, c, alpha, &g));
  GemmEpilogue ge{};
  ge.kind = ep->kind;
  if (ep->kind != SB_EPI_BIAS && ep->kind != SB_EPI_RESIDUAL && ep->kind != SB_EPI_BIAS_ACT_DROPOUT)
    return fail(SB_ERR_ARG, "einsum_fused: unknown epilogue kind");
  if (!same_geometry(ep->out2, c)) return fail(SB_ERR_ARG, "einsum_fused: out2 must have the sizes and strides of c");
  ge.out2 = ep->out2->ptr;
  const std::string ad(a_dims), bd(b_dims), cd(c_dims);
  if (ep->kind == SB_EPI_BIAS || ep->kind == SB_EPI_BIAS_ACT_DROPOUT) {
    if (!ep->bias || !ep->bias->ptr || !ep->bias_dims) return fail(SB_ERR_ARG, "einsum_fused: bias missing");
    const std::string vd(ep->bias_dims);
    if ((int)vd.size() != ep->bias->ndim) return fail(SB_ERR_ARG, "einsum_fused: bias dims do not match its rank");
    // the bias indices must be exactly the indices of c that come from one operand only
    auto only = [&](const std::string& mine, const std::string& other) {
      std::string r;
      for (char ch : cd)
        if (mine.find(ch) != std::string::npos && other.find(ch) == std::string::npos) r += ch;
      return r;
    };
    const std::string m_group = only(ad, bd), n_group = only(bd, ad);
    auto same_set = [](std::string x, std::string y) {
      std::sort(x.begin(), x.end());
      std::sort(y.begin(), y.end());
      return x == y;
    };
    int along_m;
    if (same_set(vd, m_group)) along_m = 1;
    else if (same_set(vd, n_group)) along_m = 0;
    else return fail(SB_ERR_UNSUPPORTED, "einsum_fused: bias does not span one operand's own indices of c");
    const long long unit = along_m ? g.sCm : g.sCn;
    for (size_t i = 0; i < vd.size(); ++i) {
      const size_t ci = cd.find(vd[i]);
      if (ep->bias->size[i] != c->size[ci]) return fail(SB_ERR_ARG, "einsum_fused: bias extent differs from c");
      if (c->size[ci] > 1 && c->stride[ci] != ep->bias->stride[i] * unit)
        return fail(SB_ERR_UNSUPPORTED, "einsum_fused: bias is not nested like the matching indices of c");
    }
    ge.vec = ep->bias->ptr;
    ge.vec_along_m = along_m;
  }
  if (ep->kind == SB_EPI_RESIDUAL) {
    if (!same_geometry(ep->resid, c)) return fail(SB_ERR_ARG, "einsum_fused: resid must have the sizes and strides of c");
    ge.resid = ep->resid->ptr;
  }
  if (ep->kind == SB_EPI_BIAS_ACT_DROPOUT) {
    if (!same_geometry(ep->out3, c) || !same_geometry(ep->mask, c))
      return fail(SB_ERR_ARG, "einsum_fused: out3 and mask must have the sizes and strides of c");
    SB_TRY(check_activation(ep->activation));
    SB_TRY(to_rng(ep->dropout, &ge.rng));
    ge.out3 = ep->out3->ptr;
    ge.mask = ep->mask->ptr;
    ge.activation = ep->activation;
    if (ge.rng.philox) {
      // the generator is keyed by the logical element index: c must be dense in logical order
      if (!ep->logical_dims || cd != ep->logical_dims)
        return fail(SB_ERR_UNSUPPORTED, "einsum_fused: in-kernel masks need c stored in its logical order");
      long long dense = 1;
      for (int i = c->ndim - 1; i >= 0; --i) {
        if (c->size[i] > 1 && c->stride[i] != dense)
          return fail(SB_ERR_UNSUPPORTED, "einsum_fused: in-kernel masks need a dense c");
        dense *= c->size[i];
      }
    }
  }
  ge.skip_c = ep->discard_c ? 1 : 0;
  // The epilogue reads bias, residual and mask with 128-bit accesses: refuse operands it could not read that
  // way before anything is launched (the caller then runs the two operators separately).
  if (ge.vec && !aligned(ge.vec, 16)) return fail(SB_ERR_ALIGNMENT, "einsum_fused: bias must be 16-byte aligned");
  if (ge.resid && !aligned(ge.resid, 16)) return fail(SB_ERR_ALIGNMENT, "einsum_fused: resid must be 16-byte aligned");
  if (ge.mask && (!aligned(ge.mask, 16) || std::max(g.sCm, g.sCn) % 16 != 0))
    return fail(SB_ERR_ALIGNMENT, "einsum_fused: mask must be 16-byte aligned and the row pitch of c a multiple of 16");
  return run_gemm_fused((cudaStream_t)stream, g, ge);
}
extern "C" int sb_einsum_last_impl(void) { return g_last_gemm_impl; }
extern "C" int sb_set_sm_budget(int n_sms) {
  if (n_sms < 0) return fail(SB_ERR_ARG, "sb_set_sm_budget: negative SM count");
  set_gemm_sm_budget(n_sms);
  return SB_OK;
}
extern "C" int sb_device_error(void* stream, int* code) {
  if (!code) return fail(SB_ERR_ARG, "sb_device_error: null argument");
  // tcgen05 kernels record codes 1-7, the ring-fed LayerNorm kernels 11-14
  SB_TRY(gemm_device_error((cudaStream_t)stream, code));
  if (*code == 0) SB_TRY(ring_device_error((cudaStream_t)stream, code));
  return SB_OK;
}
extern "C" int sb_device_error_reset(void* stream) {
  SB_TRY(gemm_device_error_reset((cudaStream_t)stream));
  return ring_device_error_reset((cudaStream_t)stream);
}
extern "C" int sb_mma_peak_probe(void* stream, int k_blocks, int bf16, double* flops) {
  return run_mma_peak_probe((cudaStream_t)stream, k_blocks, bf16, flops);
}

// ---------------------------------------------------------------------------
// Whole layer
// ---------------------------------------------------------------------------
namespace {

const char* const kParamNames[SB_NUM_PARAMS] = {"WKQV", "BKQV", "WO", "BO", "S1", "B1",
                                                "LINB1", "LINW1", "S2", "B2", "LINB2", "LINW2"};
const char* const kFwdNames[SB_NUM_FWD_INTERM] = {
    "KKQQVV", "WKKWQQWVV", "BETA", "ALPHA", "ATTN_DROP_MASK", "ATTN_DROP", "GAMMA", "ATT",
    "DROP1MASK", "SB1", "SB1_LINW1", "DROP2", "LIN1", "DROP2_LINW2", "LIN2", "LN2", "LN2STD",
    "LN2DIFF", "DROP2MASK", "DROP3MASK", "LN1", "LN1STD", "LN1DIFF"};
const char* const kBwdNames[SB_NUM_BWD_INTERM] = {
    "DLN2", "DRESID2", "DLIN2", "DDROP2", "DLIN1", "DLIN1_LINW1", "DLN1", "DRESID1", "DATT",
    "DXATT", "DGAMMA", "DATTN_DROP", "DBETA", "DKKQQVV"};

const std::map<std::string, std::string>& logical_dims() {
  static const std::map<std::string, std::string> m = {
      {"X", "BJI"}, {"SB2", "BJI"},
      {"WKQV", "QPHI"}, {"BKQV", "QPH"}, {"WO", "IPH"}, {"BO", "I"}, {"S1", "I"}, {"B1", "I"},
      {"S2", "I"}, {"B2", "I"}, {"LINW1", "IU"}, {"LINB1", "U"}, {"LINW2", "UI"}, {"LINB2", "I"},
      {"KKQQVV", "QPHBJ"}, {"WKKWQQWVV", "QPHBJ"}, {"BETA", "HBJK"}, {"ALPHA", "HBJK"},
      {"ATTN_DROP_MASK", "HBJK"}, {"ATTN_DROP", "HBJK"}, {"GAMMA", "PHBJ"}, {"ATT", "BJI"},
      {"DROP1MASK", "BJI"}, {"SB1", "BJI"}, {"SB1_LINW1", "BJU"}, {"DROP2", "BJU"}, {"LIN1", "BJU"},
      {"DROP2_LINW2", "BJI"}, {"LIN2", "BJI"}, {"LN2", "BJI"}, {"LN2STD", "BJ"}, {"LN2DIFF", "BJI"},
      {"DROP2MASK", "BJU"}, {"DROP3MASK", "BJI"}, {"LN1", "BJI"}, {"LN1STD", "BJ"}, {"LN1DIFF", "BJI"},
      {"DLN2", "BJI"}, {"DRESID2", "BJI"}, {"DLIN2", "BJI"}, {"DDROP2", "BJU"}, {"DLIN1", "BJU"},
      {"DLIN1_LINW1", "BJI"}, {"DLN1", "BJI"}, {"DRESID1", "BJI"}, {"DATT", "BJI"}, {"DXATT", "BJI"},
      {"DGAMMA", "PHBJ"}, {"DATTN_DROP", "HBJK"}, {"DBETA", "HBJK"}, {"DKKQQVV", "QPHBJ"}};
  return m;
}

bool is_permutation(const std::string& a, const std::string& b) {
  if (a.size() != b.size()) return false;
  std::string x = a, y = b;
  std::sort(x.begin(), x.end());
  std::sort(y.begin(), y.end());
  return x == y;
}

}  // namespace

struct sb_encoder {
  int B, S, H, P, I, U;
  int activation;
  float p_softmax, p_resid1, p_act, p_resid2;
  std::map<std::string, std::string> layout;  // name -> dim order in memory
  std::vector<std::string> param_order, fwd_order, bwd_order;
  void* workspace = nullptr;
  void* gemm_ws = nullptr;     // fp32 split-K partials of the weight-gradient contractions
  size_t gemm_ws_bytes = 0;
  int device = 0;
  int launches = 0;
  long long kernels_fwd = 0, kernels_bwd = 0, kernel_base = 0;   // kernels launched by the most recent passes
  // Replay of whole passes as CUDA graphs: a pass whose pointer arguments repeat is captured once (on a private
  // stream, the second time the same arguments are seen) and replayed from then on with one graph launch.
  struct PassGraph {
    std::vector<uint64_t> key;
    cudaGraphExec_t exec = nullptr;
    int launches = 0;
    long long kernels = 0;
    unsigned long long last_use = 0;
  };
  struct GraphCache {
    std::vector<PassGraph> entries;
    std::vector<std::vector<uint64_t>> seen;   // arguments of recent eager calls (a repeat gets captured)
    unsigned long long tick = 0;
    long long captures = 0, replays = 0;
  };
  GraphCache graph_fwd, graph_bwd;
  cudaStream_t capture_stream = nullptr;
  cudaEvent_t ffn_grads_event = nullptr;   // recorded in backward once the feed-forward gradients are final
  bool graphs = true;           // sb_encoder_set_graphs / SUBSTATION_B200_GRAPHS=0
  bool timing = false;
  bool fuse = true;            // use the fused multi-operator kernels where the layouts allow
  bool dead_stores = true;     // write the intermediates nothing reads again (sb_encoder_set_dead_stores)
  std::vector<std::pair<std::string, cudaEvent_t>> marks;
  std::vector<cudaEvent_t> event_pool;
  std::vector<std::pair<std::string, float>> last_times;

  long long extent(char c) const {
    switch (c) {
      case 'B': return B;
      case 'J': case 'K': case 'S': return S;
      case 'H': return H;
      case 'P': return P;
      case 'I': return I;
      case 'U': return U;
      case 'Q': return 3;
      default: return -1;
    }
  }
  long long numel(const std::string& dims) const {
    long long n = 1;
    for (char c : dims) n *= extent(c);
    return n;
  }
  // Tensor in MEMORY order: dims string = layout (optionally with letters renamed), contiguous strides.
  sb_tensor mem(const void* ptr, const std::string& dims) const {
    sb_tensor t;
    t.ptr = const_cast<void*>(ptr);
    t.ndim = (int)dims.size();
    long long st = 1;
    for (int i = t.ndim - 1; i >= 0; --i) {
      t.size[i] = extent(dims[i]);
      t.stride[i] = st;
      st *= t.size[i];
    }
    return t;
  }
  // Tensor viewed in LOGICAL order `logical`, stored contiguously as `lay`.
  sb_tensor view(const void* ptr, const std::string& lay, const std::string& logical) const {
    const sb_tensor m = mem(ptr, lay);
    sb_tensor t;
    t.ptr = m.ptr;
    t.ndim = (int)logical.size();
    for (int i = 0; i < t.ndim; ++i) {
      const size_t d = lay.find(logical[i]);
      t.size[i] = m.size[d];
      t.stride[i] = m.stride[d];
    }
    return t;
  }
  sb_tensor view(const void* ptr, const char* name) const {
    return view(ptr, layout.at(name), logical_dims().at(name));
  }

  // forget the operator just marked (a fused attempt declined before launching anything)
  void unmark() {
    --launches;
    if (timing) close_range();
    if (timing && !marks.empty()) {
      event_pool.push_back(marks.back().second);
      marks.pop_back();
    }
  }
  // rename the operator just marked (a fused attempt fell back to its first separate operator)
  void relabel(const char* name) {
    if (timing && !marks.empty()) {
      marks.back().first = name;
      close_range();
      nvtxRangePushA(name);
      range_open = true;
    }
  }
  // With timing on, every operator is also an NVTX range named like the reference's (pytorch_module/encoder.cu:32-53):
  // a range opens where the operator is enqueued and closes where the next one opens (or the pass ends), so a
  // timeline shows the same names the event table reports.  Without a profiler attached the calls do nothing.
  bool range_open = false;
  void close_range() {
    if (range_open) nvtxRangePop();
    range_open = false;
  }
  void mark(cudaStream_t s, const char* name) {
    ++launches;
    if (!timing) return;
    close_range();
    if (name[0]) {
      nvtxRangePushA(name);
      range_open = true;
    }
    cudaEvent_t e;
    if (event_pool.empty()) cudaEventCreate(&e);
    else { e = event_pool.back(); event_pool.pop_back(); }
    cudaEventRecord(e, s);
    marks.emplace_back(name, e);
  }
};

namespace {

std::string rename(std::string s, char from, char to) {
  for (char& c : s)
    if (c == from) c = to;
  return s;
}

struct Ptrs {
  std::map<std::string, void*> p;
  void* operator[](const char* n) const { return p.at(n); }
};

int einsum(sb_encoder* e, cudaStream_t s, const char* name, const std::string& ad, const void* a,
           const std::string& bd, const void* b, const std::string& cd, void* c, float alpha) {
  e->mark(s, name);
  const sb_tensor ta = e->mem(a, ad), tb = e->mem(b, bd), tc = e->mem(c, cd);
  GemmProblem g;
  SB_TRY(plan_einsum(ad.c_str(), &ta, bd.c_str(), &tb, cd.c_str(), &tc, alpha, &g));
  return run_gemm(s, g, SB_GEMM_AUTO, e->gemm_ws, e->gemm_ws_bytes);
}

// Contraction with the following elementwise operator in its epilogue; SB_ERR_UNSUPPORTED (nothing launched,
// nothing marked) when the contraction kernel that can do it does not take this problem.
int einsum_fused(sb_encoder* e, cudaStream_t s, const char* name, const std::string& ad, const void* a,
                 const std::string& bd, const void* b, const std::string& cd, void* c, float alpha,
                 const sb_epilogue* ep) {
  e->mark(s, name);
  const sb_tensor ta = e->mem(a, ad), tb = e->mem(b, bd), tc = e->mem(c, cd);
  const int st = sb_einsum_fused((void*)s, ad.c_str(), &ta, bd.c_str(), &tb, cd.c_str(), &tc, alpha, ep);
  if (st == SB_ERR_UNSUPPORTED || st == SB_ERR_ALIGNMENT) {
    e->unmark();
    return SB_ERR_UNSUPPORTED;
  }
  return st;
}

}  // namespace

extern "C" int sb_encoder_create(const sb_encoder_config* cfg, sb_encoder** out) {
  if (!cfg || !out) return fail(SB_ERR_ARG, "sb_encoder_create: null argument");
  *out = nullptr;
  if (cfg->batch <= 0 || cfg->seq <= 0 || cfg->heads <= 0 || cfg->embed <= 0)
    return fail(SB_ERR_ARG, "sb_encoder_create: sizes must be positive");
  if (cfg->embed % cfg->heads != 0)
    return fail(SB_ERR_ARG, "sb_encoder_create: embedding size must be a multiple of the head count");
  SB_TRY(check_activation(cfg->activation));
  for (float p : {cfg->p_softmax, cfg->p_resid1, cfg->p_activation, cfg->p_resid2})
    if (!(p >= 0.f && p < 1.f)) return fail(SB_ERR_ARG, "sb_encoder_create: dropout probabilities must be in [0,1)");
  if (cfg->n_tensors <= 0 || !cfg->names || !cfg->dims) return fail(SB_ERR_ARG, "sb_encoder_create: no layouts given");

  std::unique_ptr<sb_encoder> e(new sb_encoder);
  e->B = cfg->batch; e->S = cfg->seq; e->H = cfg->heads; e->I = cfg->embed;
  e->P = cfg->embed / cfg->heads; e->U = 4 * cfg->embed;
  e->activation = cfg->activation;
  e->p_softmax = cfg->p_softmax; e->p_resid1 = cfg->p_resid1;
  e->p_act = cfg->p_activation; e->p_resid2 = cfg->p_resid2;
  const auto& logical = logical_dims();
  auto in_list = [](const char* const* list, int n, const std::string& name) {
    for (int i = 0; i < n; ++i)
      if (name == list[i]) return true;
    return false;
  };
  for (int i = 0; i < cfg->n_tensors; ++i) {
    if (!cfg->names[i] || !cfg->dims[i]) return fail(SB_ERR_ARG, "sb_encoder_create: null layout entry");
    const std::string name = cfg->names[i], dims = cfg->dims[i];
    auto it = logical.find(name);
    if (it == logical.end()) return fail(SB_ERR_LAYOUT, "sb_encoder_create: unknown tensor '" + name + "'");
    if (!is_permutation(dims, it->second))
      return fail(SB_ERR_LAYOUT, "sb_encoder_create: layout '" + dims + "' of " + name +
                                     " is not a permutation of its dims '" + it->second + "'");
    if (e->layout.count(name)) return fail(SB_ERR_LAYOUT, "sb_encoder_create: tensor '" + name + "' listed twice");
    e->layout[name] = dims;
    if (in_list(kParamNames, SB_NUM_PARAMS, name)) e->param_order.push_back(name);
    else if (in_list(kFwdNames, SB_NUM_FWD_INTERM, name)) e->fwd_order.push_back(name);
    else if (in_list(kBwdNames, SB_NUM_BWD_INTERM, name)) e->bwd_order.push_back(name);
  }
  for (const auto& kv : logical)
    if (!e->layout.count(kv.first)) return fail(SB_ERR_LAYOUT, "sb_encoder_create: no layout given for '" + kv.first + "'");
  // Stacked tensors are sliced by pointer offset, so the stacking dim must be outermost.
  for (const char* n : {"KKQQVV", "DKKQQVV", "WKKWQQWVV", "BKQV", "WKQV"})
    if (e->layout[n][0] != 'Q')
      return fail(SB_ERR_LAYOUT, std::string("sb_encoder_create: stacked tensor ") + n + " must have Q outermost");
  if (e->layout["X"] != e->layout["SB2"])
    return fail(SB_ERR_LAYOUT, "sb_encoder_create: input and output layouts must be equal so that layers chain");
  SB_CUDA_OK(cudaGetDevice(&e->device));
  SB_CUDA_OK(cudaMalloc(&e->workspace, kWsBytes));
  SB_CUDA_OK(cudaMemset(e->workspace, 0, kWsBytes));
  // up to four fp32 partial copies of the largest weight gradient (the stacked [3E, E] projection)
  e->gemm_ws_bytes = std::min<size_t>((size_t)4 * 3 * e->I * e->I * sizeof(float), (size_t)512 << 20);
  if (cudaMalloc(&e->gemm_ws, e->gemm_ws_bytes) != cudaSuccess) {
    cudaGetLastError();
    e->gemm_ws = nullptr;       // split-K is an optimisation; run without it
    e->gemm_ws_bytes = 0;
  }
  *out = e.release();
  return SB_OK;
}

extern "C" int sb_encoder_destroy(sb_encoder* e) {
  if (!e) return SB_OK;
  for (auto& m : e->marks) cudaEventDestroy(m.second);
  for (auto ev : e->event_pool) cudaEventDestroy(ev);
  if (e->workspace) cudaFree(e->workspace);
  if (e->gemm_ws) cudaFree(e->gemm_ws);
  for (auto* c : {&e->graph_fwd, &e->graph_bwd})
    for (auto& g : c->entries) cudaGraphExecDestroy(g.exec);
  if (e->capture_stream) cudaStreamDestroy(e->capture_stream);
  delete e;
  return SB_OK;
}

extern "C" int sb_encoder_set_timing(sb_encoder* e, int enabled) {
  if (!e) return fail(SB_ERR_ARG, "null handle");
  e->timing = enabled != 0;
  return SB_OK;
}

extern "C" int sb_encoder_launch_count(sb_encoder* e) { return e ? e->launches : 0; }
extern "C" int sb_encoder_kernel_count(sb_encoder* e) { return e ? (int)(e->kernels_fwd + e->kernels_bwd) : 0; }
extern "C" int sb_encoder_set_fusion(sb_encoder* e, int enabled) {
  if (!e) return fail(SB_ERR_ARG, "null handle");
  e->fuse = enabled != 0;
  return SB_OK;
}

extern "C" int sb_encoder_set_dead_stores(sb_encoder* e, int enabled) {
  if (!e) return fail(SB_ERR_ARG, "null handle");
  e->dead_stores = enabled != 0;
  return SB_OK;
}

extern "C" int sb_encoder_set_graphs(sb_encoder* e, int enabled) {
  if (!e) return fail(SB_ERR_ARG, "null handle");
  e->graphs = enabled != 0;
  return SB_OK;
}

extern "C" int sb_encoder_set_ffn_grads_event(sb_encoder* e, void* event) {
  if (!e) return fail(SB_ERR_ARG, "null handle");
  if (e->ffn_grads_event != (cudaEvent_t)event) {
    // graphs captured so far record the previous event (or none): drop them
    for (auto& g : e->graph_bwd.entries) cudaGraphExecDestroy(g.exec);
    e->graph_bwd.entries.clear();
    e->graph_bwd.seen.clear();
  }
  e->ffn_grads_event = (cudaEvent_t)event;
  return SB_OK;
}

extern "C" int sb_encoder_graph_stats(sb_encoder* e, long long* captures, long long* replays) {
  if (!e || !captures || !replays) return fail(SB_ERR_ARG, "sb_encoder_graph_stats: null argument");
  *captures = e->graph_fwd.captures + e->graph_bwd.captures;
  *replays = e->graph_fwd.replays + e->graph_bwd.replays;
  return SB_OK;
}

extern "C" int sb_encoder_get_timing(sb_encoder* e, int max, const char** names, float* ms) {
  if (!e) return 0;
  if (!e->marks.empty()) {
    // marks: begin-of-op events plus one closing event named "" per pass
    cudaEventSynchronize(e->marks.back().second);
    e->last_times.clear();
    for (size_t i = 0; i + 1 < e->marks.size(); ++i) {
      if (e->marks[i].first.empty()) continue;
      float t = 0.f;
      cudaEventElapsedTime(&t, e->marks[i].second, e->marks[i + 1].second);
      e->last_times.emplace_back(e->marks[i].first, t);
    }
    for (auto& m : e->marks) e->event_pool.push_back(m.second);
    e->marks.clear();
  }
  int n = 0;
  for (auto& kv : e->last_times) {
    if (n >= max) break;
    names[n] = kv.first.c_str();
    ms[n] = kv.second;
    ++n;
  }
  return n;
}

namespace {

int gather(sb_encoder* e, const void* x, const void* const* params, void* const* fwd, Ptrs* P) {
  if (!x || !params || !fwd) return fail(SB_ERR_ARG, "encoder: null pointer table");
  P->p["X"] = const_cast<void*>(x);
  for (size_t i = 0; i < e->param_order.size(); ++i) {
    if (!params[i]) return fail(SB_ERR_ARG, "encoder: null parameter pointer (" + e->param_order[i] + ")");
    P->p[e->param_order[i]] = const_cast<void*>(params[i]);
  }
  for (size_t i = 0; i < e->fwd_order.size(); ++i) {
    if (!fwd[i]) return fail(SB_ERR_ARG, "encoder: null forward-intermediate pointer (" + e->fwd_order[i] + ")");
    P->p[e->fwd_order[i]] = fwd[i];
  }
  return SB_OK;
}

sb_dropout drop(float p, int mode, uint64_t seed, uint64_t offset) {
  sb_dropout d;
  d.p = p; d.mode = mode; d.seed = seed; d.offset = offset;
  return d;
}

}  // namespace

static int forward_pass(sb_encoder* e, void* stream, const void* x, const void* const* params,
                        void* const* fwd, void* y, int mask_mode, uint64_t seed, uint64_t offset) {
  if (!e || !y) return fail(SB_ERR_ARG, "sb_encoder_forward: null argument");
  if (mask_mode != SB_MASK_EXPLICIT && mask_mode != SB_MASK_PHILOX)
    return fail(SB_ERR_ARG, "sb_encoder_forward: unknown mask mode");
  cudaStream_t s = (cudaStream_t)stream;
  Ptrs T;
  SB_TRY(gather(e, x, params, fwd, &T));
  T.p["SB2"] = y;
  e->launches = 0;
  e->kernel_base = g_kernel_launches;
  const auto& L = e->layout;
  const long long slice = (long long)e->P * e->H * e->B * e->S;  // elements per stacked projection
  auto q_slice = [&](const char* name, int q) { return (void*)((sb_half*)T[name] + q * slice); };
  const std::string lKK = L.at("KKQQVV").substr(1);

  // F1: stacked K,Q,V projections
  {
    // the input biases ride on the projection's epilogue when both stacked tensors share a layout
    int st = SB_ERR_UNSUPPORTED;
    if (e->fuse && L.at("WKKWQQWVV") == L.at("KKQQVV")) {
      const sb_tensor out2 = e->mem(T["KKQQVV"], L.at("KKQQVV")), bias = e->mem(T["BKQV"], L.at("BKQV"));
      sb_epilogue ep{};
      ep.kind = SB_EPI_BIAS;
      ep.bias_dims = L.at("BKQV").c_str();
      ep.bias = &bias;
      ep.out2 = &out2;
      ep.discard_c = e->dead_stores ? 0 : 1;   // WKKWQQWVV: only the bias operator reads it
      st = einsum_fused(e, s, "QKV-fused+aib", L.at("X"), T["X"], L.at("WKQV"), T["WKQV"], L.at("WKKWQQWVV"),
                        T["WKKWQQWVV"], 1.f, &ep);
      if (st != SB_OK && st != SB_ERR_UNSUPPORTED) return st;
    }
    if (st == SB_ERR_UNSUPPORTED) {
      SB_TRY(einsum(e, s, "QKV-fused", L.at("X"), T["X"], L.at("WKQV"), T["WKQV"], L.at("WKKWQQWVV"),
                    T["WKKWQQWVV"], 1.f));
      e->mark(s, "aib");
      sb_tensor in = e->view(T["WKKWQQWVV"], "WKKWQQWVV"), out = e->view(T["KKQQVV"], "KKQQVV");
      sb_tensor bias = e->view(T["BKQV"], "BKQV");
      SB_TRY(sb_attention_input_biases(stream, &in, &bias, &out));
    }
  }
  // F2 + softmax.  K and V views are the J-indexed projections relabelled with K.
  {
    sb_tensor beta = e->view(T["BETA"], "BETA"), alpha = e->view(T["ALPHA"], "ALPHA");
    sb_tensor mask = e->view(T["ATTN_DROP_MASK"], "ATTN_DROP_MASK"), dr = e->view(T["ATTN_DROP"], "ATTN_DROP");
    sb_dropout d = drop(e->p_softmax, mask_mode, seed, offset + 0);
    const float scale = 1.f / std::sqrt((float)e->P);
    int st = SB_ERR_UNSUPPORTED;
    if (e->fuse) {
      e->mark(s, "QKT+softmax");
      sb_tensor kk = e->view(q_slice("KKQQVV", 0), lKK, "PHBJ"), qq = e->view(q_slice("KKQQVV", 1), lKK, "PHBJ");
      // BETA is consumed inside the kernel
      st = sb_attention_scores_softmax(stream, &qq, &kk, e->dead_stores ? &beta : nullptr, &alpha, &mask, &dr, scale, &d);
      if (st != SB_OK && st != SB_ERR_UNSUPPORTED) return st;
      if (st == SB_ERR_UNSUPPORTED) e->unmark();
    }
    if (st == SB_ERR_UNSUPPORTED) {
      SB_TRY(einsum(e, s, "QKT", rename(lKK, 'J', 'K'), q_slice("KKQQVV", 0), lKK, q_slice("KKQQVV", 1),
                    L.at("BETA"), T["BETA"], scale));
      e->mark(s, "softmax");
      SB_TRY(sb_softmax_dropout(stream, &beta, &alpha, &mask, &dr, 1.f, &d));
    }
  }
  {
    // one CTA per (head, sample) streams ATTN_DROP once
    int st = SB_ERR_UNSUPPORTED;
    if (e->fuse) {
      e->mark(s, "gamma");
      sb_tensor sc = e->view(T["ATTN_DROP"], "ATTN_DROP"), vv = e->view(q_slice("KKQQVV", 2), lKK, "PHBJ");
      sb_tensor gm = e->view(T["GAMMA"], "GAMMA");
      st = sb_attention_score_contractions(stream, &sc, &vv, &gm, nullptr, nullptr, 1.f);
      if (st != SB_OK && st != SB_ERR_UNSUPPORTED) return st;
      if (st == SB_ERR_UNSUPPORTED) e->unmark();
    }
    if (st == SB_ERR_UNSUPPORTED)
      SB_TRY(einsum(e, s, "gamma", rename(lKK, 'J', 'K'), q_slice("KKQQVV", 2), L.at("ATTN_DROP"), T["ATTN_DROP"],
                    L.at("GAMMA"), T["GAMMA"], 1.f));
  }
  SB_TRY(einsum(e, s, "out", L.at("WO"), T["WO"], L.at("GAMMA"), T["GAMMA"], L.at("ATT"), T["ATT"], 1.f));
  {
    e->mark(s, "bdrln1");
    sb_tensor in = e->view(T["ATT"], "ATT"), resid = e->view(T["X"], "X");
    sb_tensor bias = e->view(T["BO"], "BO"), gamma = e->view(T["S1"], "S1"), beta = e->view(T["B1"], "B1");
    sb_tensor mask = e->view(T["DROP1MASK"], "DROP1MASK"), diff = e->view(T["LN1DIFF"], "LN1DIFF");
    sb_tensor istd = e->view(T["LN1STD"], "LN1STD"), ln = e->view(T["LN1"], "LN1"), out = e->view(T["SB1"], "SB1");
    sb_dropout d = drop(e->p_resid1, mask_mode, seed, offset + 1);
    // the biased projection is written back over ATT (nothing reads it again)
    SB_TRY(sb_bias_dropout_residual_layernorm(stream, &in, &bias, &resid, &gamma, &beta, &mask,
                                              e->dead_stores ? &in : nullptr, &diff, &istd, &ln, &out, &d));
  }
  {
    // bias + activation + dropout in the epilogue of the first feed-forward contraction
    sb_dropout d = drop(e->p_act, mask_mode, seed, offset + 2);
    int st = SB_ERR_UNSUPPORTED;
    const std::string& lc = L.at("SB1_LINW1");
    if (e->fuse && lc == L.at("LIN1") && lc == L.at("DROP2") && lc == L.at("DROP2MASK")) {
      const sb_tensor out2 = e->mem(T["LIN1"], lc), out3 = e->mem(T["DROP2"], lc), mask = e->mem(T["DROP2MASK"], lc);
      const sb_tensor bias = e->mem(T["LINB1"], L.at("LINB1"));
      sb_epilogue ep{};
      ep.kind = SB_EPI_BIAS_ACT_DROPOUT;
      ep.bias_dims = L.at("LINB1").c_str();
      ep.bias = &bias;
      ep.mask = &mask;
      ep.out2 = &out2;
      ep.out3 = &out3;
      ep.activation = e->activation;
      ep.dropout = &d;
      ep.logical_dims = "BJU";
      ep.discard_c = e->dead_stores ? 0 : 1;   // SB1_LINW1: only the bias operator reads it
      st = einsum_fused(e, s, "lin1+bad", L.at("SB1"), T["SB1"], L.at("LINW1"), T["LINW1"], lc, T["SB1_LINW1"], 1.f, &ep);
      if (st != SB_OK && st != SB_ERR_UNSUPPORTED) return st;
    }
    if (st == SB_ERR_UNSUPPORTED) {
      SB_TRY(einsum(e, s, "lin1", L.at("SB1"), T["SB1"], L.at("LINW1"), T["LINW1"], L.at("SB1_LINW1"),
                    T["SB1_LINW1"], 1.f));
      e->mark(s, "bad");
      sb_tensor in = e->view(T["SB1_LINW1"], "SB1_LINW1"), bias = e->view(T["LINB1"], "LINB1");
      sb_tensor mask = e->view(T["DROP2MASK"], "DROP2MASK"), lin1 = e->view(T["LIN1"], "LIN1");
      sb_tensor d2 = e->view(T["DROP2"], "DROP2");
      SB_TRY(sb_bias_activation_dropout(stream, &in, &bias, &mask, &lin1, &d2, e->activation, &d));
    }
  }
  SB_TRY(einsum(e, s, "lin2", L.at("DROP2"), T["DROP2"], L.at("LINW2"), T["LINW2"], L.at("DROP2_LINW2"),
                T["DROP2_LINW2"], 1.f));
  {
    e->mark(s, "bdrln2");
    sb_tensor in = e->view(T["DROP2_LINW2"], "DROP2_LINW2"), resid = e->view(T["SB1"], "SB1");
    sb_tensor bias = e->view(T["LINB2"], "LINB2"), gamma = e->view(T["S2"], "S2"), beta = e->view(T["B2"], "B2");
    sb_tensor mask = e->view(T["DROP3MASK"], "DROP3MASK"), lin = e->view(T["LIN2"], "LIN2");
    sb_tensor diff = e->view(T["LN2DIFF"], "LN2DIFF"), istd = e->view(T["LN2STD"], "LN2STD");
    sb_tensor ln = e->view(T["LN2"], "LN2"), out = e->view(T["SB2"], "SB2");
    sb_dropout d = drop(e->p_resid2, mask_mode, seed, offset + 3);
    // LIN2 is never read again
    SB_TRY(sb_bias_dropout_residual_layernorm(stream, &in, &bias, &resid, &gamma, &beta, &mask,
                                              e->dead_stores ? &lin : nullptr, &diff, &istd, &ln, &out, &d));
  }
  if (e->timing) { e->mark(s, ""); --e->launches; }
  e->kernels_fwd = g_kernel_launches - e->kernel_base;
  return SB_OK;
}

static int backward_pass(sb_encoder* e, void* stream, const void* dy, void* const* dparams,
                         void* const* bwd, const void* const* params, void* const* fwd,
                         const void* x, void* dx) {
  if (!e || !dy || !dparams || !bwd || !dx) return fail(SB_ERR_ARG, "sb_encoder_backward: null argument");
  cudaStream_t s = (cudaStream_t)stream;
  Ptrs T;
  SB_TRY(gather(e, x, params, fwd, &T));
  for (size_t i = 0; i < e->bwd_order.size(); ++i) {
    if (!bwd[i]) return fail(SB_ERR_ARG, "encoder: null backward-intermediate pointer (" + e->bwd_order[i] + ")");
    T.p[e->bwd_order[i]] = bwd[i];
  }
  std::map<std::string, void*> D;  // parameter gradients
  for (size_t i = 0; i < e->param_order.size(); ++i) {
    if (!dparams[i]) return fail(SB_ERR_ARG, "encoder: null gradient pointer (" + e->param_order[i] + ")");
    D[e->param_order[i]] = dparams[i];
  }
  e->launches = 0;
  e->kernel_base = g_kernel_launches;
  const auto& L = e->layout;
  const long long slice = (long long)e->P * e->H * e->B * e->S;
  auto q_slice = [&](void* base, int q) { return (void*)((sb_half*)base + q * slice); };
  const std::string lKK = L.at("KKQQVV").substr(1), lDKK = L.at("DKKQQVV").substr(1);
  void* ws = e->workspace;
  auto v = [&](const char* name) { return e->view(T[name], name); };
  auto pv = [&](const char* name) { return e->view(T[name], name); };
  auto dv = [&](const char* name) { return e->view(D.at(name), L.at(name), logical_dims().at(name)); };
  const sb_tensor tDY = e->view(dy, L.at("SB2"), "BJI");
  const sb_tensor tDX = e->view(dx, L.at("X"), "BJI");

  {
    // LayerNorm-2 backward: one fused pass when every view is feature-innermost, else the two separate operators
    sb_tensor ln = v("LN2"), gamma = pv("S2"), dln = v("DLN2"), dg = dv("S2"), db = dv("B2");
    sb_tensor istd = v("LN2STD"), diff = v("LN2DIFF"), mask = v("DROP3MASK"), dres = v("DRESID2"), dlin = v("DLIN2");
    e->mark(s, "bsb+blnrd1");
    int st = e->fuse ? sb_backward_scale_bias_layernorm(stream, ws, &tDY, &ln, &gamma, &istd, &diff, &mask,
                                                         e->dead_stores ? &dln : nullptr, &dres, &dlin, &dg, &db)
                     : SB_ERR_UNSUPPORTED;
    if (st == SB_ERR_UNSUPPORTED) {
      e->relabel("bsb");
      SB_TRY(sb_backward_scale_bias(stream, ws, &tDY, &ln, &gamma, &dln, &dg, &db));
      e->mark(s, "blnrd1");
      SB_TRY(sb_backward_layernorm_residual_dropout(stream, &dln, &istd, &diff, &mask, &dres, &dlin));
    } else if (st != SB_OK) {
      return st;
    }
  }
  SB_TRY(einsum(e, s, "dXlin2", L.at("DLIN2"), T["DLIN2"], L.at("LINW2"), T["LINW2"], L.at("DDROP2"),
                T["DDROP2"], 1.f));
  SB_TRY(einsum(e, s, "dWlin2", L.at("DLIN2"), T["DLIN2"], L.at("DROP2"), T["DROP2"], L.at("LINW2"),
                D.at("LINW2"), 1.f));
  {
    e->mark(s, "bdrlb");
    sb_tensor g = v("DDROP2"), mask = v("DROP2MASK"), lin1 = v("LIN1"), o = v("DLIN1"), db = dv("LINB1");
    SB_TRY(sb_backward_dropout_activation_bias(stream, ws, &g, &mask, &lin1, &o, &db, e->activation));
  }
  SB_TRY(einsum(e, s, "dXlin1", L.at("DLIN1"), T["DLIN1"], L.at("LINW1"), T["LINW1"], L.at("DLIN1_LINW1"),
                T["DLIN1_LINW1"], 1.f));
  SB_TRY(einsum(e, s, "dWlin1", L.at("DLIN1"), T["DLIN1"], L.at("SB1"), T["SB1"], L.at("LINW1"),
                D.at("LINW1"), 1.f));
  {
    sb_tensor ln1 = v("LN1"), gamma = pv("S1"), dres2 = v("DRESID2"), dlw = v("DLIN1_LINW1"), dlin2 = v("DLIN2");
    sb_tensor dln1 = v("DLN1"), dg = dv("S1"), db = dv("B1"), dlb2 = dv("LINB2"), dbo = dv("BO");
    sb_tensor istd = v("LN1STD"), diff = v("LN1DIFF"), mask = v("DROP1MASK"), dres1 = v("DRESID1"), datt = v("DATT");
    e->mark(s, "ebsb+blnrd2+baob");
    int st = e->fuse ? sb_extended_backward_scale_bias_layernorm(stream, ws, &ln1, &gamma, &dres2, &dlw, &dlin2, &istd,
                                                                  &diff, &mask, e->dead_stores ? &dln1 : nullptr, &dres1,
                                                                  &datt, &dg, &db, &dlb2, &dbo)
                     : SB_ERR_UNSUPPORTED;
    if (st == SB_ERR_UNSUPPORTED) {
      e->relabel("ebsb");
      SB_TRY(sb_extended_backward_scale_bias(stream, ws, &ln1, &gamma, &dres2, &dlw, &dlin2, &dln1, &dg, &db, &dlb2));
      e->mark(s, "blnrd2");
      SB_TRY(sb_backward_layernorm_residual_dropout(stream, &dln1, &istd, &diff, &mask, &dres1, &datt));
      e->mark(s, "baob");
      SB_TRY(sb_backward_attn_out_bias(stream, ws, &datt, &dbo));
    } else if (st != SB_OK) {
      return st;
    }
  }
  if (e->ffn_grads_event) {
    // Everything the feed-forward half and both LayerNorms contribute to the parameter gradients (LINW1, LINB1,
    // LINW2, LINB2, S1, B1, S2, B2, BO) is final here: a data-parallel caller can start summing those while the
    // attention half of the backward pass still runs.  Inside a stream capture the record becomes an
    // event-record node that code outside the graph may wait for.
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    SB_CUDA_OK(cudaStreamIsCapturing(s, &cap));
    SB_CUDA_OK(cudaEventRecordWithFlags(e->ffn_grads_event, s,
                                        cap == cudaStreamCaptureStatusActive ? cudaEventRecordExternal : cudaEventRecordDefault));
  }
  SB_TRY(einsum(e, s, "dWout", L.at("GAMMA"), T["GAMMA"], L.at("DATT"), T["DATT"], L.at("WO"), D.at("WO"), 1.f));
  SB_TRY(einsum(e, s, "dXout", L.at("WO"), T["WO"], L.at("DATT"), T["DATT"], L.at("DGAMMA"), T["DGAMMA"], 1.f));
  const float scale = 1.f / std::sqrt((float)e->P);
  void *KK = q_slice(T["KKQQVV"], 0), *QQ = q_slice(T["KKQQVV"], 1), *VV = q_slice(T["KKQQVV"], 2);
  void *DKK = q_slice(T["DKKQQVV"], 0), *DQQ = q_slice(T["DKKQQVV"], 1), *DVV = q_slice(T["DKKQQVV"], 2);
  {
    sb_tensor alpha = v("ALPHA"), mask = v("ATTN_DROP_MASK"), g = v("DATTN_DROP"), o = v("DBETA");
    int st = SB_ERR_UNSUPPORTED;
    if (e->fuse) {
      e->mark(s, "dX1gamma+bs");
      sb_tensor dgm = e->view(T["DGAMMA"], "DGAMMA"), vvt = e->view(VV, lKK, "PHBJ");
      st = sb_attention_scores_softmax_backward(stream, &dgm, &vvt, &alpha, &mask, e->dead_stores ? &g : nullptr, &o);
      if (st != SB_OK && st != SB_ERR_UNSUPPORTED) return st;
      if (st == SB_ERR_UNSUPPORTED) e->unmark();
    }
    if (st == SB_ERR_UNSUPPORTED)
      SB_TRY(einsum(e, s, "dX1gamma", rename(lKK, 'J', 'K'), VV, L.at("DGAMMA"), T["DGAMMA"], L.at("DATTN_DROP"),
                    T["DATTN_DROP"], 1.f));
    {
      int st2 = SB_ERR_UNSUPPORTED;
      if (e->fuse) {
        e->mark(s, "dX2gamma");
        sb_tensor sc = e->view(T["ATTN_DROP"], "ATTN_DROP"), dgm = e->view(T["DGAMMA"], "DGAMMA");
        sb_tensor dvv = e->view(DVV, lDKK, "PHBJ");
        st2 = sb_attention_score_contractions(stream, &sc, nullptr, nullptr, &dgm, &dvv, 1.f);
        if (st2 != SB_OK && st2 != SB_ERR_UNSUPPORTED) return st2;
        if (st2 == SB_ERR_UNSUPPORTED) e->unmark();
      }
      if (st2 == SB_ERR_UNSUPPORTED)
        SB_TRY(einsum(e, s, "dX2gamma", L.at("DGAMMA"), T["DGAMMA"], L.at("ATTN_DROP"), T["ATTN_DROP"],
                      rename(lDKK, 'J', 'K'), DVV, 1.f));
    }
    if (st == SB_ERR_UNSUPPORTED) {
      e->mark(s, "bs");
      SB_TRY(sb_backward_softmax(stream, &alpha, &mask, &g, &o));
    }
  }
  {
    // both projection gradients from one pass over DBETA
    int st = SB_ERR_UNSUPPORTED;
    if (e->fuse) {
      e->mark(s, "dX1QKT+dX2QKT");
      sb_tensor sc = e->view(T["DBETA"], "DBETA"), kk = e->view(KK, lKK, "PHBJ"), qq = e->view(QQ, lKK, "PHBJ");
      sb_tensor dqq = e->view(DQQ, lDKK, "PHBJ"), dkk = e->view(DKK, lDKK, "PHBJ");
      st = sb_attention_score_contractions(stream, &sc, &kk, &dqq, &qq, &dkk, scale);
      if (st != SB_OK && st != SB_ERR_UNSUPPORTED) return st;
      if (st == SB_ERR_UNSUPPORTED) e->unmark();
    }
    if (st == SB_ERR_UNSUPPORTED) {
      SB_TRY(einsum(e, s, "dX1QKT", rename(lKK, 'J', 'K'), KK, L.at("DBETA"), T["DBETA"], lDKK, DQQ, scale));
      SB_TRY(einsum(e, s, "dX2QKT", lKK, QQ, L.at("DBETA"), T["DBETA"], rename(lDKK, 'J', 'K'), DKK, scale));
    }
  }
  // the encoder-input gradient (DXATT + DRESID1) rides on the epilogue of the contraction that produces DXATT
  int st_bei = SB_ERR_UNSUPPORTED;
  if (e->fuse && L.at("DXATT") == L.at("DRESID1") && L.at("DXATT") == L.at("X")) {
    const sb_tensor resid = e->mem(T["DRESID1"], L.at("DRESID1")), out2 = e->mem(dx, L.at("X"));
    sb_epilogue ep{};
    ep.kind = SB_EPI_RESIDUAL;
    ep.resid = &resid;
    ep.out2 = &out2;
    ep.discard_c = e->dead_stores ? 0 : 1;   // DXATT: only the encoder-input sum reads it
    st_bei = einsum_fused(e, s, "dXQKV-fused+bei", L.at("WKQV"), T["WKQV"], L.at("DKKQQVV"), T["DKKQQVV"], L.at("DXATT"),
                          T["DXATT"], 1.f, &ep);
    if (st_bei != SB_OK && st_bei != SB_ERR_UNSUPPORTED) return st_bei;
  }
  if (st_bei == SB_ERR_UNSUPPORTED)
    SB_TRY(einsum(e, s, "dXQKV-fused", L.at("WKQV"), T["WKQV"], L.at("DKKQQVV"), T["DKKQQVV"], L.at("DXATT"),
                  T["DXATT"], 1.f));
  SB_TRY(einsum(e, s, "dWQKV-fused", L.at("X"), T["X"], L.at("DKKQQVV"), T["DKKQQVV"], L.at("WKQV"),
                D.at("WKQV"), 1.f));
  {
    e->mark(s, "baib");
    sb_tensor d = v("DKKQQVV"), db = dv("BKQV");
    SB_TRY(sb_backward_attention_input_biases(stream, &d, &db));
  }
  if (st_bei == SB_ERR_UNSUPPORTED) {
    e->mark(s, "bei");
    sb_tensor a = v("DXATT"), b = v("DRESID1");
    SB_TRY(sb_backward_encoder_input(stream, &a, &b, &tDX));
  }
  if (e->timing) { e->mark(s, ""); --e->launches; }
  e->kernels_bwd = g_kernel_launches - e->kernel_base;
  return SB_OK;
}

// ---- whole-pass CUDA graphs ---------------------------------------------------------------
namespace {

bool graphs_allowed(const sb_encoder* e) {
  static const bool env_on = [] {
    const char* v = getenv("SUBSTATION_B200_GRAPHS");
    return !(v && v[0] == '0');
  }();
  return env_on && e->graphs && !e->timing;
}

// Runs `pass(stream)` eagerly, or replays / captures it as a graph when its arguments repeat.
// `counted(launches, kernels)` restores the handle's counters on a replay.
template <class Pass>
int run_pass(sb_encoder* e, sb_encoder::GraphCache& cache, std::vector<uint64_t>&& key, cudaStream_t s, int* launches,
             long long* kernels, Pass&& pass) {
  cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
  if (!graphs_allowed(e) || cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return pass(s);
  }
  ++cache.tick;
  for (auto& g : cache.entries)
    if (g.key == key) {
      g.last_use = cache.tick;
      ++cache.replays;
      SB_CUDA_OK(cudaGraphLaunch(g.exec, s));
      *launches = g.launches;
      *kernels = g.kernels;
      return SB_OK;
    }
  bool seen_before = false;
  for (size_t i = 0; i < cache.seen.size(); ++i)
    if (cache.seen[i] == key) {
      seen_before = true;
      cache.seen.erase(cache.seen.begin() + i);
      break;
    }
  if (!seen_before) {  // first sighting: run it as it is and remember the arguments
    if (cache.seen.size() >= 32) cache.seen.erase(cache.seen.begin());
    cache.seen.push_back(key);
    return pass(s);
  }
  // second sighting: capture on the private stream, then launch the graph on the caller's stream
  if (!e->capture_stream && cudaStreamCreateWithFlags(&e->capture_stream, cudaStreamNonBlocking) != cudaSuccess) {
    cudaGetLastError();
    e->graphs = false;
    return pass(s);
  }
  if (cudaStreamBeginCapture(e->capture_stream, cudaStreamCaptureModeRelaxed) != cudaSuccess) {
    cudaGetLastError();
    e->graphs = false;
    return pass(s);
  }
  const int st = pass(e->capture_stream);
  cudaGraph_t graph = nullptr;
  const cudaError_t ce = cudaStreamEndCapture(e->capture_stream, &graph);
  cudaGraphExec_t exec = nullptr;
  if (st != SB_OK || ce != cudaSuccess || !graph || cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) {
    // nothing has run yet (the launches only went into the capture): this handle goes back to plain
    // launches for good, and a real error shows again in the eager pass
    cudaGetLastError();
    if (graph) cudaGraphDestroy(graph);
    e->graphs = false;
    return pass(s);
  }
  cudaGraphDestroy(graph);
  static const size_t max_graphs = [] {
    const char* v = getenv("SUBSTATION_B200_GRAPH_CACHE");
    const int n = v ? atoi(v) : 0;
    return (size_t)(n > 0 ? n : 16);
  }();
  if (cache.entries.size() >= max_graphs) {  // drop the least recently used
    size_t victim = 0;
    for (size_t i = 1; i < cache.entries.size(); ++i)
      if (cache.entries[i].last_use < cache.entries[victim].last_use) victim = i;
    cudaGraphExecDestroy(cache.entries[victim].exec);
    cache.entries.erase(cache.entries.begin() + victim);
  }
  sb_encoder::PassGraph g;
  g.key = std::move(key);
  g.exec = exec;
  g.launches = *launches;
  g.kernels = *kernels;
  g.last_use = cache.tick;
  cache.entries.push_back(std::move(g));
  ++cache.captures;
  SB_CUDA_OK(cudaGraphLaunch(exec, s));
  return SB_OK;
}

}  // namespace

extern "C" int sb_encoder_forward(sb_encoder* e, void* stream, const void* x, const void* const* params,
                                  void* const* fwd, void* y, int mask_mode, uint64_t seed, uint64_t offset) {
  if (!e || !y || !params || !fwd) return fail(SB_ERR_ARG, "sb_encoder_forward: null argument");
  auto pass = [&](cudaStream_t s) { return forward_pass(e, (void*)s, x, params, fwd, y, mask_mode, seed, offset); };
  // in-kernel masks take a new offset every call, so only explicit-mask passes repeat
  if (mask_mode != SB_MASK_EXPLICIT) return pass((cudaStream_t)stream);
  std::vector<uint64_t> key{(uint64_t)(uintptr_t)x, (uint64_t)(uintptr_t)y, (uint64_t)e->fuse | ((uint64_t)e->dead_stores << 1),
                            (uint64_t)gemm_sm_budget()};
  for (size_t i = 0; i < e->param_order.size(); ++i) key.push_back((uint64_t)(uintptr_t)params[i]);
  for (size_t i = 0; i < e->fwd_order.size(); ++i) key.push_back((uint64_t)(uintptr_t)fwd[i]);
  return run_pass(e, e->graph_fwd, std::move(key), (cudaStream_t)stream, &e->launches, &e->kernels_fwd, pass);
}

extern "C" int sb_encoder_backward(sb_encoder* e, void* stream, const void* dy, void* const* dparams,
                                   void* const* bwd, const void* const* params, void* const* fwd,
                                   const void* x, void* dx) {
  if (!e || !dy || !dparams || !bwd || !dx || !params || !fwd)
    return fail(SB_ERR_ARG, "sb_encoder_backward: null argument");
  auto pass = [&](cudaStream_t s) { return backward_pass(e, (void*)s, dy, dparams, bwd, params, fwd, x, dx); };
  std::vector<uint64_t> key{(uint64_t)(uintptr_t)dy, (uint64_t)(uintptr_t)x, (uint64_t)(uintptr_t)dx, (uint64_t)e->fuse | ((uint64_t)e->dead_stores << 1),
                            (uint64_t)gemm_sm_budget()};
  for (size_t i = 0; i < e->param_order.size(); ++i) {
    key.push_back((uint64_t)(uintptr_t)dparams[i]);
    key.push_back((uint64_t)(uintptr_t)params[i]);
  }
  for (size_t i = 0; i < e->bwd_order.size(); ++i) key.push_back((uint64_t)(uintptr_t)bwd[i]);
  for (size_t i = 0; i < e->fwd_order.size(); ++i) key.push_back((uint64_t)(uintptr_t)fwd[i]);
  return run_pass(e, e->graph_bwd, std::move(key), (cudaStream_t)stream, &e->launches, &e->kernels_bwd, pass);
}

