// The operators that only training graphs contain (appended by graph_autodiff.cpp): their checks, scratch sizes, host
// implementations (reference semantics, used on device -1 and by the CPU tests) and, at the end of the file, the dispatch
// to the sm_100a kernels.
//
//   fill            out = value
//   cast            out = scale * in, between bf16 and fp32 in either direction
//   copy accumulate=1   out[view] += in[view] (the backward of every view copy; bf16 or fp32 on either side)
//   column_sum      out[c] += sum over rows of in[r, c]              (fp32 out; bias gradients)
//   unary_bwd       dx = dy * fn'(x)
//   layer_norm_bwd  (dy, x, gamma, stats [, add_to_dx]) -> dx [, dgamma, dbeta]   (fp32 parameter gradients, added when
//                   accumulate=1; add_to_dx is the residual branch's gradient, added while dx is written)
//   softmax_bwd     (y, dy) -> dx = scale * y * (dy - sum(dy * y))
//   attention_bwd   (q, k, v, o, do, lse) -> dq, dk, dv, each written through a token stride
//   embedding_bwd   (ids, dy) -> table gradient (fp32, scatter-add)
//   cross_entropy   (logits, targets) -> mean loss [, d loss / d logits]
//   mse             (a, b) -> mean squared difference
//   dropout         y = x * keep / (1 - p); the mask is a function of (seed, call number, operator index, element), so the
//                   backward operator is the same operator applied to the gradient and nothing is stored
//   grad_clip       gradients -> {sum of squares, non-finite count, clip factor, global norm}
//   adamw_update / sgd_update   gradients [, clip] -> parameters (bf16), fp32 master weights and optimizer state, in place
// Operators marked when=first / when=last run only on the first / last micro-batch of an optimizer step (gradient accumulation).
//
// Reference counterparts: oneflow/user/kernels/{layer_norm_gpu_kernel.cu, softmax_kernel.cpp, sparse_softmax_cross_entropy_kernel.cu,
// unsorted_segment_sum_kernel.cpp, reduce_kernel.cpp, model_update_kernels.cpp}, oneflow/user/ops/*_grad*.
#include <cmath>
#include <cstring>
#include <stdexcept>

#include "../common/dropout_hash.h"
#include "../kernels/ofb_kernels.h"
#include "graph_impl.h"

extern "C" {
int ofb_graph_unary_bwd(const void* x, const void* dy, void* dx, long long n, int fn, float alpha, void* stream);
int ofb_graph_strided_acc(const void* x, int x_dtype, void* y, int y_dtype, int ndim, const long long* shape, const long long* in_strides,
                          long long in_offset, const long long* out_strides, long long out_offset, void* stream);
int ofb_graph_dropout(const void* x, void* y, long long n, unsigned long long seed, const unsigned long long* counter, unsigned int op_index,
                      float p, void* stream);
int ofb_graph_mse_parts(void);
int ofb_graph_mse(const void* a, const void* b, float* loss, float* scratch, long long n, void* stream);
int ofb_graph_sum_f32(const float* x, float* out, long long n, float scale, void* stream);
int ofb_cast_scale(const void* x, int in_dtype, void* y, int out_dtype, long long n, float scale, const float* scale_by_tensor, void* stream);
int ofb_column_sum(const void* x, float* out, int rows, int cols, void* stream);
int ofb_layer_norm_bwd_parts(int rows);
int ofb_layer_norm_bwd(const void* dy, const void* x, const void* gamma, const float* mean, const float* rstd, const void* add_to_dx, void* dx,
                       float* dgamma, float* dbeta, float* scratch, int accumulate_param_grads, int rows, int cols, void* stream);
int ofb_softmax_bwd(const void* softmax_y, const void* dy, const void* dropout_mask, void* dx, long long rows, int cols, int tril, int tril_rows,
                    int diagonal, float scale, float out_scale, void* stream);
long long ofb_fmha_bwd_scratch_floats(int B, int S, int H, int D);
int ofb_fmha_bwd_ex(const void* q, const void* k, const void* v, long long q_row_stride, long long kv_row_stride, const void* o, const void* d_o,
                    const float* lse, void* dq, void* dk, void* dv, long long dq_row_stride, long long dkv_row_stride, float* scratch,
                    const int* kv_len, int B, int Sq, int Sk, int H, int Hk, int D, int causal, float scale, float p_dropout,
                    unsigned long long seed, unsigned int offset, void* stream);
int ofb_embedding_bwd(const long long* ids, const void* dout, float* dwte, float* dwpe, long long tokens, int seq, int hidden, long long vocab_start,
                      long long vocab_rows, int pos_offset, void* stream);
int ofb_xent_stats(const void* logits, const long long* labels, float* stats, int rows, int cols, long long ld, int vocab_start, void* stream);
int ofb_xent_grad(const void* logits, const long long* labels, const float* merged, float* loss, void* dlogits, int rows, int cols, long long ld,
                  int vocab_start, float grad_scale, long long ignore_index, void* stream);
int ofb_multi_tensor_adamw(int n, void* const* grads, float* const* masters, void* const* copies, float* const* ms, float* const* vs,
                           const long long* sizes, int grad_is_bf16, float lr, float beta1, float beta2, float eps, float weight_decay, float l2,
                           float scale, float bc1, float bc2, const float* lr_ptr, const float* scale_ptr, const long long* skip_if, void* stream);
int ofb_multi_tensor_adamw_dev(int n, void* const* grads, float* const* masters, void* const* copies, float* const* ms, float* const* vs,
                               const long long* sizes, int grad_is_bf16, float beta1, float beta2, float eps, float weight_decay, const float* step,
                               const float* scale_ptr, void* stream);
int ofb_sqsum_scratch_floats(void);
int ofb_multi_tensor_sqsum(int n, void* const* grads, const long long* sizes, int grad_is_bf16, float* scratch, float* out, int accumulate, void* stream);
int ofb_clip_factor(const float* sq_and_bad, float max_norm, float* factor, long long* found_inf, float* total_norm, void* stream);
int ofb_multi_tensor_sgd(int n, void* const* grads, float* const* masters, void* const* copies, float* const* ms, const long long* sizes,
                         int grad_is_bf16, float lr, float momentum, float dampening, int nesterov, int maximize, float weight_decay, float l1,
                         float l2, float scale, const float* lr_ptr, const float* scale_ptr, const long long* skip_if, void* stream);
}

namespace oneflow_api {

namespace {

inline float ld(const void* p, DType dt, int64_t i) {
  return dt == DType::kFloat ? static_cast<const float*>(p)[i] : from_bf16(static_cast<const uint16_t*>(p)[i]);
}
inline void st(void* p, DType dt, int64_t i, float v) {
  if (dt == DType::kFloat) static_cast<float*>(p)[i] = v;
  else static_cast<uint16_t*>(p)[i] = to_bf16(v);
}
inline float ldb(const void* p, int64_t i) { return from_bf16(static_cast<const uint16_t*>(p)[i]); }
inline void stb(void* p, int64_t i, float v) { static_cast<uint16_t*>(p)[i] = to_bf16(v); }

}  // namespace

float host_unary_grad(float x, int fn, float alpha) {
  switch (fn) {
    case 0: return alpha;
    case 1: return 0.5f * (1.f + std::erf(x * 0.7071067811865476f)) + x * 0.3989422804014327f * std::exp(-0.5f * x * x);
    case 2: {
      const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x), t = std::tanh(u);
      return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * 0.7978845608028654f * (1.f + 3.f * 0.044715f * x * x);
    }
    case 3: return x > 0.f ? 1.f : 0.f;
    case 4: {
      const float t = std::tanh(x);
      return 1.f - t * t;
    }
    case 5: {
      const float s = 1.f / (1.f + std::exp(-x));
      return s * (1.f - s);
    }
    case 6: {
      const float s = 1.f / (1.f + std::exp(-x));
      return s * (1.f + x * (1.f - s));
    }
    case 7: return 1.f;
    case 8: return std::exp(x);
    case 9: return -0.5f / (std::sqrt(x) * x);
    case 10: return 2.f * x;
    default: return 1.f;
  }
}

namespace {

inline float unary_grad(float x, int fn, float alpha) { return host_unary_grad(x, fn, alpha); }

bool is_float_type(DType d) { return d == DType::kBFloat16 || d == DType::kFloat; }

}  // namespace

// ------------------------------------------------------------------------------------------------ checks and scratch
bool check_train_op(const OpDef& op, const IR& ir, const Plan& plan) {
  auto need = [&](bool c, const std::string& why) {
    if (!c) throw std::runtime_error("operator " + op.type + ": " + why);
  };
  auto shp = [&](int t) -> const std::vector<int64_t>& { return plan.shape[static_cast<size_t>(t)]; };
  auto dt = [&](int t) { return ir.tensors[static_cast<size_t>(t)].dtype; };
  auto n = [&](int t) { return numel(shp(t)); };
  for (int t : op.in) need(t >= 0, "absent input");
  auto bf16 = [&](std::initializer_list<int> ts) {
    for (int x : ts)
      if (dt(x) != DType::kBFloat16) return false;
    return true;
  };
  auto strided_view_fits = [&](int x, int64_t rows, int64_t row_elems, int64_t stride) {
    if (stride < row_elems || rows <= 0 || stride > (int64_t{1} << 40)) return false;
    const int r = plan.root[static_cast<size_t>(x)];
    const int64_t first = plan.byte_off[static_cast<size_t>(x)] / SizeOf(dt(x));
    return first + (rows - 1) * stride + row_elems <= numel(shp(r));
  };
  const std::string& t = op.type;
  if (t == "fill") {
    need(op.in.empty() && op.out.size() == 1 && is_float_type(dt(op.out[0])), "one bf16 / fp32 output, no input");
  } else if (t == "cast") {
    need(op.in.size() == 1 && op.out.size() == 1 && n(op.in[0]) == n(op.out[0]) && is_float_type(dt(op.in[0])) && is_float_type(dt(op.out[0])),
         "one input and one output of the same length, bf16 or fp32");
  } else if (t == "column_sum") {
    need(op.in.size() == 1 && shp(op.in[0]).size() == 2 && dt(op.in[0]) == DType::kBFloat16, "a [rows, cols] bf16 input");
    need(dt(op.out[0]) == DType::kFloat && n(op.out[0]) == shp(op.in[0])[1], "an fp32 output with one element per column");
  } else if (t == "dropout") {
    need(op.in.size() == 1 && op.out.size() == 1 && n(op.in[0]) == n(op.out[0]) && dt(op.in[0]) == DType::kBFloat16 && dt(op.out[0]) == DType::kBFloat16,
         "one bf16 input and output of the same length");
    need(attr_float(op, "p", 0.5) >= 0.0 && attr_float(op, "p", 0.5) < 1.0, "p must be in [0, 1)");
  } else if (t == "unary_bwd") {
    need(op.in.size() == 2 && op.out.size() == 1 && n(op.in[0]) == n(op.in[1]) && n(op.in[0]) == n(op.out[0]) && bf16({op.in[0], op.in[1], op.out[0]}),
         "bf16 x, dy and dx of the same length");
  } else if (t == "layer_norm_bwd") {
    need((op.in.size() == 4 || op.in.size() == 5) && (op.out.size() == 1 || op.out.size() == 3), "(dy, x, gamma, stats [, add_to_dx]) -> dx [, dgamma, dbeta]");
    if (op.in.size() == 5) need(n(op.in[4]) == n(op.in[1]) && dt(op.in[4]) == DType::kBFloat16, "the tensor added to dx must match x");
    const int64_t cols = shp(op.in[1]).back(), rows = n(op.in[1]) / cols;
    need(n(op.in[0]) == n(op.in[1]) && n(op.out[0]) == n(op.in[1]) && n(op.in[2]) == cols && n(op.in[3]) == 2 * rows && dt(op.in[3]) == DType::kFloat &&
             bf16({op.in[0], op.in[1], op.in[2], op.out[0]}),
         "shape or dtype mismatch");
    if (op.out.size() == 3) need(n(op.out[1]) == cols && n(op.out[2]) == cols && dt(op.out[1]) == DType::kFloat && dt(op.out[2]) == DType::kFloat, "fp32 parameter gradients with one element per column");
  } else if (t == "softmax_bwd") {
    need(op.in.size() == 2 && op.out.size() == 1 && n(op.in[0]) == n(op.in[1]) && n(op.in[0]) == n(op.out[0]) && bf16({op.in[0], op.in[1], op.out[0]}) &&
             !shp(op.in[0]).empty() && shp(op.in[0]).back() > 0,
         "bf16 y, dy and dx of the same length");
  } else if (t == "attention_bwd") {
    need(op.in.size() == 6 && op.out.size() == 3, "(q, k, v, o, do, lse) -> dq, dk, dv");
    const auto& q = shp(op.in[0]);
    const auto& k = shp(op.in[1]);
    need(q.size() == 4 && k.size() == 4 && shp(op.in[2]) == k && q[0] == k[0] && q[3] == k[3] && q[2] % k[2] == 0, "q [B,Sq,H,D], k / v [B,Sk,Hk,D]");
    need(n(op.in[3]) == numel(q) && n(op.in[4]) == numel(q) && n(op.in[5]) == q[0] * q[1] * q[2] && dt(op.in[5]) == DType::kFloat, "o / do / lse sizes");
    need(n(op.out[0]) == numel(q) && n(op.out[1]) == numel(k) && n(op.out[2]) == numel(k), "gradient sizes");
    need(bf16({op.in[0], op.in[1], op.in[2], op.in[3], op.in[4], op.out[0], op.out[1], op.out[2]}), "bf16 operands");
    const int64_t qr = q[0] * q[1], kr = k[0] * k[1], qe = q[2] * q[3], ke = k[2] * k[3];
    need(strided_view_fits(op.in[0], qr, qe, attr_int(op, "q_stride", qe)) && strided_view_fits(op.in[1], kr, ke, attr_int(op, "kv_stride", ke)) &&
             strided_view_fits(op.in[2], kr, ke, attr_int(op, "kv_stride", ke)) && strided_view_fits(op.out[0], qr, qe, attr_int(op, "dq_stride", qe)) &&
             strided_view_fits(op.out[1], kr, ke, attr_int(op, "dkv_stride", ke)) && strided_view_fits(op.out[2], kr, ke, attr_int(op, "dkv_stride", ke)),
         "a token stride reaches outside its storage");
  } else if (t == "embedding_bwd") {
    need(op.in.size() == 2 && dt(op.in[0]) == DType::kInt64 && shp(op.in[1]).size() == 2 && shp(op.in[1])[0] == n(op.in[0]), "ids and a [ids, cols] gradient");
    need(op.out.size() == 1 && dt(op.out[0]) == DType::kFloat && shp(op.out[0]).size() == 2 && shp(op.out[0])[1] == shp(op.in[1])[1] && bf16({op.in[1]}),
         "a bf16 gradient and an fp32 [rows, cols] table gradient");
  } else if (t == "cross_entropy") {
    need(op.in.size() == 2 && shp(op.in[0]).size() >= 2 && dt(op.in[0]) == DType::kBFloat16 && dt(op.in[1]) == DType::kInt64, "bf16 logits [.., classes] and int64 targets");
    need(n(op.in[1]) * shp(op.in[0]).back() == n(op.in[0]), "one target per row of logits");
    need(dt(op.out[0]) == DType::kFloat && n(op.out[0]) == 1, "a scalar fp32 loss");
    if (op.out.size() > 1) need(n(op.out[1]) == n(op.in[0]) && dt(op.out[1]) == DType::kBFloat16, "the logits gradient must match the logits");
  } else if (t == "mse") {
    need(op.in.size() == 2 && n(op.in[0]) == n(op.in[1]) && dt(op.in[0]) == DType::kBFloat16 && dt(op.in[1]) == DType::kBFloat16, "two bf16 inputs of the same length");
    need(dt(op.out[0]) == DType::kFloat && n(op.out[0]) == 1, "a scalar fp32 loss");
  } else if (t == "grad_clip") {
    need(!op.in.empty() && op.out.size() == 1 && n(op.out[0]) == 4 && dt(op.out[0]) == DType::kFloat, "gradients -> four fp32 values");
    for (int g : op.in) need(dt(g) == DType::kFloat, "fp32 gradients");
  } else if (t == "adamw_update" || t == "sgd_update") {
    const int64_t np = attr_int(op, "n", 0), states = attr_int(op, "states", 0), clip = attr_int(op, "clip", 0);
    need(np > 0 && static_cast<int64_t>(op.in.size()) == np + clip && static_cast<int64_t>(op.out.size()) == np * (2 + states), "n gradients [+ clip] -> n parameters, n master copies, n * states state tensors");
    if (clip) need(n(op.in[static_cast<size_t>(np)]) == 4 && dt(op.in[static_cast<size_t>(np)]) == DType::kFloat, "the clip record is four fp32 values");
    need(t == "adamw_update" ? states == 2 : states <= 1, "state tensors per parameter");
    for (int64_t i = 0; i < np; ++i) {
      const int64_t len = n(op.in[static_cast<size_t>(i)]);
      need(dt(op.in[static_cast<size_t>(i)]) == DType::kFloat && dt(op.out[static_cast<size_t>(i)]) == DType::kBFloat16, "fp32 gradients, bf16 parameters");
      for (int64_t s = 0; s < 2 + states; ++s) need(n(op.out[static_cast<size_t>(s * np + i)]) == len, "lengths differ");
      for (int64_t s = 1; s < 2 + states; ++s) need(dt(op.out[static_cast<size_t>(s * np + i)]) == DType::kFloat, "fp32 master weights and state");
    }
  } else {
    return false;
  }
  return true;
}

int64_t train_workspace_for(const OpDef& op, const Plan& plan) {
  auto shp = [&](int t) -> const std::vector<int64_t>& { return plan.shape[static_cast<size_t>(t)]; };
  if (op.type == "layer_norm_bwd") {
    const int64_t cols = shp(op.in[1]).back(), rows = numel(shp(op.in[1])) / cols;
    return 2 * static_cast<int64_t>(ofb_layer_norm_bwd_parts(static_cast<int>(rows))) * cols * 4;
  }
  if (op.type == "attention_bwd") {
    const auto& q = shp(op.in[0]);
    return ofb_fmha_bwd_scratch_floats(static_cast<int>(q[0]), static_cast<int>(q[1]), static_cast<int>(q[2]), static_cast<int>(q[3])) * 4;
  }
  if (op.type == "cross_entropy") {
    const int64_t rows = numel(shp(op.in[1]));
    // [rows, 3] statistics + [rows] losses (+ a throw-away gradient when nobody asked for one)
    return rows * 16 + (op.out.size() > 1 ? 0 : numel(shp(op.in[0])) * 2);
  }
  if (op.type == "mse") return static_cast<int64_t>(ofb_graph_mse_parts()) * 4;
  if (op.type == "grad_clip") return static_cast<int64_t>(ofb_sqsum_scratch_floats()) * 4;
  return 0;
}

// ------------------------------------------------------------------------------------------------ host
bool Graph::Impl::run_train_op_host(const PlannedOp& p) {
  const OpDef& op = *p.def;
  auto shp = [&](int t) -> const std::vector<int64_t>& { return plan->shape[static_cast<size_t>(t)]; };
  auto dt = [&](int t) { return ir.tensors[static_cast<size_t>(t)].dtype; };
  auto n = [&](int t) { return numel(shp(t)); };
  const std::string& t = op.type;
  if (t == "fill") {
    const float v = static_cast<float>(attr_float(op, "value", 0.0));
    void* y = addr(op.out[0]);
    for (int64_t i = 0; i < n(op.out[0]); ++i) st(y, dt(op.out[0]), i, v);
  } else if (t == "cast") {
    const float scale = static_cast<float>(attr_float(op, "scale", 1.0));
    const void* x = addr(op.in[0]);
    void* y = addr(op.out[0]);
    for (int64_t i = 0; i < n(op.in[0]); ++i) st(y, dt(op.out[0]), i, ld(x, dt(op.in[0]), i) * scale);
  } else if (t == "copy") {
    if (attr_int(op, "accumulate", 0) == 0) return false;
    const auto sh = int_list(attr_str(op, "shape", "")), is = int_list(attr_str(op, "in_strides", "")), os = int_list(attr_str(op, "out_strides", ""));
    const void* x = addr(op.in[0]);
    void* y = addr(op.out[0]);
    const int64_t total = numel(sh), io = attr_int(op, "in_offset", 0), oo = attr_int(op, "out_offset", 0);
    for (int64_t i = 0; i < total; ++i) {
      int64_t r = i, in = io, out = oo;
      for (int d = static_cast<int>(sh.size()) - 1; d >= 0; --d) {
        const int64_t c = r % sh[static_cast<size_t>(d)];
        r /= sh[static_cast<size_t>(d)];
        in += c * is[static_cast<size_t>(d)];
        out += c * os[static_cast<size_t>(d)];
      }
      st(y, dt(op.out[0]), out, ld(y, dt(op.out[0]), out) + ld(x, dt(op.in[0]), in));
    }
  } else if (t == "column_sum") {
    const int64_t rows = shp(op.in[0])[0], cols = shp(op.in[0])[1];
    const void* x = addr(op.in[0]);
    float* y = static_cast<float*>(addr(op.out[0]));
    for (int64_t c = 0; c < cols; ++c) {
      float acc = 0.f;
      for (int64_t r = 0; r < rows; ++r) acc += ldb(x, r * cols + c);
      y[c] += acc;
    }
  } else if (t == "dropout" && (!ir.training || call_kind == 4)) {
    std::memcpy(addr(op.out[0]), addr(op.in[0]), static_cast<size_t>(n(op.in[0]) * 2));   // evaluation: the identity
  } else if (t == "dropout") {
    const float p = static_cast<float>(attr_float(op, "p", 0.5)), scale = 1.f / (1.f - p);
    const uint64_t base = ofb::dropout_base(train.seed, call_counter, static_cast<uint32_t>(attr_int(op, "index", 0)));
    const uint32_t thr = ofb::dropout_threshold(p);
    const void* x = addr(op.in[0]);
    void* y = addr(op.out[0]);
    for (int64_t i = 0; i < n(op.in[0]); ++i) {
      const bool keep = ofb::dropout_keep(ofb::dropout_draw(base, static_cast<uint64_t>(i >> 2)), static_cast<int>(i & 3), thr);
      stb(y, i, keep ? ldb(x, i) * scale : 0.f);
    }
  } else if (t == "unary_bwd") {
    const int fn = static_cast<int>(attr_int(op, "fn", 0));
    const float alpha = static_cast<float>(attr_float(op, "alpha", 1.0));
    const void *x = addr(op.in[0]), *dy = addr(op.in[1]);
    void* dx = addr(op.out[0]);
    for (int64_t i = 0; i < n(op.in[0]); ++i) stb(dx, i, ldb(dy, i) * unary_grad(ldb(x, i), fn, alpha));
  } else if (t == "layer_norm_bwd") {
    const int64_t cols = shp(op.in[1]).back(), rows = n(op.in[1]) / cols;
    const void *dy = addr(op.in[0]), *x = addr(op.in[1]), *gamma = addr(op.in[2]);
    const float* stats = static_cast<const float*>(addr(op.in[3]));
    void* dx = addr(op.out[0]);
    const bool params = op.out.size() == 3, accumulate = attr_int(op, "accumulate", 0) != 0;
    std::vector<float> dg(static_cast<size_t>(cols), 0.f), db(static_cast<size_t>(cols), 0.f);
    for (int64_t r = 0; r < rows; ++r) {
      const float mean = stats[r], rstd = stats[rows + r];
      float s1 = 0.f, s2 = 0.f;
      for (int64_t c = 0; c < cols; ++c) {
        const float xh = (ldb(x, r * cols + c) - mean) * rstd, g = ldb(dy, r * cols + c) * ldb(gamma, c);
        s1 += g;
        s2 += g * xh;
        dg[static_cast<size_t>(c)] += ldb(dy, r * cols + c) * xh;
        db[static_cast<size_t>(c)] += ldb(dy, r * cols + c);
      }
      s1 /= static_cast<float>(cols);
      s2 /= static_cast<float>(cols);
      for (int64_t c = 0; c < cols; ++c) {
        const float xh = (ldb(x, r * cols + c) - mean) * rstd, g = ldb(dy, r * cols + c) * ldb(gamma, c);
        stb(dx, r * cols + c, rstd * (g - s1 - xh * s2) + (op.in.size() > 4 ? ldb(addr(op.in[4]), r * cols + c) : 0.f));
      }
    }
    if (params) {
      float *pg = static_cast<float*>(addr(op.out[1])), *pb = static_cast<float*>(addr(op.out[2]));
      for (int64_t c = 0; c < cols; ++c) {
        pg[c] = (accumulate ? pg[c] : 0.f) + dg[static_cast<size_t>(c)];
        pb[c] = (accumulate ? pb[c] : 0.f) + db[static_cast<size_t>(c)];
      }
    }
  } else if (t == "softmax_bwd") {
    const int64_t cols = shp(op.in[0]).back(), rows = n(op.in[0]) / cols;
    const float scale = static_cast<float>(attr_float(op, "scale", 1.0));
    const void *y = addr(op.in[0]), *dy = addr(op.in[1]);
    void* dx = addr(op.out[0]);
    for (int64_t r = 0; r < rows; ++r) {
      float dot = 0.f;
      for (int64_t c = 0; c < cols; ++c) dot += ldb(y, r * cols + c) * ldb(dy, r * cols + c);
      for (int64_t c = 0; c < cols; ++c) stb(dx, r * cols + c, scale * ldb(y, r * cols + c) * (ldb(dy, r * cols + c) - dot));
    }
  } else if (t == "attention_bwd") {
    const auto& q = shp(op.in[0]);
    const auto& k = shp(op.in[1]);
    const int64_t B = q[0], Sq = q[1], H = q[2], D = q[3], Sk = k[1], Hk = k[2];
    const int64_t qs = attr_int(op, "q_stride", H * D), ks = attr_int(op, "kv_stride", Hk * D);
    const int64_t dqs = attr_int(op, "dq_stride", H * D), dks = attr_int(op, "dkv_stride", Hk * D);
    const bool causal = attr_int(op, "causal", 0) != 0;
    const float scale = static_cast<float>(attr_float(op, "scale", 1.0 / std::sqrt(static_cast<double>(D))));
    const void *qp = addr(op.in[0]), *kp = addr(op.in[1]), *vp = addr(op.in[2]), *dop = addr(op.in[4]);
    void *dq = addr(op.out[0]), *dk = addr(op.out[1]), *dv = addr(op.out[2]);
    std::vector<float> dkf(static_cast<size_t>(B * Sk * Hk * D), 0.f), dvf(dkf.size(), 0.f), pr(static_cast<size_t>(Sk)), dqr(static_cast<size_t>(D));
    for (int64_t b = 0; b < B; ++b)
      for (int64_t h = 0; h < H; ++h) {
        const int64_t hk = h / (H / Hk);
        for (int64_t i = 0; i < Sq; ++i) {
          const int64_t vis = causal ? std::min<int64_t>(Sk, i + (Sk - Sq) + 1) : Sk;
          float mx = -INFINITY, sum = 0.f;
          for (int64_t j = 0; j < vis; ++j) {
            float s = 0.f;
            for (int64_t d = 0; d < D; ++d) s += ldb(qp, (b * Sq + i) * qs + h * D + d) * ldb(kp, (b * Sk + j) * ks + hk * D + d);
            pr[static_cast<size_t>(j)] = s * scale;
            mx = std::max(mx, s * scale);
          }
          for (int64_t j = 0; j < vis; ++j) sum += (pr[static_cast<size_t>(j)] = std::exp(pr[static_cast<size_t>(j)] - mx));
          float delta = 0.f;
          std::vector<float> dp(static_cast<size_t>(std::max<int64_t>(vis, 0)));
          for (int64_t j = 0; j < vis; ++j) {
            pr[static_cast<size_t>(j)] /= sum;
            float a = 0.f;
            for (int64_t d = 0; d < D; ++d) a += ldb(dop, ((b * Sq + i) * H + h) * D + d) * ldb(vp, (b * Sk + j) * ks + hk * D + d);
            dp[static_cast<size_t>(j)] = a;
            delta += pr[static_cast<size_t>(j)] * a;
          }
          std::fill(dqr.begin(), dqr.end(), 0.f);
          for (int64_t j = 0; j < vis; ++j) {
            const float pj = pr[static_cast<size_t>(j)], ds = pj * (dp[static_cast<size_t>(j)] - delta) * scale;
            const size_t kv = static_cast<size_t>(((b * Sk + j) * Hk + hk) * D);
            for (int64_t d = 0; d < D; ++d) {
              dqr[static_cast<size_t>(d)] += ds * ldb(kp, (b * Sk + j) * ks + hk * D + d);
              dkf[kv + static_cast<size_t>(d)] += ds * ldb(qp, (b * Sq + i) * qs + h * D + d);
              dvf[kv + static_cast<size_t>(d)] += pj * ldb(dop, ((b * Sq + i) * H + h) * D + d);
            }
          }
          for (int64_t d = 0; d < D; ++d) stb(dq, (b * Sq + i) * dqs + h * D + d, dqr[static_cast<size_t>(d)]);
        }
      }
    for (int64_t b = 0; b < B; ++b)
      for (int64_t j = 0; j < Sk; ++j)
        for (int64_t hk = 0; hk < Hk; ++hk)
          for (int64_t d = 0; d < D; ++d) {
            const size_t src = static_cast<size_t>(((b * Sk + j) * Hk + hk) * D + d);
            stb(dk, (b * Sk + j) * dks + hk * D + d, dkf[src]);
            stb(dv, (b * Sk + j) * dks + hk * D + d, dvf[src]);
          }
  } else if (t == "embedding_bwd") {
    const int64_t ids_n = n(op.in[0]), cols = shp(op.in[1])[1], rows = shp(op.out[0])[0];
    const int64_t* ids = static_cast<const int64_t*>(addr(op.in[0]));
    const void* dy = addr(op.in[1]);
    float* g = static_cast<float*>(addr(op.out[0]));
    for (int64_t i = 0; i < ids_n; ++i)
      if (ids[i] >= 0 && ids[i] < rows)
        for (int64_t c = 0; c < cols; ++c) g[ids[i] * cols + c] += ldb(dy, i * cols + c);
  } else if (t == "cross_entropy") {
    const int64_t cols = shp(op.in[0]).back(), rows = n(op.in[1]);
    const int64_t ignore = attr_int(op, "ignore_index", -100);
    const float grad_scale = static_cast<float>(attr_float(op, "grad_scale", 1.0));   // 1 / accumulation steps
    const void* x = addr(op.in[0]);
    const int64_t* y = static_cast<const int64_t*>(addr(op.in[1]));
    void* dx = op.out.size() > 1 ? addr(op.out[1]) : nullptr;
    double total = 0.0;
    for (int64_t r = 0; r < rows; ++r) {
      float mx = -INFINITY, sum = 0.f;
      for (int64_t c = 0; c < cols; ++c) mx = std::max(mx, ldb(x, r * cols + c));
      for (int64_t c = 0; c < cols; ++c) sum += std::exp(ldb(x, r * cols + c) - mx);
      const bool live = y[r] != ignore && y[r] >= 0 && y[r] < cols;
      if (live) total += std::log(sum) + mx - ldb(x, r * cols + y[r]);
      if (dx)
        for (int64_t c = 0; c < cols; ++c)
          stb(dx, r * cols + c, live ? (std::exp(ldb(x, r * cols + c) - mx) / sum - (c == y[r] ? 1.f : 0.f)) * grad_scale / static_cast<float>(rows) : 0.f);
    }
    static_cast<float*>(addr(op.out[0]))[0] = static_cast<float>(total / static_cast<double>(rows));
  } else if (t == "mse") {
    const void *a = addr(op.in[0]), *b = addr(op.in[1]);
    double total = 0.0;
    for (int64_t i = 0; i < n(op.in[0]); ++i) {
      const double d = static_cast<double>(ldb(a, i)) - static_cast<double>(ldb(b, i));
      total += d * d;
    }
    static_cast<float*>(addr(op.out[0]))[0] = static_cast<float>(total / static_cast<double>(n(op.in[0])));
  } else if (t == "grad_clip") {
    double sq = 0.0, bad = 0.0;
    for (int g : op.in) {
      const float* p = static_cast<const float*>(addr(g));
      for (int64_t e = 0; e < n(g); ++e) {
        if (!std::isfinite(p[e])) bad += 1.0;
        else sq += static_cast<double>(p[e]) * p[e];
      }
    }
    const float max_norm = static_cast<float>(attr_float(op, "max_norm", 0.0)), norm = static_cast<float>(std::sqrt(sq));
    float* out = static_cast<float*>(addr(op.out[0]));
    out[0] = static_cast<float>(sq);
    out[1] = static_cast<float>(bad);
    out[2] = max_norm > 0.f ? std::min(1.f, max_norm / (norm + 1e-6f)) : 1.f;
    out[3] = norm;
  } else if (t == "adamw_update" || t == "sgd_update") {
    const int64_t np = attr_int(op, "n", 0), states = attr_int(op, "states", 0);
    const bool adam = t == "adamw_update";
    const float gscale = attr_int(op, "clip", 0) ? static_cast<const float*>(addr(op.in[static_cast<size_t>(np)]))[2] : 1.f;
    const float lr = scheduled_lr(std::max<int64_t>(train_steps, 1)), b1 = train.beta1, b2 = train.beta2;
    const float wd = attr_int(op, "decay", 1) != 0 ? train.weight_decay : 0.f;   // the group of vectors is not decayed
    const float bc1 = 1.f - std::pow(b1, static_cast<float>(train_steps)), bc2 = 1.f - std::pow(b2, static_cast<float>(train_steps));
    for (int64_t i = 0; i < np; ++i) {
      const float* g = static_cast<const float*>(addr(op.in[static_cast<size_t>(i)]));
      void* copy = addr(op.out[static_cast<size_t>(i)]);
      float* w = static_cast<float*>(addr(op.out[static_cast<size_t>(np + i)]));
      float* s1 = states >= 1 ? static_cast<float*>(addr(op.out[static_cast<size_t>(2 * np + i)])) : nullptr;
      float* s2 = states >= 2 ? static_cast<float*>(addr(op.out[static_cast<size_t>(3 * np + i)])) : nullptr;
      for (int64_t e = 0; e < n(op.in[static_cast<size_t>(i)]); ++e) {
        float grad = g[e] * gscale;
        if (adam) {
          s1[e] = b1 * s1[e] + (1.f - b1) * grad;
          s2[e] = b2 * s2[e] + (1.f - b2) * grad * grad;
          const float denom = std::sqrt(s2[e]) / std::sqrt(bc2) + train.eps;
          w[e] = w[e] - (lr / bc1) * (s1[e] / denom) - lr * wd * w[e];
        } else {
          if (s1) {
            s1[e] = train.momentum * s1[e] + grad;
            grad = s1[e];
          }
          w[e] = w[e] - lr * grad - lr * wd * w[e];
        }
        stb(copy, e, w[e]);
      }
    }
  } else {
    return false;
  }
  return true;
}

// ------------------------------------------------------------------------------------------------ GPU
bool Graph::Impl::run_train_op_device(const PlannedOp& p, cudaStream_t s) {
  const OpDef& op = *p.def;
  auto ok = [&](int rc) {
    if (rc != 0) throw std::runtime_error(op.type + ": " + ofb_last_error());
  };
  auto shp = [&](int t) -> const std::vector<int64_t>& { return plan->shape[static_cast<size_t>(t)]; };
  auto dt = [&](int t) { return ir.tensors[static_cast<size_t>(t)].dtype; };
  auto n = [&](int t) { return numel(shp(t)); };
  auto code = [&](int t) { return dt(t) == DType::kFloat ? 0 : 1; };   // dtype codes of the kernel library
  const std::string& t = op.type;
  if (t == "fill") {
    if (attr_float(op, "value", 0.0) != 0.0) throw std::runtime_error("fill: only zero is built on the GPU");
    check_cuda(cudaMemsetAsync(addr(op.out[0]), 0, static_cast<size_t>(n(op.out[0]) * SizeOf(dt(op.out[0]))), s), "cudaMemsetAsync");
  } else if (t == "cast") {
    ok(ofb_cast_scale(addr(op.in[0]), code(op.in[0]), addr(op.out[0]), code(op.out[0]), n(op.in[0]), static_cast<float>(attr_float(op, "scale", 1.0)),
                      nullptr, s));
  } else if (t == "copy") {
    if (attr_int(op, "accumulate", 0) == 0) return false;
    const auto sh = int_list(attr_str(op, "shape", "")), is = int_list(attr_str(op, "in_strides", "")), os = int_list(attr_str(op, "out_strides", ""));
    std::vector<long long> a(sh.begin(), sh.end()), b(is.begin(), is.end()), c(os.begin(), os.end());
    ok(ofb_graph_strided_acc(addr(op.in[0]), code(op.in[0]), addr(op.out[0]), code(op.out[0]), static_cast<int>(a.size()), a.data(), b.data(),
                             attr_int(op, "in_offset", 0), c.data(), attr_int(op, "out_offset", 0), s));
  } else if (t == "column_sum") {
    ok(ofb_column_sum(addr(op.in[0]), static_cast<float*>(addr(op.out[0])), static_cast<int>(shp(op.in[0])[0]), static_cast<int>(shp(op.in[0])[1]), s));
  } else if (t == "dropout" && (!ir.training || call_kind == 4)) {
    check_cuda(cudaMemcpyAsync(addr(op.out[0]), addr(op.in[0]), static_cast<size_t>(n(op.in[0]) * 2), cudaMemcpyDeviceToDevice, s), "cudaMemcpyAsync");
  } else if (t == "dropout") {
    ok(ofb_graph_dropout(addr(op.in[0]), addr(op.out[0]), n(op.in[0]), train.seed, call_counter_device(), static_cast<unsigned int>(attr_int(op, "index", 0)),
                         static_cast<float>(attr_float(op, "p", 0.5)), s));
  } else if (t == "unary_bwd") {
    ok(ofb_graph_unary_bwd(addr(op.in[0]), addr(op.in[1]), addr(op.out[0]), n(op.in[0]), static_cast<int>(attr_int(op, "fn", 0)),
                           static_cast<float>(attr_float(op, "alpha", 1.0)), s));
  } else if (t == "layer_norm_bwd") {
    const int64_t cols = shp(op.in[1]).back(), rows = n(op.in[1]) / cols;
    const float* stats = static_cast<const float*>(addr(op.in[3]));
    const bool params = op.out.size() == 3;
    ok(ofb_layer_norm_bwd(addr(op.in[0]), addr(op.in[1]), addr(op.in[2]), stats, stats + rows, op.in.size() > 4 ? addr(op.in[4]) : nullptr, addr(op.out[0]),
                          params ? static_cast<float*>(addr(op.out[1])) : nullptr, params ? static_cast<float*>(addr(op.out[2])) : nullptr,
                          static_cast<float*>(p.workspace), attr_int(op, "accumulate", 0) != 0 ? 1 : 0, static_cast<int>(rows), static_cast<int>(cols), s));
  } else if (t == "softmax_bwd") {
    const int64_t cols = shp(op.in[0]).back(), rows = n(op.in[0]) / cols;
    ok(ofb_softmax_bwd(addr(op.in[0]), addr(op.in[1]), nullptr, addr(op.out[0]), rows, static_cast<int>(cols), 0, 0, 0,
                       static_cast<float>(attr_float(op, "scale", 1.0)), 1.f, s));
  } else if (t == "attention_bwd") {
    const auto& q = shp(op.in[0]);
    const auto& k = shp(op.in[1]);
    const int64_t H = q[2], D = q[3], Hk = k[2];
    ok(ofb_fmha_bwd_ex(addr(op.in[0]), addr(op.in[1]), addr(op.in[2]), attr_int(op, "q_stride", H * D), attr_int(op, "kv_stride", Hk * D), addr(op.in[3]),
                       addr(op.in[4]), static_cast<const float*>(addr(op.in[5])), addr(op.out[0]), addr(op.out[1]), addr(op.out[2]),
                       attr_int(op, "dq_stride", H * D), attr_int(op, "dkv_stride", Hk * D), static_cast<float*>(p.workspace), nullptr, static_cast<int>(q[0]),
                       static_cast<int>(q[1]), static_cast<int>(k[1]), static_cast<int>(H), static_cast<int>(Hk), static_cast<int>(D),
                       static_cast<int>(attr_int(op, "causal", 0)), static_cast<float>(attr_float(op, "scale", 1.0 / std::sqrt(static_cast<double>(D)))), 0.f,
                       0ull, 0u, s));
  } else if (t == "embedding_bwd") {
    const int64_t cols = shp(op.in[1])[1], rows = shp(op.out[0])[0];
    ok(ofb_embedding_bwd(static_cast<const long long*>(addr(op.in[0])), addr(op.in[1]), static_cast<float*>(addr(op.out[0])), nullptr, n(op.in[0]), 1,
                         static_cast<int>(cols), 0, rows, 0, s));
  } else if (t == "cross_entropy") {
    const int64_t cols = shp(op.in[0]).back(), rows = n(op.in[1]);
    float* stats = static_cast<float*>(p.workspace);
    float* row_loss = stats + rows * 3;
    void* dx = op.out.size() > 1 ? addr(op.out[1]) : static_cast<void*>(row_loss + rows);
    const long long* labels = static_cast<const long long*>(addr(op.in[1]));
    ok(ofb_xent_stats(addr(op.in[0]), labels, stats, static_cast<int>(rows), static_cast<int>(cols), cols, 0, s));
    ok(ofb_xent_grad(addr(op.in[0]), labels, stats, row_loss, dx, static_cast<int>(rows), static_cast<int>(cols), cols, 0,
                     static_cast<float>(attr_float(op, "grad_scale", 1.0)) / static_cast<float>(rows), attr_int(op, "ignore_index", -100), s));
    ok(ofb_graph_sum_f32(row_loss, static_cast<float*>(addr(op.out[0])), rows, 1.f / static_cast<float>(rows), s));
  } else if (t == "mse") {
    ok(ofb_graph_mse(addr(op.in[0]), addr(op.in[1]), static_cast<float*>(addr(op.out[0])), static_cast<float*>(p.workspace), n(op.in[0]), s));
  } else if (t == "grad_clip") {
    float* out = static_cast<float*>(addr(op.out[0]));
    const int64_t ng = static_cast<int64_t>(op.in.size());
    for (int64_t first = 0; first < ng; first += 48) {
      const int cnt = static_cast<int>(std::min<int64_t>(48, ng - first));
      std::vector<void*> grads;
      std::vector<long long> sizes;
      for (int i = 0; i < cnt; ++i) {
        grads.push_back(addr(op.in[static_cast<size_t>(first + i)]));
        sizes.push_back(n(op.in[static_cast<size_t>(first + i)]));
      }
      ok(ofb_multi_tensor_sqsum(cnt, grads.data(), sizes.data(), 0, static_cast<float*>(p.workspace), out, first > 0 ? 1 : 0, s));
    }
    ok(ofb_clip_factor(out, static_cast<float>(attr_float(op, "max_norm", 0.0)), out + 2, nullptr, out + 3, s));
  } else if (t == "adamw_update" || t == "sgd_update") {
    const int64_t np = attr_int(op, "n", 0), states = attr_int(op, "states", 0);
    const bool adam = t == "adamw_update";
    const float* gscale = attr_int(op, "clip", 0) ? static_cast<const float*>(addr(op.in[static_cast<size_t>(np)])) + 2 : nullptr;
    const float wd = attr_int(op, "decay", 1) != 0 ? train.weight_decay : 0.f;   // the group of vectors is not decayed
    for (int64_t first = 0; first < np; first += 48) {   // the multi-tensor kernels take 48 tensors per launch
      const int cnt = static_cast<int>(std::min<int64_t>(48, np - first));
      std::vector<void*> grads, copies;
      std::vector<float*> masters, s1, s2;
      std::vector<long long> sizes;
      for (int i = 0; i < cnt; ++i) {
        const size_t e = static_cast<size_t>(first + i);
        grads.push_back(addr(op.in[e]));
        copies.push_back(addr(op.out[e]));
        masters.push_back(static_cast<float*>(addr(op.out[static_cast<size_t>(np) + e])));
        if (states >= 1) s1.push_back(static_cast<float*>(addr(op.out[static_cast<size_t>(2 * np) + e])));
        if (states >= 2) s2.push_back(static_cast<float*>(addr(op.out[static_cast<size_t>(3 * np) + e])));
        sizes.push_back(n(op.in[e]));
      }
      // learning rate and bias corrections come from the device (refreshed before every step), nothing here depends on the step
      if (adam)
        ok(ofb_multi_tensor_adamw_dev(cnt, grads.data(), masters.data(), copies.data(), s1.data(), s2.data(), sizes.data(), 0, train.beta1,
                                      train.beta2, train.eps, wd, step_scalars, gscale, s));
      else
        ok(ofb_multi_tensor_sgd(cnt, grads.data(), masters.data(), copies.data(), states >= 1 ? s1.data() : nullptr, sizes.data(), 0, 0.f,
                                train.momentum, 0.f, 0, 0, wd, 0.f, 0.f, 1.f, step_scalars, gscale, nullptr, s));
    }
  } else {
    return false;
  }
  return true;
}

}  // namespace oneflow_api
