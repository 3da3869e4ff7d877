// Reverse-mode differentiation of the operator IR: turns a forward graph whose first output is a scalar loss into a
// training step by appending gradient buffers, backward operators and one optimizer update operator. The result is an IR
// like any other: the plan compiler shares memory between forward activations, gradients and temporaries from their
// lifetimes, derives the dependency edges and spreads independent chains (the weight-gradient GEMMs, for one) over streams.
//
// Gradient storage follows the forward storage: every forward storage ("root" tensor) that needs a gradient gets one
// gradient root of the same length (bf16 for activations, fp32 for parameters), and the gradient of a view is the same view
// of that root. A root with a single whole-tensor consumer is written directly by that consumer's backward operator; a
// root with several consumers (a residual stream, tied weights, slices of one buffer) is zero-filled first and every
// consumer adds its part: natively where the kernel can (fp32 GEMM accumulation, column sums, scatter-add, LayerNorm
// parameter gradients) and through a temporary plus a strided accumulate otherwise.
//
// Reference counterparts: the autograd pass over a job (oneflow/core/job_rewriter/autograd.cpp, generate_optimizer_op_confs
// in oneflow/core/job_rewriter/optimizer.cpp) and the per-operator gradient builders (oneflow/core/autograd/gradient_funcs/).
#include <algorithm>
#include <sstream>
#include <stdexcept>

#include "graph_impl.h"

namespace oneflow_api {

namespace {

// kResidualLayerNorm: the pre-LN residual pattern, x read by a LayerNorm and (later) by a same-shape addition. The addition's
// part of dx is its own output gradient; the LayerNorm backward kernel adds it while it writes dx, so the storage needs
// neither a zero fill nor an accumulate pass.
enum class Mode { kNone, kDirect, kDirectStrided, kAccumulate, kResidualLayerNorm };

struct Use {
  int op, slot, tensor;
};

struct Target {
  int out = -1;          // tensor the backward operator writes
  bool native = false;   // the operator adds into it (fp32 parameter gradient)
  int temp = -1;         // flat temporary to be accumulated afterwards, or -1
  int tensor = -1;       // forward tensor whose gradient this is
};

std::string join(const std::vector<int64_t>& v) {
  std::string s;
  for (size_t i = 0; i < v.size(); ++i) s += (i ? "," : "") + std::to_string(v[i]);
  return s;
}
std::string fstr(double v) {
  std::ostringstream ss;
  ss.precision(9);
  ss << v;
  return ss.str();
}

std::vector<int> diff_slots(const OpDef& op) {
  const std::string& t = op.type;
  if (t == "linear") return {0, 1, 2, 3};
  if (t == "matmul" || t == "binary" || t == "mse") return {0, 1};
  if (t == "layer_norm" || t == "attention") return {0, 1, 2};
  if (t == "embedding") return {1};
  if (t == "unary" || t == "softmax" || t == "copy" || t == "cross_entropy" || t == "dropout" || t == "column_sum" || t == "cast") return {0};
  return {};
}

struct Builder {
  IR& ir;
  const TrainOptions& opt;
  std::vector<OpDef> out_ops;
  std::vector<int> grad_root;   // forward root -> gradient root, or -1
  std::vector<Mode> mode;
  std::vector<char> requires_grad, reaches_loss;
  std::map<int, int> pending_add;   // kResidualLayerNorm roots: the addition's output gradient, waiting for the LayerNorm backward

  Builder(IR& i, const TrainOptions& o) : ir(i), opt(o) {}

  int root(int t) const {
    while (ir.tensors[static_cast<size_t>(t)].alias_of >= 0) t = ir.tensors[static_cast<size_t>(t)].alias_of;
    return t;
  }
  int64_t abs_off(int t) const {
    int64_t off = 0;
    while (ir.tensors[static_cast<size_t>(t)].alias_of >= 0) {
      off += ir.tensors[static_cast<size_t>(t)].alias_off;
      t = ir.tensors[static_cast<size_t>(t)].alias_of;
    }
    return off;
  }
  // NOTE: a reference into the tensor table; it dies with the next new_root / alias
  const std::vector<int64_t>& shape(int t) const { return ir.tensors[static_cast<size_t>(t)].shape; }
  int64_t count(int t) const { return numel(shape(t)); }
  bool whole(int t) const { return abs_off(t) == 0 && count(t) == count(root(t)); }

  int new_root(DType dt, int64_t n, int kind = 2) {
    TensorDef t;
    t.dtype = dt;
    t.shape = {std::max<int64_t>(n, 1)};
    t.kind = kind;
    ir.tensors.push_back(t);
    grad_root.push_back(-1);
    mode.push_back(Mode::kNone);
    requires_grad.push_back(0);
    reaches_loss.push_back(0);
    return static_cast<int>(ir.tensors.size()) - 1;
  }
  int alias(int of, int64_t off, const std::vector<int64_t>& shp) {
    const int r = root(of);
    TensorDef t;
    t.dtype = ir.tensors[static_cast<size_t>(r)].dtype;
    t.kind = ir.tensors[static_cast<size_t>(r)].kind;
    t.shape = shp;
    t.alias_of = r;
    t.alias_off = abs_off(of) + off;
    ir.tensors.push_back(t);
    grad_root.push_back(-1);
    mode.push_back(Mode::kNone);
    requires_grad.push_back(0);
    reaches_loss.push_back(0);
    return static_cast<int>(ir.tensors.size()) - 1;
  }
  int view2d(int t, int64_t rows, int64_t cols) { return alias(t, 0, {rows, cols}); }

  OpDef& emit(const std::string& type, std::vector<int> in, std::vector<int> out, std::map<std::string, std::string> attr = {}) {
    OpDef op;
    op.type = type;
    op.in = std::move(in);
    op.out = std::move(out);
    op.attr = std::move(attr);
    out_ops.push_back(std::move(op));
    return out_ops.back();
  }

  // ---- gradient storage
  int grad_storage(int r) {
    if (grad_root[static_cast<size_t>(r)] >= 0) return grad_root[static_cast<size_t>(r)];
    const bool param = ir.tensors[static_cast<size_t>(r)].kind == 1;
    // with gradient accumulation a parameter gradient outlives the call: persistent storage, cleared on the first micro-batch only
    const bool persistent = param && (opt.accumulation_steps > 1 || opt.external_gradient_reduction);
    const int g = new_root(param ? DType::kFloat : DType::kBFloat16, count(r), persistent ? 3 : 2);
    grad_root[static_cast<size_t>(r)] = g;
    if (mode[static_cast<size_t>(r)] != Mode::kDirect && mode[static_cast<size_t>(r)] != Mode::kResidualLayerNorm) {
      OpDef& f = emit("fill", {}, {g}, {{"value", "0"}});
      if (persistent) f.attr["when"] = "first";
    }
    return g;
  }
  bool has_grad(int t) const { return grad_root[static_cast<size_t>(root(t))] >= 0; }
  int grad_of(int t) {
    const int g = grad_storage(root(t));   // may append tensors: take the shape afterwards, by value
    const std::vector<int64_t> s = shape(t);
    return alias(g, abs_off(t), s);
  }
  bool wants(int t) const { return t >= 0 && requires_grad[static_cast<size_t>(root(t))]; }

  Target target_for(int t, bool op_adds_fp32) {
    const int r = root(t);
    Target tg;
    tg.tensor = t;
    if (mode[static_cast<size_t>(r)] == Mode::kDirect || mode[static_cast<size_t>(r)] == Mode::kResidualLayerNorm) {
      tg.out = grad_of(t);
    } else if (ir.tensors[static_cast<size_t>(r)].kind == 1 && op_adds_fp32) {
      tg.out = grad_of(t);
      tg.native = true;
    } else {
      tg.temp = new_root(DType::kBFloat16, count(t));
      tg.out = alias(tg.temp, 0, shape(t));
    }
    return tg;
  }
  // adds the contiguous tensor `src` (as many elements as t) into the gradient of t
  void accumulate_into(int t, int src) {
    const int64_t n = count(t);
    emit("copy", {root(src)}, {grad_storage(root(t))},
         {{"shape", std::to_string(n)}, {"in_strides", "1"}, {"in_offset", std::to_string(abs_off(src))}, {"out_strides", "1"},
          {"out_offset", std::to_string(abs_off(t))}, {"accumulate", "1"}});
  }
  void finish(const Target& tg) {
    if (tg.temp >= 0) accumulate_into(tg.tensor, tg.temp);
  }
  // the gradient of t is scale * src (src contiguous, same element count)
  void pass_grad(int t, int src, double scale = 1.0) {
    const int r = root(t);
    const bool same_type = ir.tensors[static_cast<size_t>(root(src))].dtype == (ir.tensors[static_cast<size_t>(r)].kind == 1 ? DType::kFloat : DType::kBFloat16);
    if (mode[static_cast<size_t>(r)] == Mode::kResidualLayerNorm) {
      pending_add[r] = src;
    } else if (mode[static_cast<size_t>(r)] == Mode::kDirect && scale == 1.0 && same_type && whole(t) && whole(src) && grad_root[static_cast<size_t>(r)] < 0) {
      // the gradient IS the source: both are complete and read-only from here on, so the storage is shared instead of copied
      grad_root[static_cast<size_t>(r)] = root(src);
    } else if (mode[static_cast<size_t>(r)] == Mode::kDirect) {
      emit("cast", {src}, {grad_of(t)}, {{"scale", fstr(scale)}});
    } else if (scale == 1.0) {
      accumulate_into(t, src);
    } else {
      const int tmp = new_root(ir.tensors[static_cast<size_t>(root(src))].dtype, count(t));
      emit("cast", {src}, {tmp}, {{"scale", fstr(scale)}});
      accumulate_into(t, tmp);
    }
  }

  [[noreturn]] void refuse(const OpDef& op, const std::string& why) const {
    throw std::runtime_error("training graph: operator " + op.type + ": " + why);
  }

  void run();
  void backward_of(const OpDef& op, OpDef& fwd);
};

void Builder::run() {
  if (ir.dynamic_rows) throw std::runtime_error("training graph: export with static shapes (export_graph), not the layer-list form");
  if (opt.optimizer != "adamw" && opt.optimizer != "sgd") throw std::runtime_error("training graph: optimizer must be \"adamw\" or \"sgd\"");
  if (opt.accumulation_steps < 1 || opt.accumulation_steps > 65536) throw std::runtime_error("training graph: accumulation_steps must be between 1 and 65536");
  if (opt.clip_grad_norm < 0.f) throw std::runtime_error("training graph: clip_grad_norm must not be negative");
  const size_t nt = ir.tensors.size();
  const int n_ops = static_cast<int>(ir.ops.size());
  grad_root.assign(nt, -1);
  mode.assign(nt, Mode::kNone);
  requires_grad.assign(nt, 0);
  reaches_loss.assign(nt, 0);

  // the loss
  const int loss = ir.outputs.at(0);
  if (ir.tensors[static_cast<size_t>(loss)].dtype != DType::kFloat || count(loss) != 1)
    throw std::runtime_error("training graph: the first output must be a scalar fp32 loss (cross_entropy or mse)");
  int loss_op = -1;
  for (int i = 0; i < n_ops; ++i)
    for (int t : ir.ops[static_cast<size_t>(i)].out)
      if (root(t) == root(loss)) loss_op = i;
  if (loss_op < 0 || (ir.ops[static_cast<size_t>(loss_op)].type != "cross_entropy" && ir.ops[static_cast<size_t>(loss_op)].type != "mse"))
    throw std::runtime_error("training graph: the loss must be produced by a cross_entropy or mse operator");

  // trainable parameters and what depends on them / what the loss depends on
  for (size_t i = 0; i < nt; ++i) {
    const TensorDef& t = ir.tensors[i];
    if (t.kind == 1 && t.alias_of < 0 && !t.name.empty() && t.dtype == DType::kBFloat16) {
      ir.trainable.push_back(static_cast<int>(i));
      requires_grad[i] = 1;
    }
  }
  if (ir.trainable.empty()) throw std::runtime_error("training graph: the export names no trainable parameter");
  for (int i = 0; i < n_ops; ++i) {
    const OpDef& op = ir.ops[static_cast<size_t>(i)];
    bool any = false;
    for (int s : diff_slots(op))
      if (s < static_cast<int>(op.in.size()) && wants(op.in[static_cast<size_t>(s)])) any = true;
    if (any)
      for (int t : op.out) requires_grad[static_cast<size_t>(root(t))] = 1;
  }
  reaches_loss[static_cast<size_t>(root(loss))] = 1;
  std::vector<char> active(static_cast<size_t>(n_ops), 0);
  for (int i = n_ops - 1; i >= 0; --i) {
    const OpDef& op = ir.ops[static_cast<size_t>(i)];
    bool reach = false, req = false;
    for (int t : op.out) reach = reach || reaches_loss[static_cast<size_t>(root(t))];
    if (!reach) continue;
    for (int s : diff_slots(op))
      if (s < static_cast<int>(op.in.size()) && op.in[static_cast<size_t>(s)] >= 0) {
        reaches_loss[static_cast<size_t>(root(op.in[static_cast<size_t>(s)]))] = 1;
        req = req || wants(op.in[static_cast<size_t>(s)]);
      }
    active[static_cast<size_t>(i)] = req ? 1 : 0;
  }
  // values must be written once: an operator that rewrites its input loses what the backward pass has to read
  {
    std::vector<int> writer(nt, -1);
    for (int i = 0; i < n_ops; ++i) {
      const OpDef& op = ir.ops[static_cast<size_t>(i)];
      for (int t : op.out) {
        const int r = root(t);
        if (!requires_grad[static_cast<size_t>(r)] || !reaches_loss[static_cast<size_t>(r)]) continue;
        for (int in : op.in)
          if (in >= 0 && root(in) == r) refuse(op, "works in place on a tensor the backward pass needs; export the module without in-place operators");
        // several writers are fine when they build one value together: copies into slices (concatenation), a zero fill
        // followed by column sums into it (a reduction)
        auto builds_jointly = [](const std::string& ty) { return ty == "copy" || ty == "fill" || ty == "column_sum"; };
        if (writer[static_cast<size_t>(r)] >= 0 && !(builds_jointly(op.type) && builds_jointly(ir.ops[static_cast<size_t>(writer[static_cast<size_t>(r)])].type)))
          refuse(op, "rewrites a tensor another operator produced");
        writer[static_cast<size_t>(r)] = i;
      }
    }
  }
  // how each storage receives its gradient
  std::vector<std::vector<Use>> uses(nt);
  for (int i = 0; i < n_ops; ++i) {
    if (!active[static_cast<size_t>(i)]) continue;
    const OpDef& op = ir.ops[static_cast<size_t>(i)];
    for (int s : diff_slots(op))
      if (s < static_cast<int>(op.in.size()) && wants(op.in[static_cast<size_t>(s)]))
        uses[static_cast<size_t>(root(op.in[static_cast<size_t>(s)]))].push_back(Use{i, s, op.in[static_cast<size_t>(s)]});
  }
  for (size_t r = 0; r < nt; ++r) {
    const auto& u = uses[r];
    if (u.empty()) continue;
    const OpDef& first = ir.ops[static_cast<size_t>(u[0].op)];
    if (ir.tensors[r].kind == 1) {
      // A parameter with one consumer whose backward operator can overwrite (a GEMM, the LayerNorm backward) owns its
      // gradient: no zero fill, no read-modify-write in the GEMM epilogue. Everything else (tied weights, bias column sums,
      // embedding scatter-adds, gradients kept across micro-batches) accumulates into a cleared buffer.
      const bool overwrites = (first.type == "linear" && u[0].slot == 1) || first.type == "matmul" || (first.type == "layer_norm" && u[0].slot >= 1);
      const bool kept_across_calls = opt.accumulation_steps > 1 || opt.external_gradient_reduction;
      mode[r] = !kept_across_calls && u.size() == 1 && overwrites && whole(u[0].tensor) ? Mode::kDirect : Mode::kAccumulate;
      continue;
    }
    if (u.size() == 1 && first.type != "copy" && first.type != "column_sum" && whole(u[0].tensor)) {
      mode[r] = Mode::kDirect;
      continue;
    }
    if (u.size() == 2) {
      const Use* ln = nullptr;
      const Use* add = nullptr;
      for (const Use& x : u) {
        const OpDef& o = ir.ops[static_cast<size_t>(x.op)];
        if (o.type == "layer_norm" && x.slot == 0) ln = &x;
        if (o.type == "binary" && attr_int(o, "fn", 0) == 0 && attr_int(o, "bmode", 0) == 0) add = &x;
      }
      if (ln && add && add->op > ln->op && whole(ln->tensor) && whole(add->tensor)) {
        mode[r] = Mode::kResidualLayerNorm;
        continue;
      }
    }
    bool one_attention = first.type == "attention";
    for (const Use& x : u) one_attention = one_attention && x.op == u[0].op;
    for (size_t a = 0; one_attention && a < u.size(); ++a)
      for (size_t b = a + 1; b < u.size(); ++b)
        if (abs_off(u[a].tensor) == abs_off(u[b].tensor)) one_attention = false;   // the same view twice: the parts would collide
    mode[r] = one_attention ? Mode::kDirectStrided : Mode::kAccumulate;
  }

  // backward operators, last forward operator first
  for (int i = n_ops - 1; i >= 0; --i) {
    if (!active[static_cast<size_t>(i)]) continue;
    OpDef& fwd = ir.ops[static_cast<size_t>(i)];
    const OpDef snapshot = fwd;
    backward_of(snapshot, fwd);
  }

  // the update: fp32 master weights + optimizer state per trainable parameter that received a gradient
  std::vector<int> grads, params, masters, s1, s2;
  std::vector<int> kept;
  const bool adam = opt.optimizer == "adamw";
  for (int p : ir.trainable) {
    if (grad_root[static_cast<size_t>(p)] < 0) continue;   // not on any path to the loss
    kept.push_back(p);
    grads.push_back(grad_root[static_cast<size_t>(p)]);
    params.push_back(p);
    const int m = new_root(DType::kFloat, count(p), 3);
    ir.tensors[static_cast<size_t>(m)].init_from = p;
    masters.push_back(m);
    if (adam || opt.momentum != 0.f) s1.push_back(new_root(DType::kFloat, count(p), 3));
    if (adam) s2.push_back(new_root(DType::kFloat, count(p), 3));
  }
  if (kept.empty()) throw std::runtime_error("training graph: no trainable parameter is connected to the loss");
  ir.trainable = kept;
  ir.masters = masters;
  ir.grad_tensors = grads;
  std::map<std::string, std::string> when;
  if (opt.accumulation_steps > 1 || opt.external_gradient_reduction) when["when"] = "last";
  // parameter groups: with decay_matrices_only, parameters that are only ever used as vectors (biases, LayerNorm scale and
  // shift) form a second group that the optimizer does not decay
  std::vector<char> is_matrix(params.size(), 1);
  if (opt.decay_matrices_only) {
    for (size_t i = 0; i < params.size(); ++i) {
      size_t axes = 1;
      for (size_t t = 0; t < ir.tensors.size(); ++t)
        if (ir.tensors[t].alias_of >= 0 && root(static_cast<int>(t)) == params[i]) {
          size_t real = 0;
          for (auto dim : ir.tensors[t].shape) real += dim > 1 ? 1 : 0;
          axes = std::max(axes, real);
        }
      is_matrix[i] = axes >= 2 ? 1 : 0;
    }
  }
  int clip = -1;
  if (opt.clip_grad_norm > 0.f) {
    // {sum of squares, non-finite count, clip factor, norm}; the update reads the factor on the device
    clip = new_root(DType::kFloat, 4);
    std::map<std::string, std::string> cattr = when;
    cattr["max_norm"] = fstr(opt.clip_grad_norm);
    emit("grad_clip", grads, {clip}, cattr);
  }
  for (int group = 1; group >= 0; --group) {
    std::vector<int> gin, gp, gm, g1, g2;
    for (size_t i = 0; i < params.size(); ++i) {
      if (is_matrix[i] != group) continue;
      gin.push_back(grads[i]);
      gp.push_back(params[i]);
      gm.push_back(masters[i]);
      if (!s1.empty()) g1.push_back(s1[i]);
      if (!s2.empty()) g2.push_back(s2[i]);
    }
    if (gp.empty()) continue;
    std::vector<int> outs = gp;
    outs.insert(outs.end(), gm.begin(), gm.end());
    outs.insert(outs.end(), g1.begin(), g1.end());
    outs.insert(outs.end(), g2.begin(), g2.end());
    std::map<std::string, std::string> uattr = {{"n", std::to_string(gp.size())}, {"states", std::to_string((s1.empty() ? 0 : 1) + (s2.empty() ? 0 : 1))},
                                                {"decay", group ? "1" : "0"}};
    if (clip >= 0) {
      gin.push_back(clip);
      uattr["clip"] = "1";
    }
    uattr.insert(when.begin(), when.end());
    emit(adam ? "adamw_update" : "sgd_update", gin, outs, uattr);
  }

  ir.n_forward_ops = n_ops;
  for (int i = 0; i < n_ops; ++i) ir.ops[static_cast<size_t>(i)].attr["fwd"] = "1";   // what an evaluation call runs
  ir.recompute_cheap = opt.recompute_cheap_activations;
  ir.recompute_full = opt.recompute_all_but_residual_stream;
  for (auto& op : out_ops) ir.ops.push_back(std::move(op));
  ir.training = true;
}

void Builder::backward_of(const OpDef& op, OpDef& fwd) {
  const std::string& t = op.type;
  auto in = [&](size_t s) { return s < op.in.size() ? op.in[s] : -1; };

  if (t == "cross_entropy") {
    // the forward operator writes d loss / d logits (already divided by the row count) beside the loss
    const int logits = in(0);
    if (opt.accumulation_steps > 1) fwd.attr["grad_scale"] = fstr(1.0 / opt.accumulation_steps);
    if (mode[static_cast<size_t>(root(logits))] == Mode::kDirect) {
      fwd.out.push_back(grad_of(logits));
    } else {
      const int tmp = new_root(DType::kBFloat16, count(logits));
      fwd.out.push_back(alias(tmp, 0, shape(logits)));
      // queued after the forward operators: the accumulate reads the temporary the forward operator fills
      accumulate_into(logits, tmp);
    }
    return;
  }
  if (t == "mse") {
    const int a = in(0), b = in(1);
    const int diff = new_root(DType::kBFloat16, count(a));
    emit("binary", {alias(root(a), abs_off(a), {count(a)}), alias(root(b), abs_off(b), {count(b)})}, {diff}, {{"fn", "1"}, {"bmode", "0"}, {"cols", "1"}});
    const double g = 2.0 / static_cast<double>(count(a)) / static_cast<double>(opt.accumulation_steps);
    if (wants(a)) pass_grad(a, diff, g);
    if (wants(b)) pass_grad(b, diff, -g);
    return;
  }

  // every other operator needs the gradient of its output
  const int y = op.out[0];
  if (!has_grad(y)) return;   // nothing downstream produced a gradient for it
  const int dy = grad_of(y);

  if (t == "linear") {
    if (attr_str(op, "act", "none") != "none") refuse(op, "has a fused activation; export the training graph with fuse=False");
    const int x = in(0), w = in(1), bias = in(2), res = in(3);
    const int64_t N = shape(w)[0], K = shape(w)[1], M = count(x) / K;
    const int dy2 = view2d(dy, M, N);
    if (wants(x)) {
      Target tg = target_for(x, false);
      emit("matmul", {dy2, w}, {view2d(tg.out, M, K)}, {{"tb", "0"}, {"alpha", "1.0"}});
      finish(tg);
    }
    if (wants(w)) {
      Target tg = target_for(w, true);
      emit("matmul", {dy2, view2d(x, M, K)}, {tg.out}, {{"ta", "1"}, {"tb", "0"}, {"alpha", "1.0"}, {"accumulate", tg.native ? "1" : "0"}});
      finish(tg);
    }
    if (wants(bias)) {
      if (ir.tensors[static_cast<size_t>(root(bias))].kind == 1) {
        emit("column_sum", {dy2}, {grad_of(bias)});
      } else {
        const int tmp = new_root(DType::kFloat, N);
        emit("fill", {}, {tmp}, {{"value", "0"}});
        emit("column_sum", {dy2}, {tmp});
        pass_grad(bias, tmp);
      }
    }
    if (wants(res)) pass_grad(res, dy);
  } else if (t == "matmul") {
    const int a = in(0), b = in(1);
    if (attr_int(op, "ta", 0) != 0) refuse(op, "transposed left operands are not differentiated");
    const bool tb = attr_int(op, "tb", 0) != 0;
    const std::string alpha = attr_str(op, "alpha", "1.0");
    const std::vector<int64_t> as = shape(a), bs = shape(b);   // copies: the tensor table grows below
    const int64_t M = as[as.size() - 2], K = as.back(), N = tb ? bs[bs.size() - 2] : bs.back();
    const int64_t batch = count(a) / (M * K), batch_b = count(b) / (N * K);
    std::vector<int64_t> lead(as.begin(), as.end() - 2);
    auto with_lead = [&](int64_t r, int64_t c) {
      std::vector<int64_t> s = lead;
      s.push_back(r);
      s.push_back(c);
      return s;
    };
    const int dy3 = alias(dy, 0, with_lead(M, N));
    if (wants(a)) {
      Target tg = target_for(a, false);
      emit("matmul", {dy3, b}, {alias(tg.out, 0, with_lead(M, K))}, {{"tb", tb ? "0" : "1"}, {"alpha", alpha}});
      finish(tg);
    }
    if (wants(b)) {
      Target tg = target_for(b, true);
      const std::string acc = tg.native ? "1" : "0";
      if (batch_b == 1) {
        // one GEMM over all batches: the batch axis joins the contracted one
        const int a2 = view2d(a, batch * M, K), d2 = view2d(dy, batch * M, N);
        if (tb) emit("matmul", {d2, a2}, {view2d(tg.out, N, K)}, {{"ta", "1"}, {"tb", "0"}, {"alpha", alpha}, {"accumulate", acc}});
        else emit("matmul", {a2, d2}, {view2d(tg.out, K, N)}, {{"ta", "1"}, {"tb", "0"}, {"alpha", alpha}, {"accumulate", acc}});
      } else {
        if (tb) emit("matmul", {dy3, a}, {tg.out}, {{"ta", "1"}, {"tb", "0"}, {"alpha", alpha}, {"accumulate", acc}});
        else emit("matmul", {a, dy3}, {tg.out}, {{"ta", "1"}, {"tb", "0"}, {"alpha", alpha}, {"accumulate", acc}});
      }
      finish(tg);
    }
  } else if (t == "layer_norm") {
    const int x = in(0), gamma = in(1), beta = in(2);
    const int64_t cols = shape(x).back(), rows = count(x) / cols;
    // the forward operator keeps mean and 1/std per row for the backward one
    const int stats = new_root(DType::kFloat, 2 * rows);
    fwd.out.push_back(stats);
    Target tx = wants(x) ? target_for(x, false) : Target{};
    if (!wants(x)) {
      tx.out = new_root(DType::kBFloat16, count(x));
    }
    const bool pg = wants(gamma) || wants(beta);
    int dg = -1, db = -1;
    bool native = false;
    if (pg) {
      const bool gp = wants(gamma) && ir.tensors[static_cast<size_t>(root(gamma))].kind == 1;
      const bool bp = wants(beta) && ir.tensors[static_cast<size_t>(root(beta))].kind == 1;
      if (wants(gamma) != gp || wants(beta) != bp) refuse(op, "scale and shift must be parameters");
      // both parameter gradients are written by one kernel call: they overwrite together or accumulate together
      const bool g_direct = gp && mode[static_cast<size_t>(root(gamma))] == Mode::kDirect, b_direct = bp && mode[static_cast<size_t>(root(beta))] == Mode::kDirect;
      if (!(g_direct && b_direct)) {
        if (g_direct) mode[static_cast<size_t>(root(gamma))] = Mode::kAccumulate;
        if (b_direct) mode[static_cast<size_t>(root(beta))] = Mode::kAccumulate;
      }
      native = !(g_direct && b_direct);
      auto scratch = [&] {
        const int s = new_root(DType::kFloat, cols);
        emit("fill", {}, {s}, {{"value", "0"}});
        return s;
      };
      dg = gp ? grad_of(gamma) : scratch();
      db = bp ? grad_of(beta) : scratch();
    }
    std::vector<int> outs = {tx.out};
    if (pg) {
      outs.push_back(dg);
      outs.push_back(db);
    }
    std::vector<int> ins = {dy, x, gamma, stats};
    if (mode[static_cast<size_t>(root(x))] == Mode::kResidualLayerNorm) {
      if (!pending_add.count(root(x))) refuse(op, "the residual addition that shares its input produced no gradient");
      ins.push_back(pending_add.at(root(x)));   // added to dx by the same kernel
    }
    emit("layer_norm_bwd", ins, outs, {{"accumulate", native ? "1" : "0"}});
    if (wants(x)) finish(tx);
  } else if (t == "embedding") {
    const int ids = in(0), table = in(1);
    if (ir.tensors[static_cast<size_t>(root(table))].kind != 1) refuse(op, "the table must be a parameter");
    const int64_t cols = shape(table)[1];
    emit("embedding_bwd", {ids, view2d(dy, count(ids), cols)}, {grad_of(table)});
  } else if (t == "binary") {
    const int a = in(0), b = in(1);
    const int64_t fn = attr_int(op, "fn", 0), bmode = attr_int(op, "bmode", 0), cols = attr_int(op, "cols", 1);
    if (fn > 2) refuse(op, "only add, sub and mul are differentiated");
    const std::map<std::string, std::string> same = {{"fn", "2"}, {"bmode", std::to_string(bmode)}, {"cols", std::to_string(cols)}};
    if (wants(a)) {
      if (fn == 2) {
        Target tg = target_for(a, false);
        emit("binary", {dy, b}, {tg.out}, same);
        finish(tg);
      } else {
        pass_grad(a, dy);
      }
    }
    if (wants(b)) {
      int g = dy;   // gradient with the output's shape, before the reduction over the broadcast axes
      if (fn == 2) {
        g = new_root(DType::kBFloat16, count(y));
        emit("binary", {alias(dy, 0, {count(y)}), alias(a, 0, {count(a)})}, {g}, {{"fn", "2"}, {"bmode", "0"}, {"cols", "1"}});
      }
      const double sign = fn == 1 ? -1.0 : 1.0;
      if (bmode == 0) {
        pass_grad(b, g, sign);
      } else if (bmode == 1) {
        const int64_t rows = count(y) / cols;
        const bool param = ir.tensors[static_cast<size_t>(root(b))].kind == 1;
        if (param && sign == 1.0) {
          emit("column_sum", {view2d(g, rows, cols)}, {grad_of(b)});
        } else {
          const int tmp = new_root(DType::kFloat, cols);
          emit("fill", {}, {tmp}, {{"value", "0"}});
          emit("column_sum", {view2d(g, rows, cols)}, {tmp});
          pass_grad(b, tmp, sign);
        }
      } else {
        refuse(op, "the gradient of an operand with one value per row is not built");
      }
    }
  } else if (t == "unary") {
    const int x = in(0);
    Target tg = target_for(x, false);
    emit("unary_bwd", {x, dy}, {tg.out}, {{"fn", attr_str(op, "fn", "0")}, {"alpha", attr_str(op, "alpha", "1.0")}});
    finish(tg);
  } else if (t == "column_sum") {
    // every row of the [rows, cols] input receives the gradient of its column's sum: a copy that repeats dy over the rows
    const int x = in(0);
    const std::vector<int64_t> xs = shape(x);
    emit("copy", {root(dy)}, {grad_storage(root(x))},
         {{"shape", join(xs)}, {"in_strides", join({0, 1})}, {"in_offset", std::to_string(abs_off(dy))}, {"out_strides", join({xs[1], 1})},
          {"out_offset", std::to_string(abs_off(x))}, {"accumulate", "1"}});
  } else if (t == "cast") {
    pass_grad(in(0), dy, attr_float(op, "scale", 1.0));
  } else if (t == "dropout") {
    // the same mask (same seed, call and operator index) applied to the gradient
    const int x = in(0);
    Target tg = target_for(x, false);
    emit("dropout", {dy}, {tg.out}, {{"p", attr_str(op, "p", "0.5")}, {"index", attr_str(op, "index", "0")}});
    finish(tg);
  } else if (t == "softmax") {
    const int x = in(0);
    Target tg = target_for(x, false);
    emit("softmax_bwd", {y, dy}, {tg.out}, {{"scale", attr_str(op, "scale", "1.0")}});
    finish(tg);
  } else if (t == "attention") {
    const int q = in(0), k = in(1), v = in(2);
    const std::vector<int64_t> qs = shape(q), ks = shape(k);   // copies: the tensor table grows below
    const int64_t B = qs[0], Sq = qs[1], H = qs[2], D = qs[3], Hk = ks[2];
    const int64_t q_stride = attr_int(op, "q_stride", H * D), kv_stride = attr_int(op, "kv_stride", Hk * D);
    const int lse = new_root(DType::kFloat, B * H * Sq);
    fwd.out.push_back(lse);
    std::map<std::string, std::string> at = {{"causal", attr_str(op, "causal", "0")}, {"q_stride", std::to_string(q_stride)},
                                             {"kv_stride", std::to_string(kv_stride)}};
    if (op.attr.count("scale")) at["scale"] = op.attr.at("scale");
    const bool strided = mode[static_cast<size_t>(root(q))] == Mode::kDirectStrided && root(k) == root(q) && root(v) == root(q);
    const bool direct = mode[static_cast<size_t>(root(q))] == Mode::kDirect && mode[static_cast<size_t>(root(k))] == Mode::kDirect &&
                        mode[static_cast<size_t>(root(v))] == Mode::kDirect && q_stride == H * D && kv_stride == Hk * D;
    if (strided || direct) {
      at["dq_stride"] = std::to_string(q_stride);
      at["dkv_stride"] = std::to_string(kv_stride);
      emit("attention_bwd", {q, k, v, y, dy, lse}, {grad_of(q), grad_of(k), grad_of(v)}, at);
    } else {
      // contiguous temporaries, then strided accumulates into the (possibly interleaved) views
      at["dq_stride"] = std::to_string(H * D);
      at["dkv_stride"] = std::to_string(Hk * D);
      const int tq = new_root(DType::kBFloat16, count(q)), tk = new_root(DType::kBFloat16, count(k)), tv = new_root(DType::kBFloat16, count(v));
      emit("attention_bwd", {q, k, v, y, dy, lse}, {alias(tq, 0, qs), alias(tk, 0, ks), alias(tv, 0, ks)}, at);
      auto scatter = [&](int src, int dst, const std::vector<int64_t>& s, int64_t stride) {
        if (!wants(dst)) return;
        if (mode[static_cast<size_t>(root(dst))] == Mode::kDirect && stride == s[2] * s[3]) {
          emit("cast", {src}, {grad_of(dst)}, {{"scale", "1"}});
          return;
        }
        if (mode[static_cast<size_t>(root(dst))] == Mode::kDirect) refuse(op, "a strided operand cannot own its gradient storage");
        emit("copy", {src}, {grad_storage(root(dst))},
             {{"shape", join(s)}, {"in_strides", join({s[1] * s[2] * s[3], s[2] * s[3], s[3], 1})}, {"in_offset", "0"},
              {"out_strides", join({s[1] * stride, stride, s[3], 1})}, {"out_offset", std::to_string(abs_off(dst))}, {"accumulate", "1"}});
      };
      scatter(tq, q, qs, q_stride);
      scatter(tk, k, ks, kv_stride);
      scatter(tv, v, ks, kv_stride);
    }
  } else if (t == "copy") {
    const int x = in(0);
    const auto is = int_list(attr_str(op, "in_strides", "")), sh = int_list(attr_str(op, "shape", ""));
    bool broadcast = false;
    for (size_t d = 0; d < sh.size(); ++d) broadcast = broadcast || (sh[d] > 1 && is[d] == 0);
    if (broadcast) {
      // A source repeated over leading axes (a class token or a table expanded over the batch): its gradient is the sum of
      // the output gradient over those axes. The output gradient's view is gathered into a [repeats, block] matrix, summed
      // over its rows in fp32 and added to the source's gradient. Broadcasts in inner axes are not built.
      size_t k = 0;
      while (k < sh.size() && (sh[k] == 1 || is[k] == 0)) ++k;
      int64_t rows = 1, cols = 1, expect = 1;
      for (size_t d = 0; d < k; ++d) rows *= sh[d];
      bool dense = true;
      for (size_t d = sh.size(); d-- > k;) {
        if (sh[d] > 1 && is[d] != expect) dense = false;
        expect *= sh[d];
        cols *= sh[d];
      }
      if (!dense || k == sh.size()) refuse(op, "reads a view that is broadcast in an inner axis; its gradient is not built");
      const int gathered = new_root(DType::kBFloat16, rows * cols);
      std::vector<int64_t> dense_strides(sh.size(), 1);
      for (size_t d = sh.size() - 1; d-- > 0;) dense_strides[d] = dense_strides[d + 1] * sh[d + 1];
      emit("copy", {root(dy)}, {gathered},
           {{"shape", attr_str(op, "shape", "")}, {"in_strides", attr_str(op, "out_strides", "")},
            {"in_offset", std::to_string(attr_int(op, "out_offset", 0) + abs_off(y))}, {"out_strides", join(dense_strides)}, {"out_offset", "0"}});
      const int summed = new_root(DType::kFloat, cols);
      emit("fill", {}, {summed}, {{"value", "0"}});
      emit("column_sum", {view2d(gathered, rows, cols)}, {summed});
      emit("copy", {summed}, {grad_storage(root(x))},
           {{"shape", std::to_string(cols)}, {"in_strides", "1"}, {"in_offset", "0"}, {"out_strides", "1"},
            {"out_offset", std::to_string(attr_int(op, "in_offset", 0) + abs_off(x))}, {"accumulate", "1"}});
      return;
    }
    emit("copy", {root(dy)}, {grad_storage(root(x))},
         {{"shape", attr_str(op, "shape", "")}, {"in_strides", attr_str(op, "out_strides", "")},
          {"in_offset", std::to_string(attr_int(op, "out_offset", 0) + abs_off(y))}, {"out_strides", attr_str(op, "in_strides", "")},
          {"out_offset", std::to_string(attr_int(op, "in_offset", 0) + abs_off(x))}, {"accumulate", "1"}});
  } else {
    refuse(op, "has no gradient here");
  }
}

}  // namespace

void append_training_ops(IR& ir, const TrainOptions& options) {
  Builder b(ir, options);
  b.run();
}

std::string ir_to_text(const IR& ir) {
  std::ostringstream ss;
  ss << "oneflow_b200 graph v2\n";
  for (const auto& p : ir.pass_report) ss << "# pass " << p.first << " fired=" << p.second << '\n';
  for (size_t i = 0; i < ir.tensors.size(); ++i) {
    const TensorDef& t = ir.tensors[i];
    ss << "tensor " << i << ' ' << (t.dtype == DType::kBFloat16 ? "bf16" : t.dtype == DType::kInt64 ? "i64" : "f32") << ' '
       << (t.kind == 0 ? "input" : t.kind == 1 ? "param" : t.kind == 2 ? "act" : "state") << ' ' << t.shape.size();
    for (auto d : t.shape) ss << ' ' << d;
    if (!t.file.empty()) ss << " file=" << t.file;
    if (!t.name.empty()) ss << " name=" << t.name;
    if (t.alias_of >= 0) ss << " alias=" << t.alias_of << " offset=" << t.alias_off;
    if (t.init_from >= 0) ss << " init=" << t.init_from;
    ss << '\n';
  }
  for (const OpDef& op : ir.ops) {
    ss << "op " << op.type << " in=";
    for (size_t i = 0; i < op.in.size(); ++i) ss << (i ? "," : "") << op.in[i];
    ss << " out=";
    for (size_t i = 0; i < op.out.size(); ++i) ss << (i ? "," : "") << op.out[i];
    for (const auto& kv : op.attr) ss << ' ' << kv.first << '=' << kv.second;
    ss << '\n';
  }
  for (int t : ir.inputs) ss << "input " << t << '\n';
  for (int t : ir.outputs) ss << "output " << t << '\n';
  return ss.str();
}

}  // namespace oneflow_api
