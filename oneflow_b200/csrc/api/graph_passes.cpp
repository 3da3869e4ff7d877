// Rewriting passes over the operator IR, run in a fixed order after a graph is loaded (and, for training graphs, after the
// backward operators were appended) and before the plan compiler sees it. Each pass is a peephole over operators and the
// storages ("roots") they touch; a pass only fires when the intermediate it removes has no other reader or writer.
//
//   fuse_activation_forward   linear -> gelu / relu            =>  linear with the activation in the GEMM epilogue; when a
//                                                                   backward operator still reads the pre-activation, the
//                                                                   epilogue also stores it (second output)
//   fuse_activation_backward  matmul -> unary_bwd(pre-act, .)  =>  matmul whose epilogue multiplies by act'(pre-activation):
//                                                                   the data-gradient GEMM of the NEXT layer produces the
//                                                                   gradient w.r.t. the pre-activation directly
//   recompute_cheap_activations (training, on request)  an element-wise operator or LayerNorm of the forward pass whose output
//                             the backward pass reads, and whose inputs are kept for the backward pass anyway, is run
//                             again right before its first backward reader; the backward readers use the copy, so the
//                             original dies with its last forward reader (activation checkpointing for the cheap part)
//                             With recompute_all_but_residual_stream the same pass takes every operator (GEMMs and
//                             attention included) whose result has a single forward reader: only the residual stream
//                             survives the forward pass, and the copies pull in their producers transitively
//   drop_dead_operators       operators none of whose outputs is read by an operator or returned
//
// ONEFLOW_API_PASSES=0 switches all of them off (the unfused plan is the reference the tests compare with).
//
// Reference counterparts: the ordered pass list of LazyJobBuildAndInferCtx::Complete (oneflow/core/job/job_build_and_infer_ctx.cpp),
// fuse patterns such as fused_bias_add_gelu (oneflow/ir/lib/OneFlow/PDLL/, oneflow/core/job_rewriter/fuse_*_pass.cpp) and
// dead-code elimination on the job (oneflow/core/job_rewriter/prune_*_pass.cpp).
#include <algorithm>
#include <cstdlib>
#include <set>

#include "graph_impl.h"

namespace oneflow_api {

namespace {

struct View {
  const IR& ir;
  explicit View(const IR& i) : ir(i) {}
  int root(int t) const {
    while (ir.tensors[static_cast<size_t>(t)].alias_of >= 0) t = ir.tensors[static_cast<size_t>(t)].alias_of;
    return t;
  }
  int64_t offset(int t) const {
    int64_t off = 0;
    while (ir.tensors[static_cast<size_t>(t)].alias_of >= 0) {
      off += ir.tensors[static_cast<size_t>(t)].alias_off;
      t = ir.tensors[static_cast<size_t>(t)].alias_of;
    }
    return off;
  }
  int64_t count(int t) const { return numel(ir.tensors[static_cast<size_t>(t)].shape); }
  bool whole(int t) const { return offset(t) == 0 && count(t) == count(root(t)); }
};

// operator indices that read / write each root, in order
struct Touches {
  std::vector<std::vector<int>> readers, writers;
  std::set<int> returned;
  Touches(const IR& ir, const View& v) : readers(ir.tensors.size()), writers(ir.tensors.size()) {
    for (size_t i = 0; i < ir.ops.size(); ++i) {
      for (int t : ir.ops[i].in)
        if (t >= 0) readers[static_cast<size_t>(v.root(t))].push_back(static_cast<int>(i));
      for (int t : ir.ops[i].out) writers[static_cast<size_t>(v.root(t))].push_back(static_cast<int>(i));
    }
    for (int t : ir.outputs) returned.insert(v.root(t));
  }
};

const char* act_name(int64_t fn) { return fn == 1 ? "gelu" : fn == 2 ? "gelu_tanh" : fn == 3 ? "relu" : nullptr; }

bool recompute_cheap_activations(IR& ir) {
  const View v(ir);
  const Touches tc(ir, v);
  const int F = ir.n_forward_ops;
  auto kept_for_backward = [&](int root, int except_op) {
    const int kind = ir.tensors[static_cast<size_t>(root)].kind;
    if (kind == 0 || kind == 1) return true;   // graph inputs and parameters are there anyway
    for (int r : tc.readers[static_cast<size_t>(root)])
      if (r >= F && r != except_op) return true;
    return false;
  };
  const bool full = ir.recompute_full;
  auto forward_readers = [&](int root) {
    std::set<int> ops;   // an operator that reads several views of the storage (q, k, v) counts once
    for (int r : tc.readers[static_cast<size_t>(root)])
      if (r < F) ops.insert(r);
    return static_cast<int>(ops.size());
  };
  // Last forward operator first: by the time an operator is looked at, the copies of its consumers exist, so the set of
  // backward readers of its result is final and one copy serves them all.
  for (int i = std::min(F, static_cast<int>(ir.ops.size())) - 1; i >= 0; --i) {
    const OpDef op = ir.ops[static_cast<size_t>(i)];
    if (full) {
      // everything but the loss operators (their results are consumed at once), copies into shared storage and the residual
      // additions (their results are the checkpoints)
      if (op.type == "cross_entropy" || op.type == "mse" || op.type == "copy") continue;
      if (op.type == "binary" && attr_int(op, "fn", 0) == 0 && attr_int(op, "bmode", 0) == 0) continue;
    } else if (op.type != "unary" && op.type != "binary" && op.type != "layer_norm") {
      continue;
    }
    const int R = v.root(op.out[0]);
    if (!v.whole(op.out[0]) || tc.returned.count(R) || tc.writers[static_cast<size_t>(R)].size() != 1) continue;
    if (full && forward_readers(R) > 1) continue;   // the residual stream: a checkpoint
    int first_reader = -1;
    for (int r : tc.readers[static_cast<size_t>(R)])
      if (r >= F && (first_reader < 0 || r < first_reader)) first_reader = r;
    if (first_reader < 0) continue;
    bool ok = true;
    for (int t : op.in) {
      if (t < 0) continue;
      const int r = v.root(t);
      if (r == R || (!full && !kept_for_backward(r, -1))) ok = false;
      for (int w : tc.writers[static_cast<size_t>(r)])
        if (w > i && w < first_reader) ok = false;   // the input would have changed by then
    }
    if (!ok) continue;
    // the copy: same operator, fresh outputs
    auto fresh_like = [&](int t) {
      TensorDef root = ir.tensors[static_cast<size_t>(v.root(t))];
      root.kind = 2;
      root.file.clear();
      root.name.clear();
      ir.tensors.push_back(root);
      const int rid = static_cast<int>(ir.tensors.size()) - 1;
      TensorDef al = ir.tensors[static_cast<size_t>(t)];
      if (al.alias_of < 0) return rid;
      al.alias_of = rid;
      al.alias_off = v.offset(t);
      ir.tensors.push_back(al);
      return static_cast<int>(ir.tensors.size()) - 1;
    };
    OpDef copy = op;
    copy.attr.erase("fwd");   // the copy belongs to the backward pass: an evaluation call does not run it
    for (int& t : copy.out) t = fresh_like(t);
    const int new_root = View(ir).root(copy.out[0]);
    // backward readers switch to the copy
    std::map<int, int> renamed;
    for (size_t j = static_cast<size_t>(F); j < ir.ops.size(); ++j)
      for (int& t : ir.ops[j].in) {
        if (t < 0 || View(ir).root(t) != R) continue;
        auto it = renamed.find(t);
        if (it == renamed.end()) {
          TensorDef al = ir.tensors[static_cast<size_t>(t)];
          const int64_t off = View(ir).offset(t);
          al.alias_of = new_root;
          al.alias_off = off;
          ir.tensors.push_back(al);
          it = renamed.emplace(t, static_cast<int>(ir.tensors.size()) - 1).first;
        }
        t = it->second;
      }
    ir.ops.insert(ir.ops.begin() + first_reader, copy);
    return true;
  }
  return false;
}

bool fuse_activation_forward(IR& ir) {
  const View v(ir);
  const Touches tc(ir, v);
  for (size_t i = 0; i < ir.ops.size(); ++i) {
    OpDef& lin = ir.ops[i];
    if (lin.type != "linear" || lin.out.size() != 1 || attr_str(lin, "act", "none") != "none") continue;
    if (lin.in.size() > 3 && lin.in[3] >= 0) continue;   // the epilogue applies the activation before the residual
    const int h = v.root(lin.out[0]);
    if (!v.whole(lin.out[0]) || tc.returned.count(h) || tc.writers[static_cast<size_t>(h)].size() != 1) continue;
    int act_op = -1;
    bool other = false, saved = false;
    for (int r : tc.readers[static_cast<size_t>(h)]) {
      const OpDef& o = ir.ops[static_cast<size_t>(r)];
      if (o.type == "unary" && act_op < 0 && act_name(attr_int(o, "fn", 0)) && v.whole(o.in[0]) && v.root(o.out[0]) != h) act_op = r;
      else if (r > static_cast<int>(i)) saved = true;   // another reader of the pre-activation (backward operators, recomputed copies): keep it stored
      else other = true;
    }
    if (act_op < 0 || other || act_op < static_cast<int>(i)) continue;
    const OpDef act = ir.ops[static_cast<size_t>(act_op)];
    if (!v.whole(act.out[0]) || tc.writers[static_cast<size_t>(v.root(act.out[0]))].size() != 1) continue;
    lin.attr["act"] = act_name(attr_int(act, "fn", 0));
    const int pre = lin.out[0];
    lin.out = {act.out[0]};
    if (saved) lin.out.push_back(pre);
    ir.ops.erase(ir.ops.begin() + act_op);
    return true;
  }
  return false;
}

bool fuse_activation_backward(IR& ir) {
  const View v(ir);
  const Touches tc(ir, v);
  for (size_t i = 0; i < ir.ops.size(); ++i) {
    OpDef& mm = ir.ops[i];
    if (mm.type != "matmul" || mm.in.size() != 2 || mm.out.size() != 1 || attr_int(mm, "ta", 0) != 0 || attr_int(mm, "accumulate", 0) != 0) continue;
    if (ir.tensors[static_cast<size_t>(mm.out[0])].dtype != DType::kBFloat16 || ir.tensors[static_cast<size_t>(mm.in[0])].shape.size() != 2) continue;
    const int t = v.root(mm.out[0]);
    if (!v.whole(mm.out[0]) || tc.returned.count(t) || tc.writers[static_cast<size_t>(t)].size() != 1 || tc.readers[static_cast<size_t>(t)].size() != 1) continue;
    const int j = tc.readers[static_cast<size_t>(t)][0];
    const OpDef ub = ir.ops[static_cast<size_t>(j)];
    if (ub.type != "unary_bwd" || j < static_cast<int>(i) || !act_name(attr_int(ub, "fn", 0))) continue;
    if (v.root(ub.in[1]) != t || !v.whole(ub.in[1]) || v.root(ub.in[0]) == t || !v.whole(ub.in[0]) || !v.whole(ub.out[0])) continue;
    if (tc.writers[static_cast<size_t>(v.root(ub.out[0]))].size() != 1) continue;
    bool ready = true;   // the pre-activation must exist where the GEMM runs (a recomputed copy may be produced later)
    for (int w : tc.writers[static_cast<size_t>(v.root(ub.in[0]))]) ready = ready && w < static_cast<int>(i);
    if (!ready) continue;
    mm.in.push_back(ub.in[0]);
    mm.attr["act_grad"] = act_name(attr_int(ub, "fn", 0));
    mm.out = {ub.out[0]};
    ir.ops.erase(ir.ops.begin() + j);
    return true;
  }
  return false;
}

bool drop_dead_operators(IR& ir) {
  const View v(ir);
  const Touches tc(ir, v);
  for (size_t i = ir.ops.size(); i-- > 0;) {
    const OpDef& op = ir.ops[i];
    if (op.type == "adamw_update" || op.type == "sgd_update") continue;
    bool live = false;
    for (int t : op.out) {
      const int r = v.root(t);
      if (tc.returned.count(r)) live = true;
      for (int reader : tc.readers[static_cast<size_t>(r)])
        if (reader > static_cast<int>(i)) live = true;
    }
    if (live) continue;
    ir.ops.erase(ir.ops.begin() + static_cast<long>(i));
    return true;
  }
  return false;
}

}  // namespace

std::vector<std::pair<std::string, int>> run_graph_passes(IR& ir) {
  std::vector<std::pair<std::string, int>> report;
  const char* off = std::getenv("ONEFLOW_API_PASSES");
  if (off && off[0] == '0') return report;
  struct Pass {
    const char* name;
    bool (*fn)(IR&);
  };
  // backward first: the forward pass must see which pre-activations a fused data-gradient GEMM still reads
  if (ir.training && (ir.recompute_cheap || ir.recompute_full)) {
    int fired = 0;
    while (fired < 100000 && recompute_cheap_activations(ir)) ++fired;
    report.emplace_back("recompute_cheap_activations", fired);
  }
  const Pass passes[] = {{"fuse_activation_backward", fuse_activation_backward},
                         {"fuse_activation_forward", fuse_activation_forward},
                         {"drop_dead_operators", drop_dead_operators}};
  for (const Pass& p : passes) {
    if (!ir.training && std::string(p.name) != "drop_dead_operators" && std::string(p.name) != "fuse_activation_forward") continue;
    int fired = 0;
    while (fired < 100000 && p.fn(ir)) ++fired;
    report.emplace_back(p.name, fired);
  }
  return report;
}

}  // namespace oneflow_api
