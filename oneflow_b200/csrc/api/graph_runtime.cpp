// Operator-graph compiler and executor behind oneflow_api::Graph (see oneflow_api.h for the overview).
//
//   graph.txt --parse--> IR (tensors + operators) --compile--> Plan --run--> outputs
//
// IR text (version 2), one record per line:
//   tensor <id> <bf16|i64|f32> <input|param|act> <ndim> <d0> ... [file=<raw file>] [alias=<id>] [offset=<elements>]
//                                                                  [name=<qualified parameter name>: trainable]
//   op <type> in=<id,id,...> out=<id,...> [key=value ...]          (-1 marks an absent optional input)
//   input <id> / output <id>                                      (in call order)
// Tensor ids are dense and operators are listed in a valid execution order. A dimension of -1 is the row count that is
// bound at the first Forward (only the layer-list form, version 1, uses it).
//
// Reference counterparts: the job -> OpGraph -> task graph -> plan pipeline (oneflow/core/job/job_build_and_infer_ctx.cpp,
// oneflow/core/graph/op_graph.cpp, task_graph.cpp, oneflow/core/job/plan_util.cpp), the memory-sharing pass
// (oneflow/core/job/intra_job_mem_sharing_util.cpp) and the runtime that launches the plan
// (oneflow/core/framework/nn_graph.cpp, oneflow/core/lazy/actor/).
#include "graph_impl.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <mutex>
#include <sstream>
#include <stdexcept>

#include "../core/ofc_core.h"
#include "../kernels/ofb_kernels.h"

extern "C" {
int ofb_layer_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, int rows, int cols,
                       float eps, void* stream);
int ofb_softmax_fwd(const void* x, const void* dropout_mask, const void* attn_mask, long long attn_mask_rows, void* y, void* softmax_y,
                    long long rows, int cols, int tril, int tril_rows, int diagonal, float scale, float mask_fill, float out_scale,
                    void* stream);
int ofb_fmha_fwd_ex(const void* q, const void* k, const void* v, long long q_row_stride, long long kv_row_stride, void* out, float* lse,
                    const int* kv_len, int B, int Sq, int Sk, int H, int Hk, int D, int causal, float scale, float p_dropout,
                    unsigned long long seed, unsigned int offset, void* stream);
int ofb_graph_unary(const void* x, void* y, long long n, int fn, float alpha, void* stream);
int ofb_graph_binary(const void* a, const void* b, void* y, long long n, long long cols, int b_mode, int op, void* stream);
int ofb_graph_strided_copy(const void* x, void* y, int ndim, const long long* shape, const long long* in_strides, long long in_offset,
                           const long long* out_strides, long long out_offset, int elem_bytes, void* stream);
int ofb_graph_gather_rows(const long long* ids, const void* table, void* out, long long n_ids, int cols, long long table_rows,
                          void* stream);
}

namespace oneflow_api {

using namespace detail;

namespace {

IR parse_v2(std::istream& f) {
  IR ir;
  std::string line;
  int lineno = 1;
  while (std::getline(f, line)) {
    ++lineno;
    if (line.empty() || line[0] == '#') continue;
    std::istringstream ss(line);
    std::string rec;
    ss >> rec;
    auto bad = [&](const std::string& why) { return std::runtime_error("graph.txt line " + std::to_string(lineno) + ": " + why); };
    if (rec == "tensor") {
      int id, ndim;
      std::string dt, kind;
      ss >> id >> dt >> kind >> ndim;
      if (!ss || id != static_cast<int>(ir.tensors.size())) throw bad("tensor ids must be dense and ascending");
      if (ndim < 0 || ndim > 8) throw bad("tensor rank out of range");
      TensorDef t;
      t.dtype = dt == "bf16" ? DType::kBFloat16 : dt == "i64" ? DType::kInt64 : dt == "f32" ? DType::kFloat : throw bad("unknown dtype " + dt);
      t.kind = kind == "input" ? 0 : kind == "param" ? 1 : kind == "act" ? 2 : throw bad("unknown tensor kind " + kind);
      for (int i = 0; i < ndim; ++i) {
        int64_t d;
        ss >> d;
        if (!ss || d < -1 || d > (int64_t{1} << 40)) throw bad("bad dimension");
        if (d == -1) ir.dynamic_rows = true;
        t.shape.push_back(d);
      }
      {
        int64_t total = 1;
        for (auto d : t.shape) {
          if (d > 0 && total > (int64_t{1} << 40) / d) throw bad("tensor too large");
          total *= d > 0 ? d : 1;
        }
      }
      std::string kv;
      while (ss >> kv) {
        auto eq = kv.find('=');
        if (eq == std::string::npos) throw bad("expected key=value, got " + kv);
        const std::string k = kv.substr(0, eq), v = kv.substr(eq + 1);
        if (k == "file") t.file = v;
        else if (k == "alias") t.alias_of = std::stoi(v);
        else if (k == "offset") t.alias_off = std::stoll(v);
        else if (k == "name") t.name = v;
        else throw bad("unknown tensor attribute " + k);
      }
      if (t.alias_of >= id) throw bad("an alias must point to an earlier tensor");
      if (t.kind == 1 && t.file.empty() && t.alias_of < 0) throw bad("a parameter needs file=");
      ir.tensors.push_back(std::move(t));
    } else if (rec == "op") {
      OpDef op;
      ss >> op.type;
      std::string kv;
      while (ss >> kv) {
        auto eq = kv.find('=');
        if (eq == std::string::npos) throw bad("expected key=value, got " + kv);
        const std::string k = kv.substr(0, eq), v = kv.substr(eq + 1);
        if (k == "in") for (auto x : int_list(v)) op.in.push_back(static_cast<int>(x));
        else if (k == "out") for (auto x : int_list(v)) op.out.push_back(static_cast<int>(x));
        else op.attr[k] = v;
      }
      for (int t : op.in) if (t < -1 || t >= static_cast<int>(ir.tensors.size())) throw bad("operator input out of range");
      for (int t : op.out) if (t < 0 || t >= static_cast<int>(ir.tensors.size())) throw bad("operator output out of range");
      if (op.out.empty()) throw bad("operator without output");
      ir.ops.push_back(std::move(op));
    } else if (rec == "input" || rec == "output") {
      int id;
      ss >> id;
      if (!ss || id < 0 || id >= static_cast<int>(ir.tensors.size())) throw bad("bad tensor id");
      (rec == "input" ? ir.inputs : ir.outputs).push_back(id);
    } else {
      throw bad("unknown record " + rec);
    }
  }
  if (ir.inputs.empty() || ir.outputs.empty()) throw std::runtime_error("graph.txt: the graph needs at least one input and one output");
  return ir;
}

// The layer-list form: "linear in out wfile bfile act" / "layer_norm n gfile bfile eps" / "activation n act" lines, one
// [rows, features] tensor flowing through them; translated to the operator IR with a row count bound later.
IR parse_v1(std::istream& f) {
  IR ir;
  ir.dynamic_rows = true;
  std::string line;
  int64_t width = -1;
  int cur = -1;
  auto add_tensor = [&](DType dt, std::vector<int64_t> shape, int kind, const std::string& file) {
    TensorDef t;
    t.dtype = dt; t.shape = std::move(shape); t.kind = kind; t.file = file;
    ir.tensors.push_back(t);
    return static_cast<int>(ir.tensors.size()) - 1;
  };
  auto ensure_input = [&](int64_t feat) {
    if (cur < 0) {
      cur = add_tensor(DType::kBFloat16, {-1, feat}, 0, "");
      ir.inputs.push_back(cur);
    } else if (width != feat) {
      throw std::runtime_error("layer width does not match the previous layer");
    }
  };
  while (std::getline(f, line)) {
    if (line.empty() || line[0] == '#') continue;
    std::istringstream ss(line);
    std::string kind;
    ss >> kind;
    OpDef op;
    if (kind == "linear") {
      int64_t in, out;
      std::string wf, bf, act;
      ss >> in >> out >> wf >> bf >> act;
      ensure_input(in);
      const int w = add_tensor(DType::kBFloat16, {out, in}, 1, wf);
      const int b = bf == "-" ? -1 : add_tensor(DType::kBFloat16, {out}, 1, bf);
      const int y = add_tensor(DType::kBFloat16, {-1, out}, 2, "");
      op.type = "linear"; op.in = {cur, w, b, -1}; op.out = {y}; op.attr["act"] = act;
      cur = y; width = out;
    } else if (kind == "layer_norm") {
      int64_t n;
      std::string gf, bf, eps;
      ss >> n >> gf >> bf >> eps;
      ensure_input(n);
      const int g = add_tensor(DType::kBFloat16, {n}, 1, gf);
      const int b = add_tensor(DType::kBFloat16, {n}, 1, bf);
      const int y = add_tensor(DType::kBFloat16, {-1, n}, 2, "");
      op.type = "layer_norm"; op.in = {cur, g, b}; op.out = {y}; op.attr["eps"] = eps;
      cur = y; width = n;
    } else if (kind == "activation") {
      int64_t n;
      std::string act;
      ss >> n >> act;
      ensure_input(n);
      const int y = add_tensor(DType::kBFloat16, {-1, n}, 2, "");
      op.type = "unary"; op.in = {cur}; op.out = {y}; op.attr["fn"] = std::to_string(act_code(act));
      cur = y; width = n;
    } else {
      throw std::runtime_error("unknown layer type: " + kind);
    }
    ir.ops.push_back(std::move(op));
  }
  if (ir.ops.empty()) throw std::runtime_error("empty graph");
  ir.outputs.push_back(cur);
  return ir;
}

}  // namespace


namespace {

int64_t workspace_for(const OpDef& op, const Plan& plan) {
  if (op.type == "layer_norm") {
    const auto& s = plan.shape[static_cast<size_t>(op.in[0])];
    return numel(s) / s.back() * 8;
  }
  if (op.type == "attention") {
    const auto& q = plan.shape[static_cast<size_t>(op.in[0])];
    return q[0] * q[1] * q[2] * 4;
  }
  return train_workspace_for(op, plan);
}

void check_op(const OpDef& op, const IR& ir, const Plan& plan) {
  auto need = [&](bool c, const std::string& why) {
    if (!c) throw std::runtime_error("operator " + op.type + ": " + why);
  };
  auto shp = [&](int t) -> const std::vector<int64_t>& { return plan.shape[static_cast<size_t>(t)]; };
  auto dt = [&](int t) { return ir.tensors[static_cast<size_t>(t)].dtype; };
  auto bf16 = [&](std::initializer_list<int> ts) {
    for (int x : ts)
      if (x >= 0 && dt(x) != DType::kBFloat16) return false;
    return true;
  };
  // a [rows, heads, D] view read with a token stride stays inside its storage
  auto strided_view_fits = [&](int x, int64_t rows, int64_t row_elems, int64_t stride) {
    if (stride < row_elems || rows <= 0) return false;
    const int r = plan.root[static_cast<size_t>(x)];
    const int64_t first = plan.byte_off[static_cast<size_t>(x)] / SizeOf(dt(x));
    return stride <= (int64_t{1} << 40) && first + (rows - 1) * stride + row_elems <= numel(shp(r));
  };
  const std::string& t = op.type;
  if (t != "linear")
    for (int x : op.in) need(x >= 0, "absent input");
  if (t == "linear") {
    need(op.in.size() >= 2 && op.in.size() <= 4 && op.in[0] >= 0 && op.in[1] >= 0, "needs x and weight (and optionally bias and residual)");
    const auto& x = shp(op.in[0]);
    const auto& w = shp(op.in[1]);
    need(w.size() == 2 && !x.empty() && x.back() == w[1], "weight must be [N, K] with K the last axis of x");
    need(numel(shp(op.out[0])) == numel(x) / w[1] * w[0], "output size mismatch");
    if (op.in.size() > 2 && op.in[2] >= 0) need(numel(shp(op.in[2])) == w[0], "bias must have N elements");
    if (op.in.size() > 3 && op.in[3] >= 0) need(numel(shp(op.in[3])) == numel(shp(op.out[0])), "residual must match the output");
    need(bf16({op.in[0], op.in[1], op.in.size() > 2 ? op.in[2] : -1, op.in.size() > 3 ? op.in[3] : -1, op.out[0]}), "operands must be bf16");
    if (op.out.size() > 1) need(op.out.size() == 2 && bf16({op.out[1]}) && numel(shp(op.out[1])) == numel(shp(op.out[0])), "the stored pre-activation must match the output");
  } else if (t == "matmul") {
    need(op.in.size() == 2 || op.in.size() == 3, "needs two inputs (and optionally the pre-activation whose derivative scales the result)");
    const auto& a = shp(op.in[0]);
    const auto& b = shp(op.in[1]);
    need(a.size() >= 2 && b.size() >= 2, "operands need at least two axes");
    need(bf16({op.in[0], op.in[1], op.in.size() > 2 ? op.in[2] : -1}) && op.out.size() == 1, "bf16 operands, one output");
    if (op.in.size() == 3)
      need(a.size() == 2 && numel(shp(op.in[2])) == numel(shp(op.out[0])) && act_code(attr_str(op, "act_grad", "none")) != 0 && dt(op.out[0]) == DType::kBFloat16,
           "act_grad needs a 2-D left operand, a pre-activation of the output's size and a bf16 output");
    const bool ta = attr_int(op, "ta", 0) != 0, tb = attr_int(op, "tb", 0) != 0;   // ta: the left operand is stored [.., K, M]
    const int64_t K = ta ? a[a.size() - 2] : a.back(), M = ta ? a.back() : a[a.size() - 2];
    const int64_t N = tb ? b[b.size() - 2] : b.back(), Kb = tb ? b.back() : b[b.size() - 2];
    need(K == Kb, "inner dimensions differ");
    const int64_t batch_a = numel(a) / (M * K), batch_b = numel(b) / (N * K);
    need(batch_b == 1 || batch_b == batch_a, "batch dimensions differ");
    need(numel(shp(op.out[0])) == batch_a * M * N, "output size mismatch");
    need(dt(op.out[0]) == DType::kBFloat16 || dt(op.out[0]) == DType::kFloat, "the output must be bf16 or fp32");
    need(attr_int(op, "accumulate", 0) == 0 || dt(op.out[0]) == DType::kFloat, "only fp32 outputs accumulate");
  } else if (t == "layer_norm") {
    need(op.in.size() == 3, "needs x, gamma, beta");
    need(!shp(op.in[0]).empty() && numel(shp(op.in[1])) == shp(op.in[0]).back() && numel(shp(op.in[2])) == shp(op.in[0]).back(), "gamma / beta length");
    need(bf16({op.in[0], op.in[1], op.in[2], op.out[0]}) && numel(shp(op.out[0])) == numel(shp(op.in[0])), "bf16 operands; the output matches the input");
    if (op.out.size() > 1)
      need(op.out.size() == 2 && dt(op.out[1]) == DType::kFloat && numel(shp(op.out[1])) == 2 * numel(shp(op.in[0])) / shp(op.in[0]).back(), "the statistics are two fp32 values per row");
  } else if (t == "embedding") {
    need(op.in.size() == 2 && dt(op.in[0]) == DType::kInt64 && shp(op.in[1]).size() == 2, "needs int64 ids and a [rows, cols] table");
    need(numel(shp(op.out[0])) == numel(shp(op.in[0])) * shp(op.in[1])[1], "output size mismatch");
    need(bf16({op.in[1], op.out[0]}) && op.out.size() == 1, "bf16 table and output");
  } else if (t == "binary") {
    need(op.in.size() == 2, "needs two inputs");
    const int64_t n = numel(shp(op.in[0])), nb = numel(shp(op.in[1]));
    const int64_t mode = attr_int(op, "bmode", 0), cols = attr_int(op, "cols", 1);
    need(n == numel(shp(op.out[0])), "the first operand must have the output's shape");
    need((mode == 0 && nb == n) || (mode == 1 && cols > 0 && nb == cols && n % cols == 0) || (mode == 2 && cols > 0 && nb * cols == n), "broadcast description does not match the shapes");
    need(bf16({op.in[0], op.in[1], op.out[0]}) && op.out.size() == 1, "bf16 operands");
  } else if (t == "unary" || t == "softmax") {
    need(op.in.size() == 1 && op.in[0] >= 0 && op.out.size() == 1 && numel(shp(op.in[0])) == numel(shp(op.out[0])), "shape mismatch");
    need(bf16({op.in[0], op.out[0]}), "bf16 operands");
    if (t == "softmax") need(!shp(op.in[0]).empty() && shp(op.in[0]).back() > 0, "softmax needs a last axis");
  } else if (t == "attention") {
    need(op.in.size() == 3, "needs q, k, v");
    const auto& q = shp(op.in[0]);
    const auto& k = shp(op.in[1]);
    need(q.size() == 4 && k.size() == 4 && shp(op.in[2]) == k && q[0] == k[0] && q[3] == k[3] && q[2] % k[2] == 0, "q [B,Sq,H,D], k / v [B,Sk,Hk,D]");
    need(numel(shp(op.out[0])) == numel(q), "output size mismatch");
    need(bf16({op.in[0], op.in[1], op.in[2], op.out[0]}), "bf16 operands");
    need(strided_view_fits(op.in[0], q[0] * q[1], q[2] * q[3], attr_int(op, "q_stride", q[2] * q[3])) &&
             strided_view_fits(op.in[1], k[0] * k[1], k[2] * k[3], attr_int(op, "kv_stride", k[2] * k[3])) &&
             strided_view_fits(op.in[2], k[0] * k[1], k[2] * k[3], attr_int(op, "kv_stride", k[2] * k[3])),
         "a token stride reaches outside the operand's storage");
    if (op.out.size() > 1) need(op.out.size() == 2 && dt(op.out[1]) == DType::kFloat && numel(shp(op.out[1])) == q[0] * q[1] * q[2], "the log-sum-exp is one fp32 value per (batch, head, query)");
  } else if (t == "copy") {
    need(op.in.size() == 1, "needs one input");
    const auto s = int_list(attr_str(op, "shape", "")), is = int_list(attr_str(op, "in_strides", "")), os = int_list(attr_str(op, "out_strides", ""));
    need(!s.empty() && s.size() <= 5 && is.size() == s.size() && os.size() == s.size(), "shape / in_strides / out_strides of 1..5 axes");
    // bounds of both views
    int64_t in_max = attr_int(op, "in_offset", 0), out_max = attr_int(op, "out_offset", 0);
    const int64_t lim = int64_t{1} << 40;
    need(in_max >= 0 && out_max >= 0 && in_max < lim && out_max < lim && op.out.size() == 1, "negative or absurd offset");
    for (size_t i = 0; i < s.size(); ++i) {
      need(s[i] > 0 && is[i] >= 0 && os[i] >= 0 && s[i] < lim && is[i] < lim && os[i] < lim && numel(s) < lim, "non-positive extent, negative stride or absurd size");
      in_max += (s[i] - 1) * is[i];
      out_max += (s[i] - 1) * os[i];
    }
    need(in_max < numel(shp(op.in[0])) && out_max < numel(shp(op.out[0])), "view reaches outside its tensor");
    need(dt(op.in[0]) == dt(op.out[0]) || attr_int(op, "accumulate", 0) != 0, "dtype mismatch");
    if (attr_int(op, "accumulate", 0) != 0) need(dt(op.in[0]) != DType::kInt64 && dt(op.out[0]) != DType::kInt64, "only bf16 / fp32 views accumulate");
  } else if (!check_train_op(op, ir, plan)) {
    throw std::runtime_error("unknown operator type: " + t);
  }
}

}  // namespace

void Graph::Impl::compile(int64_t rows) {
  auto p = std::make_unique<Plan>();
  p->rows = rows;
  const size_t nt = ir.tensors.size();
  p->shape.resize(nt);
  p->root.resize(nt);
  p->byte_off.assign(nt, 0);
  p->base.assign(nt, nullptr);
  for (size_t i = 0; i < nt; ++i) {
    p->shape[i] = ir.tensors[i].shape;
    for (auto& d : p->shape[i])
      if (d == -1) {
        if (rows <= 0) throw std::runtime_error("the graph has an unbound row count");
        d = rows;
      }
    {
      int64_t total = 1;
      for (auto d : p->shape[i]) {
        if (d < 0 || d > (int64_t{1} << 40) || (d > 0 && total > (int64_t{1} << 40) / d)) throw std::runtime_error("tensor " + std::to_string(i) + ": absurd size");
        total *= d;
      }
      // no single tensor can be larger than the memory of the device (180 GB) or of any host this runs on
      if (total > (int64_t{1} << 38) / SizeOf(ir.tensors[i].dtype)) throw std::runtime_error("tensor " + std::to_string(i) + ": larger than 256 GiB");
    }
    const TensorDef& t = ir.tensors[i];
    if (t.alias_of >= 0) {
      if (t.alias_off < 0) throw std::runtime_error("tensor " + std::to_string(i) + ": negative alias offset");
      const size_t a = static_cast<size_t>(t.alias_of);
      p->root[i] = p->root[a];
      p->byte_off[i] = p->byte_off[a] + t.alias_off * SizeOf(ir.tensors[a].dtype);
      const int r = p->root[i];
      if (p->byte_off[i] + numel(p->shape[i]) * SizeOf(t.dtype) > numel(p->shape[static_cast<size_t>(r)]) * SizeOf(ir.tensors[static_cast<size_t>(r)].dtype))
        throw std::runtime_error("tensor " + std::to_string(i) + ": alias reaches outside its source");
    } else {
      p->root[i] = static_cast<int>(i);
    }
  }
  auto root_bytes = [&](int r) { return numel(p->shape[static_cast<size_t>(r)]) * SizeOf(ir.tensors[static_cast<size_t>(r)].dtype); };
  auto root_kind = [&](int r) { return ir.tensors[static_cast<size_t>(r)].kind; };

  const int n_ops = static_cast<int>(ir.ops.size());
  p->ops.resize(static_cast<size_t>(n_ops));
  // every storage of kind "input" that an operator reads must be handed in by the caller
  {
    std::vector<char> fed(nt, 0);
    for (int t : ir.inputs) fed[static_cast<size_t>(p->root[static_cast<size_t>(t)])] = 1;
    for (const OpDef& op : ir.ops)
      for (int t : op.in)
        if (t >= 0 && root_kind(p->root[static_cast<size_t>(t)]) == 0 && !fed[static_cast<size_t>(p->root[static_cast<size_t>(t)])])
          throw std::runtime_error("operator " + op.type + " reads input tensor " + std::to_string(t) + ", which is not among the graph's inputs");
    for (int t : ir.inputs) {
      const int r = p->root[static_cast<size_t>(t)];
      if (root_kind(r) != 0) throw std::runtime_error("graph input " + std::to_string(t) + " is not a tensor of kind input");
      // the caller hands in exactly this tensor: it has to be the whole storage the operators may read
      if (p->byte_off[static_cast<size_t>(t)] != 0 || numel(p->shape[static_cast<size_t>(t)]) != numel(p->shape[static_cast<size_t>(r)]) ||
          ir.tensors[static_cast<size_t>(t)].dtype != ir.tensors[static_cast<size_t>(r)].dtype)
        throw std::runtime_error("graph input " + std::to_string(t) + " does not cover its whole storage");
    }
  }
  // 1. liveness of activation storages in operator order
  std::vector<int> first(nt, -1), last(nt, -1);
  for (int i = 0; i < n_ops; ++i) {
    const OpDef& op = ir.ops[static_cast<size_t>(i)];
    check_op(op, ir, *p);
    p->ops[static_cast<size_t>(i)].def = &op;
    for (int t : op.in) {
      if (t < 0) continue;
      const int r = p->root[static_cast<size_t>(t)];
      if (root_kind(r) == 2) {
        if (first[static_cast<size_t>(r)] < 0) throw std::runtime_error("operator " + op.type + " reads tensor " + std::to_string(t) + " before it is written");
        last[static_cast<size_t>(r)] = i;
      }
    }
    for (int t : op.out) {
      const int r = p->root[static_cast<size_t>(t)];
      const bool update = op.type == "adamw_update" || op.type == "sgd_update";
      if (update && (root_kind(r) == 1 || root_kind(r) == 3)) continue;   // parameters and optimizer state: persistent, not planned
      if (ir.training && root_kind(r) == 3) continue;                    // gradient accumulators that outlive the call
      if (root_kind(r) != 2) throw std::runtime_error("operator " + op.type + " writes a tensor that is not an activation");
      if (first[static_cast<size_t>(r)] < 0) first[static_cast<size_t>(r)] = i;
      last[static_cast<size_t>(r)] = i;
    }
  }
  for (int t : ir.outputs) {
    const int r = p->root[static_cast<size_t>(t)];
    if (root_kind(r) == 2) {
      if (first[static_cast<size_t>(r)] < 0) throw std::runtime_error("an output is never written");
      last[static_cast<size_t>(r)] = n_ops;   // read back after the last operator
    }
  }
  // Conflicts (read-after-write, write-after-read, write-after-write) between the ranges two operators touch; an edge that
  // a dependency already recorded implies directly is left out.
  auto add_deps = [&](std::vector<std::vector<int>>& deps_out) {
    deps_out.assign(static_cast<size_t>(n_ops), {});
    for (int i = 0; i < n_ops; ++i) {
      const PlannedOp& a = p->ops[static_cast<size_t>(i)];
      std::vector<int>& mine = deps_out[static_cast<size_t>(i)];
      for (int j = i - 1; j >= 0; --j) {
        const PlannedOp& b = p->ops[static_cast<size_t>(j)];
        bool conflict = false;
        for (const Range& w : b.writes) {
          for (const Range& r : a.reads) conflict = conflict || overlaps(w, r);
          for (const Range& r : a.writes) conflict = conflict || overlaps(w, r);
        }
        for (const Range& r : b.reads)
          for (const Range& w : a.writes) conflict = conflict || overlaps(r, w);
        if (!conflict) continue;
        bool implied = false;
        for (int d : mine) {
          const auto& dd = deps_out[static_cast<size_t>(d)];
          if (std::find(dd.begin(), dd.end(), j) != dd.end()) { implied = true; break; }
        }
        if (!implied) mine.push_back(j);   // descending order
      }
    }
  };
  auto virtual_range = [&](int t) {   // a storage as a range of its own, wherever it will live
    const int r = p->root[static_cast<size_t>(t)];
    return Range{(int64_t{1} << 62) + static_cast<int64_t>(r) * (int64_t{1} << 40), std::max<int64_t>(root_bytes(r), 1)};
  };
  // 2. data dependencies (on storages, before any memory is shared) and from them the streams: an operator continues the
  //    chain of its most recent producer that nobody continued yet, else it opens / takes another stream
  for (int i = 0; i < n_ops; ++i) {
    PlannedOp& po = p->ops[static_cast<size_t>(i)];
    for (int t : po.def->in)
      if (t >= 0 && (ir.training || root_kind(p->root[static_cast<size_t>(t)]) != 1)) po.reads.push_back(virtual_range(t));   // inference: parameters never change
    for (int t : po.def->out) po.writes.push_back(virtual_range(t));
  }
  {
    std::vector<std::vector<int>> data_deps;
    add_deps(data_deps);
    std::vector<char> continued(static_cast<size_t>(n_ops), 0);
    int next_stream = 0, used = 0;
    for (int i = 0; i < n_ops; ++i) {
      PlannedOp& a = p->ops[static_cast<size_t>(i)];
      int chosen = -1;
      for (int d : data_deps[static_cast<size_t>(i)])
        if (!continued[static_cast<size_t>(d)]) { chosen = d; break; }
      if (chosen >= 0) {
        a.stream = p->ops[static_cast<size_t>(chosen)].stream;
        continued[static_cast<size_t>(chosen)] = 1;
      } else {
        a.stream = next_stream;
        next_stream = (next_stream + 1) % n_streams;
      }
      used = std::max(used, a.stream + 1);
    }
    p->stats.n_streams_used = used;
  }
  // 3. addresses from the caching allocator, one pool per stream so that sharing memory never ties two streams together:
  //    allocate at the first write (in the pool of the writer's stream), free after the last access
  for (void* al : allocators) ofc_allocator_destroy(al);
  allocators.clear();
  if (device >= 0) check_cuda(cudaSetDevice(device), "cudaSetDevice");
  for (int sidx = 0; sidx < p->stats.n_streams_used; ++sidx) {
    void* al = ofc_allocator_create(device < 0 ? 0 : 1, int64_t{32} << 20);
    if (!al) throw std::runtime_error(std::string("allocator: ") + ofc_last_error());
    allocators.push_back(al);
  }
  auto in_use_now = [&] {
    int64_t total = 0;
    for (void* al : allocators) {
      int64_t reserved = 0, in_use = 0, chunks = 0, free_blocks = 0;
      ofc_allocator_stats(al, &reserved, &in_use, &chunks, &free_blocks);
      total += in_use;
    }
    return total;
  };
  std::vector<std::vector<int>> born(static_cast<size_t>(n_ops)), dies(static_cast<size_t>(n_ops) + 1);
  std::vector<int> pool(nt, 0);
  for (size_t r = 0; r < nt; ++r)
    if (first[r] >= 0) {
      born[static_cast<size_t>(first[r])].push_back(static_cast<int>(r));
      dies[static_cast<size_t>(last[r])].push_back(static_cast<int>(r));
    }
  for (int i = 0; i < n_ops; ++i) {
    PlannedOp& po = p->ops[static_cast<size_t>(i)];
    void* al = allocators[static_cast<size_t>(po.stream)];
    for (int r : born[static_cast<size_t>(i)]) {
      void* ptr = ofc_allocator_alloc(al, std::max<int64_t>(root_bytes(r), 16));
      if (!ptr) throw std::runtime_error(std::string("allocator: ") + ofc_last_error());
      p->base[static_cast<size_t>(r)] = ptr;
      pool[static_cast<size_t>(r)] = po.stream;
      p->stats.activation_bytes += root_bytes(r);
    }
    po.workspace_bytes = workspace_for(*po.def, *p);
    if (po.workspace_bytes < 0 || po.workspace_bytes > (int64_t{1} << 38)) throw std::runtime_error("operator " + po.def->type + ": absurd scratch size");
    if (po.workspace_bytes > 0) {
      po.workspace = ofc_allocator_alloc(al, po.workspace_bytes);
      if (!po.workspace) throw std::runtime_error(std::string("allocator: ") + ofc_last_error());
    }
    p->stats.arena_bytes = std::max(p->stats.arena_bytes, in_use_now());
    // the real ranges, taken while everything this operator touches is still allocated
    auto range_of = [&](int t) {
      const int r = p->root[static_cast<size_t>(t)];
      if (p->base[static_cast<size_t>(r)]) return Range{reinterpret_cast<int64_t>(p->base[static_cast<size_t>(r)]), std::max<int64_t>(root_bytes(r), 1)};
      return virtual_range(t);
    };
    po.reads.clear();
    po.writes.clear();
    for (int t : po.def->in)
      if (t >= 0 && (ir.training || root_kind(p->root[static_cast<size_t>(t)]) != 1)) po.reads.push_back(range_of(t));
    for (int t : po.def->out) po.writes.push_back(range_of(t));
    if (po.workspace) po.writes.push_back(Range{reinterpret_cast<int64_t>(po.workspace), po.workspace_bytes});
    if (po.workspace) ofc_allocator_free(al, po.workspace);
    for (int r : dies[static_cast<size_t>(i)]) ofc_allocator_free(allocators[static_cast<size_t>(pool[static_cast<size_t>(r)])], p->base[static_cast<size_t>(r)]);
  }
  // outputs (dies[n_ops]) stay allocated: they are read after the run
  // 4. the dependencies the scheduler enforces: conflicts on addresses, which cover the data dependencies and add the
  //    ones that memory sharing introduces (a buffer may only be rewritten after the last reader of its previous tenant)
  {
    std::vector<std::vector<int>> deps;
    add_deps(deps);
    for (int i = 0; i < n_ops; ++i) {
      p->ops[static_cast<size_t>(i)].deps = deps[static_cast<size_t>(i)];
      p->stats.n_dependencies += static_cast<int64_t>(deps[static_cast<size_t>(i)].size());
    }
  }
  p->stats.n_ops = n_ops;
  p->stats.n_tensors = static_cast<int64_t>(nt);
  // 5. runtime objects
  if (device >= 0) {
    while (static_cast<int>(streams.size()) < n_streams) {
      cudaStream_t s;
      check_cuda(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreate");
      streams.push_back(s);
    }
    while (static_cast<int>(events.size()) < n_ops) {
      cudaEvent_t e;
      check_cuda(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
      events.push_back(e);
    }
  }
  if (!executor) {
    executor = ofc_executor_create(n_streams);
    if (!executor) throw std::runtime_error(std::string("executor: ") + ofc_last_error());
  }
  for (int k = 0; k < 4; ++k) {
    if (graph_exec[k]) cudaGraphExecDestroy(graph_exec[k]);
    graph_exec[k] = nullptr;
    runs_of_plan[k] = 0;
  }
  graph_replays = 0;
  input_bufs.clear();
  if (device >= 0) {
    for (int t : ir.inputs)
      input_bufs.push_back(storage_alloc(static_cast<size_t>(numel(p->shape[static_cast<size_t>(t)]) * SizeOf(ir.tensors[static_cast<size_t>(t)].dtype)), device));
    if (!fork_event) check_cuda(cudaEventCreateWithFlags(&fork_event, cudaEventDisableTiming), "cudaEventCreate");
    while (static_cast<int>(join_events.size()) < n_streams) {
      cudaEvent_t e;
      check_cuda(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate");
      join_events.push_back(e);
    }
    const char* off = std::getenv("ONEFLOW_API_CUDA_GRAPH");
    graph_disabled = off && off[0] == '0';
  }
  plan = std::move(p);
}

// ------------------------------------------------------------------------------------------------ operators on the GPU
void Graph::Impl::run_op_device(const PlannedOp& p, cudaStream_t s) {
  if (run_train_op_device(p, s)) return;
  const OpDef& op = *p.def;
  auto shp = [&](int t) -> const std::vector<int64_t>& { return plan->shape[static_cast<size_t>(t)]; };
  auto ok = [&](int rc) {
    if (rc != 0) throw std::runtime_error(op.type + ": " + ofb_last_error());
  };
  const std::string& t = op.type;
  if (t == "linear") {
    const auto& w = shp(op.in[1]);
    const int64_t K = w[1], N = w[0], M = numel(shp(op.in[0])) / K;
    OfbGemmArgs a;
    std::memset(&a, 0, sizeof(a));
    a.A = addr(op.in[0]); a.lda = K;
    a.B = addr(op.in[1]); a.ldb = K;
    a.C = addr(op.out[0]); a.ldc = N;
    a.bias = op.in.size() > 2 && op.in[2] >= 0 ? addr(op.in[2]) : nullptr;
    if (op.in.size() > 3 && op.in[3] >= 0) { a.residual = addr(op.in[3]); a.ldr = N; }
    a.M = static_cast<int>(M); a.N = static_cast<int>(N); a.K = static_cast<int>(K);
    a.act = act_code(attr_str(op, "act", "none"));
    if (op.out.size() > 1) { a.aux_out = addr(op.out[1]); a.ld_aux = N; }   // the pre-activation, kept for the backward pass
    a.alpha = 1.f;
    ok(ofb_gemm_bf16(&a, s));
  } else if (t == "matmul") {
    const auto& as = shp(op.in[0]);
    const auto& bs = shp(op.in[1]);
    const bool ta = attr_int(op, "ta", 0) != 0, tb = attr_int(op, "tb", 0) != 0;
    const int64_t M = ta ? as.back() : as[as.size() - 2], K = ta ? as[as.size() - 2] : as.back(), N = tb ? bs[bs.size() - 2] : bs.back();
    const int64_t batch = numel(as) / (M * K), batch_b = numel(bs) / (N * K);
    const bool wide = ir.tensors[static_cast<size_t>(op.out[0])].dtype == DType::kFloat;
    for (int64_t b = 0; b < batch; ++b) {
      OfbGemmArgs a;
      std::memset(&a, 0, sizeof(a));
      a.A = static_cast<char*>(addr(op.in[0])) + b * M * K * 2;
      a.lda = ta ? M : K;
      a.a_mn_major = ta ? 1 : 0;
      a.B = static_cast<char*>(addr(op.in[1])) + (batch_b == 1 ? 0 : b) * N * K * 2;
      a.ldb = tb ? K : N;
      a.b_mn_major = tb ? 0 : 1;
      a.C = static_cast<char*>(addr(op.out[0])) + b * M * N * (wide ? 4 : 2); a.ldc = N;
      a.out_fp32 = wide ? 1 : 0;
      a.accumulate = attr_int(op, "accumulate", 0) != 0 ? 1 : 0;
      if (op.in.size() > 2) { a.aux_in = addr(op.in[2]); a.ld_aux = N; a.act = act_code(attr_str(op, "act_grad", "none")); }   // result *= act'(pre-activation)
      a.M = static_cast<int>(M); a.N = static_cast<int>(N); a.K = static_cast<int>(K);
      a.alpha = static_cast<float>(attr_float(op, "alpha", 1.0));
      ok(ofb_gemm_bf16(&a, s));
    }
  } else if (t == "layer_norm") {
    const auto& x = shp(op.in[0]);
    const int64_t cols = x.back(), rows = numel(x) / cols;
    float* mean = op.out.size() > 1 ? static_cast<float*>(addr(op.out[1])) : static_cast<float*>(p.workspace);   // kept for the backward pass
    ok(ofb_layer_norm_fwd(addr(op.in[0]), addr(op.in[1]), addr(op.in[2]), addr(op.out[0]), mean, mean + rows, static_cast<int>(rows),
                          static_cast<int>(cols), static_cast<float>(attr_float(op, "eps", 1e-5)), s));
  } else if (t == "embedding") {
    const auto& tb = shp(op.in[1]);
    ok(ofb_graph_gather_rows(static_cast<const long long*>(addr(op.in[0])), addr(op.in[1]), addr(op.out[0]), numel(shp(op.in[0])),
                             static_cast<int>(tb[1]), tb[0], s));
  } else if (t == "binary") {
    ok(ofb_graph_binary(addr(op.in[0]), addr(op.in[1]), addr(op.out[0]), numel(shp(op.in[0])), attr_int(op, "cols", 1),
                        static_cast<int>(attr_int(op, "bmode", 0)), static_cast<int>(attr_int(op, "fn", 0)), s));
  } else if (t == "unary") {
    ok(ofb_graph_unary(addr(op.in[0]), addr(op.out[0]), numel(shp(op.in[0])), static_cast<int>(attr_int(op, "fn", 0)),
                       static_cast<float>(attr_float(op, "alpha", 1.0)), s));
  } else if (t == "softmax") {
    const auto& x = shp(op.in[0]);
    const int64_t cols = x.back(), rows = numel(x) / cols;
    ok(ofb_softmax_fwd(addr(op.in[0]), nullptr, nullptr, 0, addr(op.out[0]), nullptr, rows, static_cast<int>(cols), 0, 0, 0,
                       static_cast<float>(attr_float(op, "scale", 1.0)), 0.f, 1.f, s));
  } else if (t == "attention") {
    const auto& q = shp(op.in[0]);
    const auto& k = shp(op.in[1]);
    const int64_t qs = attr_int(op, "q_stride", q[2] * q[3]), ks = attr_int(op, "kv_stride", k[2] * k[3]);
    float* lse = op.out.size() > 1 ? static_cast<float*>(addr(op.out[1])) : static_cast<float*>(p.workspace);   // kept for the backward pass
    ok(ofb_fmha_fwd_ex(addr(op.in[0]), addr(op.in[1]), addr(op.in[2]), qs, ks, addr(op.out[0]), lse, nullptr,
                       static_cast<int>(q[0]), static_cast<int>(q[1]), static_cast<int>(k[1]), static_cast<int>(q[2]), static_cast<int>(k[2]),
                       static_cast<int>(q[3]), static_cast<int>(attr_int(op, "causal", 0)),
                       static_cast<float>(attr_float(op, "scale", 1.0 / std::sqrt(static_cast<double>(q[3])))), 0.f, 0ull, 0u, s));
  } else if (t == "copy") {
    const auto sh = int_list(attr_str(op, "shape", "")), is = int_list(attr_str(op, "in_strides", "")), os = int_list(attr_str(op, "out_strides", ""));
    std::vector<long long> a(sh.begin(), sh.end()), b(is.begin(), is.end()), c(os.begin(), os.end());
    ok(ofb_graph_strided_copy(addr(op.in[0]), addr(op.out[0]), static_cast<int>(a.size()), a.data(), b.data(), attr_int(op, "in_offset", 0),
                              c.data(), attr_int(op, "out_offset", 0), static_cast<int>(SizeOf(ir.tensors[static_cast<size_t>(op.in[0])].dtype)), s));
  }
}

// ------------------------------------------------------------------------------------------------ operators on the host
namespace {

inline float ldb(const void* p, int64_t i) { return from_bf16(static_cast<const uint16_t*>(p)[i]); }
inline void stb(void* p, int64_t i, float v) { static_cast<uint16_t*>(p)[i] = to_bf16(v); }

float host_unary(float x, int fn, float alpha) {
  switch (fn) {
    case 0: return x * alpha;
    case 1: return 0.5f * x * (1.f + std::erf(x * 0.7071067811865476f));
    case 2: return 0.5f * x * (1.f + std::tanh(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    case 3: return x > 0.f ? x : 0.f;
    case 4: return std::tanh(x);
    case 5: return 1.f / (1.f + std::exp(-x));
    case 6: return x / (1.f + std::exp(-x));
    case 7: return x + alpha;
    case 8: return std::exp(x);
    case 9: return 1.f / std::sqrt(x);
    case 10: return x * x;
    default: return x;
  }
}
float host_binary(float a, float b, int op) {
  switch (op) {
    case 0: return a + b;
    case 1: return a - b;
    case 2: return a * b;
    case 3: return a / b;
    case 4: return a > b ? a : b;
    default: return a < b ? a : b;
  }
}

}  // namespace

void Graph::Impl::run_op_host(const PlannedOp& p) {
  if (run_train_op_host(p)) return;
  const OpDef& op = *p.def;
  auto shp = [&](int t) -> const std::vector<int64_t>& { return plan->shape[static_cast<size_t>(t)]; };
  const std::string& t = op.type;
  if (t == "linear") {
    const auto& w = shp(op.in[1]);
    const int64_t K = w[1], N = w[0], M = numel(shp(op.in[0])) / K;
    const void *x = addr(op.in[0]), *wt = addr(op.in[1]);
    const void* bias = op.in.size() > 2 && op.in[2] >= 0 ? addr(op.in[2]) : nullptr;
    const void* res = op.in.size() > 3 && op.in[3] >= 0 ? addr(op.in[3]) : nullptr;
    const int act = act_code(attr_str(op, "act", "none"));
    void* y = addr(op.out[0]);
    std::vector<float> xr(static_cast<size_t>(K));
    for (int64_t m = 0; m < M; ++m) {
      for (int64_t k = 0; k < K; ++k) xr[static_cast<size_t>(k)] = ldb(x, m * K + k);
      for (int64_t n = 0; n < N; ++n) {
        float acc = 0.f;
        for (int64_t k = 0; k < K; ++k) acc += xr[static_cast<size_t>(k)] * ldb(wt, n * K + k);
        if (bias) acc += ldb(bias, n);
        if (op.out.size() > 1) stb(addr(op.out[1]), m * N + n, acc);   // the pre-activation, kept for the backward pass
        if (act) acc = host_unary(acc, act, 1.f);
        if (res) acc += ldb(res, m * N + n);
        stb(y, m * N + n, acc);
      }
    }
  } else if (t == "matmul") {
    const auto& as = shp(op.in[0]);
    const auto& bs = shp(op.in[1]);
    const bool ta = attr_int(op, "ta", 0) != 0, tb = attr_int(op, "tb", 0) != 0;
    const int64_t M = ta ? as.back() : as[as.size() - 2], K = ta ? as[as.size() - 2] : as.back(), N = tb ? bs[bs.size() - 2] : bs.back();
    const int64_t batch = numel(as) / (M * K), batch_b = numel(bs) / (N * K);
    const float alpha = static_cast<float>(attr_float(op, "alpha", 1.0));
    const bool wide = ir.tensors[static_cast<size_t>(op.out[0])].dtype == DType::kFloat, accumulate = attr_int(op, "accumulate", 0) != 0;
    const void *a = addr(op.in[0]), *b = addr(op.in[1]);
    void* y = addr(op.out[0]);
    for (int64_t bi = 0; bi < batch; ++bi) {
      const int64_t ao = bi * M * K, bo = (batch_b == 1 ? 0 : bi) * N * K, yo = bi * M * N;
      for (int64_t m = 0; m < M; ++m)
        for (int64_t n = 0; n < N; ++n) {
          float acc = 0.f;
          for (int64_t k = 0; k < K; ++k)
            acc += (ta ? ldb(a, ao + k * M + m) : ldb(a, ao + m * K + k)) * (tb ? ldb(b, bo + n * K + k) : ldb(b, bo + k * N + n));
          if (wide) {
            float* yf = static_cast<float*>(y) + yo + m * N + n;
            *yf = (accumulate ? *yf : 0.f) + acc * alpha;
          } else if (op.in.size() > 2) {
            stb(y, yo + m * N + n, acc * alpha * host_unary_grad(ldb(addr(op.in[2]), yo + m * N + n), act_code(attr_str(op, "act_grad", "none")), 1.f));
          } else {
            stb(y, yo + m * N + n, acc * alpha);
          }
        }
    }
  } else if (t == "layer_norm") {
    const auto& x = shp(op.in[0]);
    const int64_t cols = x.back(), rows = numel(x) / cols;
    const float eps = static_cast<float>(attr_float(op, "eps", 1e-5));
    const void *xp = addr(op.in[0]), *g = addr(op.in[1]), *b = addr(op.in[2]);
    void* y = addr(op.out[0]);
    for (int64_t r = 0; r < rows; ++r) {
      double mean = 0, var = 0;
      for (int64_t c = 0; c < cols; ++c) mean += ldb(xp, r * cols + c);
      mean /= static_cast<double>(cols);
      for (int64_t c = 0; c < cols; ++c) {
        const double d = ldb(xp, r * cols + c) - mean;
        var += d * d;
      }
      const float rstd = 1.f / std::sqrt(static_cast<float>(var / static_cast<double>(cols)) + eps);
      if (op.out.size() > 1) {   // kept for the backward pass
        float* st = static_cast<float*>(addr(op.out[1]));
        st[r] = static_cast<float>(mean);
        st[rows + r] = rstd;
      }
      for (int64_t c = 0; c < cols; ++c)
        stb(y, r * cols + c, (ldb(xp, r * cols + c) - static_cast<float>(mean)) * rstd * ldb(g, c) + ldb(b, c));
    }
  } else if (t == "embedding") {
    const auto& tb = shp(op.in[1]);
    const int64_t n = numel(shp(op.in[0])), cols = tb[1];
    const int64_t* ids = static_cast<const int64_t*>(addr(op.in[0]));
    const uint16_t* table = static_cast<const uint16_t*>(addr(op.in[1]));
    uint16_t* y = static_cast<uint16_t*>(addr(op.out[0]));
    for (int64_t i = 0; i < n; ++i) {
      if (ids[i] >= 0 && ids[i] < tb[0]) std::memcpy(y + i * cols, table + ids[i] * cols, static_cast<size_t>(cols) * 2);
      else std::memset(y + i * cols, 0, static_cast<size_t>(cols) * 2);
    }
  } else if (t == "binary") {
    const int64_t n = numel(shp(op.in[0])), cols = attr_int(op, "cols", 1);
    const int mode = static_cast<int>(attr_int(op, "bmode", 0)), fn = static_cast<int>(attr_int(op, "fn", 0));
    const void *a = addr(op.in[0]), *b = addr(op.in[1]);
    void* y = addr(op.out[0]);
    for (int64_t i = 0; i < n; ++i) stb(y, i, host_binary(ldb(a, i), ldb(b, mode == 0 ? i : (mode == 1 ? i % cols : i / cols)), fn));
  } else if (t == "unary") {
    const int64_t n = numel(shp(op.in[0]));
    const int fn = static_cast<int>(attr_int(op, "fn", 0));
    const float alpha = static_cast<float>(attr_float(op, "alpha", 1.0));
    const void* x = addr(op.in[0]);
    void* y = addr(op.out[0]);
    for (int64_t i = 0; i < n; ++i) stb(y, i, host_unary(ldb(x, i), fn, alpha));
  } else if (t == "softmax") {
    const auto& x = shp(op.in[0]);
    const int64_t cols = x.back(), rows = numel(x) / cols;
    const float scale = static_cast<float>(attr_float(op, "scale", 1.0));
    const void* xp = addr(op.in[0]);
    void* y = addr(op.out[0]);
    std::vector<float> e(static_cast<size_t>(cols));
    for (int64_t r = 0; r < rows; ++r) {
      float mx = -INFINITY, sum = 0.f;
      for (int64_t c = 0; c < cols; ++c) mx = std::max(mx, ldb(xp, r * cols + c) * scale);
      for (int64_t c = 0; c < cols; ++c) sum += (e[static_cast<size_t>(c)] = std::exp(ldb(xp, r * cols + c) * scale - mx));
      for (int64_t c = 0; c < cols; ++c) stb(y, r * cols + c, e[static_cast<size_t>(c)] / sum);
    }
  } else if (t == "attention") {
    const auto& q = shp(op.in[0]);
    const auto& k = shp(op.in[1]);
    const int64_t B = q[0], Sq = q[1], H = q[2], D = q[3], Sk = k[1], Hk = k[2];
    const int64_t qs = attr_int(op, "q_stride", H * D), ks = attr_int(op, "kv_stride", Hk * D);
    const bool causal = attr_int(op, "causal", 0) != 0;
    const float scale = static_cast<float>(attr_float(op, "scale", 1.0 / std::sqrt(static_cast<double>(D))));
    const void *qp = addr(op.in[0]), *kp = addr(op.in[1]), *vp = addr(op.in[2]);
    void* y = addr(op.out[0]);
    std::vector<float> sc(static_cast<size_t>(Sk)), acc(static_cast<size_t>(D));
    for (int64_t b = 0; b < B; ++b)
      for (int64_t h = 0; h < H; ++h) {
        const int64_t hk = h / (H / Hk);
        for (int64_t i = 0; i < Sq; ++i) {
          const int64_t vis = causal ? std::min<int64_t>(Sk, i + (Sk - Sq) + 1) : Sk;
          float mx = -INFINITY;
          for (int64_t j = 0; j < vis; ++j) {
            float s = 0.f;
            for (int64_t d = 0; d < D; ++d) s += ldb(qp, (b * Sq + i) * qs + h * D + d) * ldb(kp, (b * Sk + j) * ks + hk * D + d);
            sc[static_cast<size_t>(j)] = s * scale;
            mx = std::max(mx, s * scale);
          }
          float sum = 0.f;
          std::fill(acc.begin(), acc.end(), 0.f);
          for (int64_t j = 0; j < vis; ++j) {
            const float e = std::exp(sc[static_cast<size_t>(j)] - mx);
            sum += e;
            for (int64_t d = 0; d < D; ++d) acc[static_cast<size_t>(d)] += e * ldb(vp, (b * Sk + j) * ks + hk * D + d);
          }
          for (int64_t d = 0; d < D; ++d) stb(y, ((b * Sq + i) * H + h) * D + d, vis > 0 ? acc[static_cast<size_t>(d)] / sum : 0.f);
          if (op.out.size() > 1) static_cast<float*>(addr(op.out[1]))[(b * H + h) * Sq + i] = vis > 0 ? mx + std::log(sum) : 0.f;   // kept for the backward pass
        }
      }
  } else if (t == "copy") {
    const auto sh = int_list(attr_str(op, "shape", "")), is = int_list(attr_str(op, "in_strides", "")), os = int_list(attr_str(op, "out_strides", ""));
    const int64_t esz = SizeOf(ir.tensors[static_cast<size_t>(op.in[0])].dtype);
    const char* x = static_cast<const char*>(addr(op.in[0]));
    char* y = static_cast<char*>(addr(op.out[0]));
    const int64_t n = numel(sh), io = attr_int(op, "in_offset", 0), oo = attr_int(op, "out_offset", 0);
    for (int64_t i = 0; i < n; ++i) {
      int64_t r = i, in = io, out = oo;
      for (int d = static_cast<int>(sh.size()) - 1; d >= 0; --d) {
        const int64_t c = r % sh[static_cast<size_t>(d)];
        r /= sh[static_cast<size_t>(d)];
        in += c * is[static_cast<size_t>(d)];
        out += c * os[static_cast<size_t>(d)];
      }
      std::memcpy(y + out * esz, x + in * esz, static_cast<size_t>(esz));
    }
  }
}

// ------------------------------------------------------------------------------------------------ execution
namespace {
struct TaskArg {
  Graph::Impl* impl;
  int index;
};
void task_trampoline(void* arg) {
  auto* a = static_cast<TaskArg*>(arg);
  a->impl->run_op(a->index);
}
}  // namespace

void Graph::Impl::run_op(int index) {
  if (failed()) return;   // an earlier operator failed: let the rest drain
  const PlannedOp& p = plan->ops[static_cast<size_t>(index)];
  try {
    if (device < 0) {
      if (op_enabled(*p.def)) run_op_host(p);
      return;
    }
    check_cuda(cudaSetDevice(device), "cudaSetDevice");
    cudaStream_t s = streams[static_cast<size_t>(p.stream)];
    // the scheduler ran every dependency's host side already, so its event has been recorded
    for (int d : p.deps)
      if (plan->ops[static_cast<size_t>(d)].stream != p.stream) check_cuda(cudaStreamWaitEvent(s, events[static_cast<size_t>(d)], 0), "cudaStreamWaitEvent");
    if (op_enabled(*p.def)) run_op_device(p, s);
    check_cuda(cudaEventRecord(events[static_cast<size_t>(index)], s), "cudaEventRecord");
  } catch (const std::exception& e) {
    fail(e.what());
  }
}

// Records the plan into a CUDA graph: stream 0 is the origin, the other streams fork from it and join it again, every
// operator is launched on its plan stream after waiting for the events of its cross-stream dependencies. Returns false (and
// leaves the scheduler path in charge) if anything in the plan cannot be captured.
bool Graph::Impl::capture_plan() {
  cudaStream_t s0 = streams[0];
  std::string why;
  auto give_up = [&](const std::string& reason) {
    std::fprintf(stderr, "oneflow_api: the plan is not replayed as a CUDA graph (%s); it keeps running through the scheduler\n", reason.c_str());
    return false;
  };
  cudaError_t rc = cudaStreamBeginCapture(s0, cudaStreamCaptureModeThreadLocal);
  if (rc != cudaSuccess) {
    cudaGetLastError();
    return give_up(std::string("cudaStreamBeginCapture: ") + cudaGetErrorString(rc));
  }
  bool ok = true;
  try {
    check_cuda(cudaEventRecord(fork_event, s0), "cudaEventRecord");
    for (size_t s = 1; s < streams.size(); ++s) check_cuda(cudaStreamWaitEvent(streams[s], fork_event, 0), "cudaStreamWaitEvent");
    for (size_t i = 0; i < plan->ops.size(); ++i) {
      const PlannedOp& p = plan->ops[i];
      cudaStream_t s = streams[static_cast<size_t>(p.stream)];
      for (int d : p.deps)
        if (plan->ops[static_cast<size_t>(d)].stream != p.stream) check_cuda(cudaStreamWaitEvent(s, events[static_cast<size_t>(d)], 0), "cudaStreamWaitEvent");
      if (op_enabled(*p.def)) run_op_device(p, s);
      check_cuda(cudaEventRecord(events[i], s), "cudaEventRecord");
    }
    for (size_t s = 1; s < streams.size(); ++s) {
      check_cuda(cudaEventRecord(join_events[s], streams[s]), "cudaEventRecord");
      check_cuda(cudaStreamWaitEvent(s0, join_events[s], 0), "cudaStreamWaitEvent");
    }
  } catch (const std::exception& e) {
    ok = false;
    why = e.what();
  }
  cudaGraph_t g = nullptr;
  rc = cudaStreamEndCapture(s0, &g);
  if (rc != cudaSuccess || !g) {
    cudaGetLastError();
    return give_up(why.empty() ? std::string("cudaStreamEndCapture: ") + cudaGetErrorString(rc) : why);
  }
  if (ok) {
    rc = cudaGraphInstantiate(&graph_exec[call_kind], g, 0);
    if (rc != cudaSuccess) {
      cudaGetLastError();
      graph_exec[call_kind] = nullptr;
      ok = false;
      why = std::string("cudaGraphInstantiate: ") + cudaGetErrorString(rc);
    }
  }
  cudaGraphDestroy(g);
  if (!ok || !graph_exec[call_kind]) return give_up(why);
  return true;
}

namespace {
std::shared_ptr<Graph::Impl> load_impl(const std::string& dir, int device, int n_streams, const TrainOptions* train) {
  std::ifstream f(dir + "/graph.txt");
  if (!f) throw std::runtime_error("cannot open " + dir + "/graph.txt");
  std::string line;
  std::getline(f, line);
  auto impl = std::make_shared<Graph::Impl>();
  {
    std::ifstream whole(dir + "/graph.txt", std::ios::binary);
    std::ostringstream text;
    text << whole.rdbuf();
    impl->graph_text = text.str();
  }
  impl->dir = dir;
  impl->device = device;
  impl->n_streams = std::max(1, std::min(n_streams, 16));
  if (line.rfind("oneflow_b200 graph v2", 0) == 0) impl->ir = parse_v2(f);
  else if (line.rfind("oneflow_b200 inference graph v1", 0) == 0) impl->ir = parse_v1(f);
  else throw std::runtime_error("not an exported graph: " + dir);
  if (train) {
    // the forward graph is compiled once on its own first: that validates every operator (shapes, dtypes, views) before the
    // differentiation pass indexes into them
    if (impl->ir.dynamic_rows) throw std::runtime_error("training graph: export with static shapes (export_graph), not the layer-list form");
    impl->compile(0);
    append_training_ops(impl->ir, *train);
    impl->train = *train;
    if (device >= 0) {
      check_cuda(cudaSetDevice(device), "cudaSetDevice");
      check_cuda(cudaMalloc(&impl->step_scalars, 8 * sizeof(float)), "cudaMalloc");
      check_cuda(cudaMallocHost(&impl->step_scalars_host, 8 * sizeof(float)), "cudaMallocHost");
    }
  }
  impl->ir.pass_report = run_graph_passes(impl->ir);
  if (const char* dump_to = std::getenv("ONEFLOW_API_DUMP_IR")) {   // the graph as the plan compiler is about to see it
    std::ofstream out(dump_to, std::ios::trunc);
    out << ir_to_text(impl->ir);
  }
  // parameters
  impl->params.resize(impl->ir.tensors.size());
  for (size_t i = 0; i < impl->ir.tensors.size(); ++i) {
    const TensorDef& t = impl->ir.tensors[i];
    if (t.kind != 1 || t.alias_of >= 0) continue;
    const size_t bytes = static_cast<size_t>(numel(t.shape) * SizeOf(t.dtype));
    std::ifstream pf(dir + "/" + t.file, std::ios::binary);
    if (!pf) throw std::runtime_error("cannot open " + dir + "/" + t.file);
    pf.seekg(0, std::ios::end);
    if (static_cast<int64_t>(pf.tellg()) != static_cast<int64_t>(bytes))
      throw std::runtime_error(t.file + " holds " + std::to_string(static_cast<int64_t>(pf.tellg())) + " bytes, the graph declares " + std::to_string(bytes));
    pf.seekg(0, std::ios::beg);
    std::vector<char> host(bytes);
    pf.read(host.data(), static_cast<std::streamsize>(bytes));
    if (static_cast<size_t>(pf.gcount()) != bytes) throw std::runtime_error("short read: " + t.file);
    impl->params[i] = storage_alloc(bytes, device);
    copy_in(impl->params[i].get(), host.data(), bytes, device);
    // optimizer state that starts as a copy of this parameter (fp32 master weights)
    for (size_t j = 0; j < impl->ir.tensors.size(); ++j) {
      const TensorDef& st = impl->ir.tensors[j];
      if (st.kind != 3 || st.init_from != static_cast<int>(i)) continue;
      const size_t n = static_cast<size_t>(numel(t.shape));
      std::vector<float> wide(n);
      for (size_t k = 0; k < n; ++k) wide[k] = from_bf16(reinterpret_cast<const uint16_t*>(host.data())[k]);
      impl->params[j] = storage_alloc(n * 4, device);
      copy_in(impl->params[j].get(), wide.data(), n * 4, device);
    }
  }
  for (size_t j = 0; j < impl->ir.tensors.size(); ++j) {
    const TensorDef& st = impl->ir.tensors[j];
    if (st.kind != 3 || st.init_from >= 0) continue;
    const size_t bytes = static_cast<size_t>(numel(st.shape) * SizeOf(st.dtype));
    std::vector<char> zeros(bytes, 0);
    impl->params[j] = storage_alloc(bytes, device);
    copy_in(impl->params[j].get(), zeros.data(), bytes, device);
  }
  if (!impl->ir.dynamic_rows) impl->compile(0);
  return impl;
}
}  // namespace

Graph Graph::Load(const std::string& dir, int device, int n_streams) {
  Graph g;
  g.impl_ = load_impl(dir, device, n_streams, nullptr);
  return g;
}

Graph Graph::LoadTraining(const std::string& dir, const TrainOptions& options, int device, int n_streams) {
  Graph g;
  g.impl_ = load_impl(dir, device, n_streams, &options);
  return g;
}

int Graph::num_parameters() const { return static_cast<int>(impl_->ir.trainable.size()); }
std::string Graph::parameter_name(int i) const { return impl_->ir.tensors[static_cast<size_t>(impl_->ir.trainable.at(static_cast<size_t>(i)))].name; }
int64_t Graph::parameter_numel(int i) const { return numel(impl_->ir.tensors[static_cast<size_t>(impl_->ir.trainable.at(static_cast<size_t>(i)))].shape); }
std::vector<float> Graph::parameter(int i) const {
  std::lock_guard<std::mutex> g(impl_->run_mu);
  const int m = impl_->ir.masters.at(static_cast<size_t>(i));
  const size_t n = static_cast<size_t>(numel(impl_->ir.tensors[static_cast<size_t>(m)].shape));
  std::vector<float> out(n);
  if (impl_->device >= 0) check_cuda(cudaSetDevice(impl_->device), "cudaSetDevice");
  copy_out(out.data(), impl_->params[static_cast<size_t>(m)].get(), n * 4, impl_->device);
  return out;
}
void Graph::set_learning_rate(float lr) {
  std::lock_guard<std::mutex> g(impl_->run_mu);
  impl_->train.lr = lr;
}
void Graph::set_lr_schedule(const std::string& kind, int64_t warmup_steps, int64_t decay_steps, float min_lr_ratio) {
  if (kind != "constant" && kind != "cosine" && kind != "linear") throw std::runtime_error("lr schedule must be \"constant\", \"cosine\" or \"linear\"");
  if (warmup_steps < 0 || decay_steps < 0 || min_lr_ratio < 0.f || min_lr_ratio > 1.f) throw std::runtime_error("lr schedule: negative step count or ratio outside [0, 1]");
  std::lock_guard<std::mutex> g(impl_->run_mu);
  impl_->train.lr_schedule = kind;
  impl_->train.warmup_steps = warmup_steps;
  impl_->train.decay_steps = decay_steps;
  impl_->train.min_lr_ratio = min_lr_ratio;
}
float Graph::learning_rate() const {
  std::lock_guard<std::mutex> g(impl_->run_mu);
  return impl_->scheduled_lr(impl_->train_steps + 1);
}
void Graph::set_seed(uint64_t seed) {
  std::lock_guard<std::mutex> g(impl_->run_mu);
  impl_->train.seed = seed;
  if (impl_->device >= 0) check_cuda(cudaSetDevice(impl_->device), "cudaSetDevice");
  for (int k = 0; k < 4; ++k) {   // the seed is a launch argument of the recorded dropout kernels: record again
    if (impl_->graph_exec[k]) cudaGraphExecDestroy(impl_->graph_exec[k]);
    impl_->graph_exec[k] = nullptr;
  }
}
int64_t Graph::steps() const {
  std::lock_guard<std::mutex> g(impl_->run_mu);
  return impl_->train_steps;
}
std::string Graph::dump() const { return ir_to_text(impl_->ir); }

namespace {
constexpr uint64_t kTrainStateMagic = 0x31545354464f4eull;   // "NOFTST1"
void write_file(const std::string& path, const void* data, size_t bytes) {
  std::ofstream f(path, std::ios::binary | std::ios::trunc);
  if (!f) throw std::runtime_error("cannot write " + path);
  f.write(static_cast<const char*>(data), static_cast<std::streamsize>(bytes));
  if (!f) throw std::runtime_error("short write: " + path);
}
}  // namespace

void Graph::Save(const std::string& dir) const {
  Impl& im = *impl_;
  std::lock_guard<std::mutex> g(im.run_mu);
  if (im.device >= 0) check_cuda(cudaSetDevice(im.device), "cudaSetDevice");
  write_file(dir + "/graph.txt", im.graph_text.data(), im.graph_text.size());
  std::vector<char> host;
  for (size_t i = 0; i < im.ir.tensors.size(); ++i) {
    const TensorDef& t = im.ir.tensors[i];
    if (t.kind != 1 || t.alias_of >= 0) continue;
    host.resize(static_cast<size_t>(numel(t.shape) * SizeOf(t.dtype)));
    copy_out(host.data(), im.params[i].get(), host.size(), im.device);
    write_file(dir + "/" + t.file, host.data(), host.size());
  }
  if (!im.ir.training) return;
  if (im.micro_step != 0) throw std::runtime_error("Save: " + std::to_string(im.micro_step) + " micro-batches of the running optimizer step are accumulated; save between steps");
  // train_state.bin: magic, steps, number of state tensors, then per state tensor (in IR order) its length and fp32 data
  std::vector<char> blob;
  auto put = [&](const void* p, size_t n) { blob.insert(blob.end(), static_cast<const char*>(p), static_cast<const char*>(p) + n); };
  uint64_t n_state = 0;
  for (const TensorDef& t : im.ir.tensors) n_state += t.kind == 3 ? 1 : 0;
  const uint64_t steps = static_cast<uint64_t>(im.train_steps);
  put(&kTrainStateMagic, 8);
  put(&steps, 8);
  put(&n_state, 8);
  for (size_t i = 0; i < im.ir.tensors.size(); ++i) {
    const TensorDef& t = im.ir.tensors[i];
    if (t.kind != 3) continue;
    const uint64_t n = static_cast<uint64_t>(numel(t.shape));
    host.resize(n * 4);
    copy_out(host.data(), im.params[i].get(), host.size(), im.device);
    put(&n, 8);
    put(host.data(), host.size());
  }
  write_file(dir + "/train_state.bin", blob.data(), blob.size());
}

void Graph::Restore(const std::string& dir) {
  Impl& im = *impl_;
  std::lock_guard<std::mutex> g(im.run_mu);
  if (!im.ir.training) throw std::runtime_error("Restore: not a training graph");
  std::ifstream f(dir + "/train_state.bin", std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + dir + "/train_state.bin");
  uint64_t magic = 0, steps = 0, n_state = 0;
  f.read(reinterpret_cast<char*>(&magic), 8);
  f.read(reinterpret_cast<char*>(&steps), 8);
  f.read(reinterpret_cast<char*>(&n_state), 8);
  if (!f || magic != kTrainStateMagic) throw std::runtime_error("train_state.bin: not a training state file");
  uint64_t have = 0;
  for (const TensorDef& t : im.ir.tensors) have += t.kind == 3 ? 1 : 0;
  if (have != n_state) throw std::runtime_error("train_state.bin: holds " + std::to_string(n_state) + " state tensors, the graph has " + std::to_string(have) + " (another optimizer?)");
  if (im.device >= 0) check_cuda(cudaSetDevice(im.device), "cudaSetDevice");
  std::vector<char> host;
  // read everything first, apply after: a truncated file leaves the graph untouched
  std::vector<std::vector<char>> staged;
  for (size_t i = 0; i < im.ir.tensors.size(); ++i) {
    const TensorDef& t = im.ir.tensors[i];
    if (t.kind != 3) continue;
    uint64_t n = 0;
    f.read(reinterpret_cast<char*>(&n), 8);
    if (!f || n != static_cast<uint64_t>(numel(t.shape))) throw std::runtime_error("train_state.bin: state tensor " + std::to_string(staged.size()) + " has another length or the file is truncated");
    host.resize(n * 4);
    f.read(host.data(), static_cast<std::streamsize>(host.size()));
    if (static_cast<size_t>(f.gcount()) != host.size()) throw std::runtime_error("train_state.bin: truncated");
    staged.push_back(host);
  }
  size_t k = 0;
  for (size_t i = 0; i < im.ir.tensors.size(); ++i) {
    if (im.ir.tensors[i].kind != 3) continue;
    copy_in(im.params[i].get(), staged[k].data(), staged[k].size(), im.device);
    ++k;
  }
  im.train_steps = static_cast<int64_t>(steps);
}

int Graph::num_inputs() const { return static_cast<int>(impl_->ir.inputs.size()); }
int Graph::num_outputs() const { return static_cast<int>(impl_->ir.outputs.size()); }
Shape Graph::input_shape(int i) const {
  const int t = impl_->ir.inputs.at(static_cast<size_t>(i));
  return Shape(impl_->plan ? impl_->plan->shape[static_cast<size_t>(t)] : impl_->ir.tensors[static_cast<size_t>(t)].shape);
}
Shape Graph::output_shape(int i) const {
  const int t = impl_->ir.outputs.at(static_cast<size_t>(i));
  return Shape(impl_->plan ? impl_->plan->shape[static_cast<size_t>(t)] : impl_->ir.tensors[static_cast<size_t>(t)].shape);
}
int64_t Graph::in_features() const {
  const auto& s = impl_->ir.tensors[static_cast<size_t>(impl_->ir.inputs[0])].shape;
  return s.empty() ? 1 : s.back();
}
int64_t Graph::out_features() const {
  const auto& s = impl_->ir.tensors[static_cast<size_t>(impl_->ir.outputs[0])].shape;
  return s.empty() ? 1 : s.back();   // a scalar output (a loss) counts as one feature
}
PlanStats Graph::stats() const {
  std::lock_guard<std::mutex> g(impl_->run_mu);
  PlanStats st = impl_->plan ? impl_->plan->stats : PlanStats();
  st.graph_replays = impl_->graph_replays;
  return st;
}

DType Graph::input_dtype(int i) const { return impl_->ir.tensors[static_cast<size_t>(impl_->ir.inputs.at(static_cast<size_t>(i)))].dtype; }
int Graph::device() const { return impl_->device; }
void Graph::BindRows(int64_t rows) {
  std::lock_guard<std::mutex> g(impl_->run_mu);
  if (!impl_->ir.dynamic_rows) throw std::runtime_error("the graph was exported with fixed shapes; the input does not match them");
  if (!impl_->plan || impl_->plan->rows != rows) impl_->compile(rows);
}

Tensor Graph::Forward(const Tensor& input) const { return Forward(std::vector<Tensor>{input}).at(0); }

std::vector<Tensor> Graph::Forward(const std::vector<Tensor>& inputs) const { return impl_->run(inputs, Impl::kStep, *this); }
std::vector<Tensor> Graph::Evaluate(const std::vector<Tensor>& inputs) const {
  return impl_->run(inputs, impl_->ir.training ? Impl::kEvaluate : Impl::kStep, *this);
}
void Graph::ApplyUpdate() {
  if (!impl_->ir.training || !impl_->train.external_gradient_reduction) throw std::runtime_error("ApplyUpdate: the graph was not loaded with external_gradient_reduction");
  impl_->run({}, Impl::kUpdateOnly, *this);
}
std::vector<float> Graph::gradient(int i) const {
  Impl& im = *impl_;
  std::lock_guard<std::mutex> g(im.run_mu);
  if (!im.train.external_gradient_reduction) throw std::runtime_error("gradient: the graph was not loaded with external_gradient_reduction");
  const int t = im.ir.grad_tensors.at(static_cast<size_t>(i));
  std::vector<float> out(static_cast<size_t>(numel(im.ir.tensors[static_cast<size_t>(t)].shape)));
  if (im.device >= 0) check_cuda(cudaSetDevice(im.device), "cudaSetDevice");
  copy_out(out.data(), im.params[static_cast<size_t>(t)].get(), out.size() * 4, im.device);
  return out;
}
void Graph::set_gradient(int i, const float* values, int64_t count) {
  Impl& im = *impl_;
  std::lock_guard<std::mutex> g(im.run_mu);
  if (!im.train.external_gradient_reduction) throw std::runtime_error("set_gradient: the graph was not loaded with external_gradient_reduction");
  const int t = im.ir.grad_tensors.at(static_cast<size_t>(i));
  if (count != numel(im.ir.tensors[static_cast<size_t>(t)].shape)) throw std::runtime_error("set_gradient: wrong number of elements");
  if (im.device >= 0) check_cuda(cudaSetDevice(im.device), "cudaSetDevice");
  copy_in(im.params[static_cast<size_t>(t)].get(), values, static_cast<size_t>(count) * 4, im.device);
}

std::vector<Tensor> Graph::Impl::run(const std::vector<Tensor>& inputs, int mode, const Graph& self) {
  Impl& im = *this;
  std::lock_guard<std::mutex> run_guard(im.run_mu);
  const bool evaluate = mode == kEvaluate, update_only = mode == kUpdateOnly;
  if (update_only && im.micro_step == 0) throw std::runtime_error("ApplyUpdate: no gradients have been accumulated since the last update");
  if (!update_only && inputs.size() != im.ir.inputs.size()) throw std::runtime_error("Forward: wrong number of inputs");
  if (im.device >= 0) check_cuda(cudaSetDevice(im.device), "cudaSetDevice");
  if (im.ir.dynamic_rows) {
    const int64_t feat = self.in_features();
    const int64_t rows = inputs[0].shape().elem_cnt() / (feat > 0 ? feat : 1);
    if (!im.plan || im.plan->rows != rows) im.compile(rows);
  }
  const Plan& plan = *im.plan;
  im.bound.assign(im.ir.tensors.size(), nullptr);
  for (size_t i = 0; i < im.ir.tensors.size(); ++i)
    if (im.params[i]) im.bound[i] = im.params[i].get();
  for (size_t i = 0; i < inputs.size(); ++i) {
    const int t = im.ir.inputs[i];
    const TensorDef& def = im.ir.tensors[static_cast<size_t>(t)];
    if (inputs[i].dtype() != def.dtype) throw std::runtime_error("Forward: input " + std::to_string(i) + " has the wrong dtype");
    if (inputs[i].shape().elem_cnt() != numel(plan.shape[static_cast<size_t>(t)]))
      throw std::runtime_error("Forward: input " + std::to_string(i) + " has the wrong number of elements");
    if (inputs[i].device() != im.device) throw std::runtime_error("Forward: input " + std::to_string(i) + " lives on another device");
    if (im.device >= 0) {
      // the plan reads its inputs from buffers of its own (fixed addresses, as a recorded graph needs)
      check_cuda(cudaSetDevice(im.device), "cudaSetDevice");
      check_cuda(cudaMemcpyAsync(im.input_bufs[i].get(), inputs[i].data(), static_cast<size_t>(inputs[i].shape().elem_cnt() * SizeOf(def.dtype)),
                                 cudaMemcpyDeviceToDevice, im.streams[0]), "cudaMemcpyAsync");
      im.bound[static_cast<size_t>(plan.root[static_cast<size_t>(t)])] = im.input_bufs[i].get();
    } else {
      im.bound[static_cast<size_t>(plan.root[static_cast<size_t>(t)])] = inputs[i].data();
    }
  }
  {
    std::lock_guard<std::mutex> g(im.err_mu);
    im.error.clear();
  }
  im.call_kind = evaluate ? 4 : (update_only ? 8 : 3);
  if (im.ir.training && !evaluate) {
    const int k = std::max(1, im.train.accumulation_steps);
    if (update_only) {
      ++im.train_steps;
    } else if (im.train.external_gradient_reduction) {
      im.call_kind = im.micro_step == 0 ? 1 : 0;   // never the updating kind: ApplyUpdate does that
    } else {
      im.call_kind = (im.micro_step == 0 ? 1 : 0) | (im.micro_step == k - 1 ? 2 : 0);
      if (im.call_kind & 2) ++im.train_steps;   // the update operator of this call sees the 1-based step number
    }
    if (!update_only) ++im.call_counter;        // dropout masks are a function of the call number
    if (im.device >= 0) {
      im.step_scalars_host[0] = im.scheduled_lr(std::max<int64_t>(im.train_steps, 1));
      im.step_scalars_host[1] = 1.f - std::pow(im.train.beta1, static_cast<float>(im.train_steps));
      im.step_scalars_host[2] = 1.f - std::pow(im.train.beta2, static_cast<float>(im.train_steps));
      im.step_scalars_host[3] = 0.f;
      std::memcpy(im.step_scalars_host + 4, &im.call_counter, 8);
      // on stream 0, which is synchronised below before anything of the step starts
      check_cuda(cudaMemcpyAsync(im.step_scalars, im.step_scalars_host, 8 * sizeof(float), cudaMemcpyHostToDevice, im.streams[0]), "cudaMemcpyAsync");
    }
  }
  bool replayed = false;
  if (im.device >= 0) {
    check_cuda(cudaStreamSynchronize(im.streams[0]), "cudaStreamSynchronize");   // inputs are in place before any stream reads them
    if (!im.graph_disabled && im.call_kind < 4 && im.runs_of_plan[im.call_kind] >= 1) {
      if (!im.graph_exec[im.call_kind] && !im.capture_plan()) im.graph_disabled = true;
      if (im.graph_exec[im.call_kind]) {
        check_cuda(cudaGraphLaunch(im.graph_exec[im.call_kind], im.streams[0]), "cudaGraphLaunch");
        check_cuda(cudaStreamSynchronize(im.streams[0]), "cudaStreamSynchronize");
        replayed = true;
        ++im.graph_replays;
      }
    }
  }
  if (im.call_kind < 4) ++im.runs_of_plan[im.call_kind];
  if (im.ir.training && !evaluate) im.micro_step = (update_only || (im.call_kind & 2)) ? 0 : im.micro_step + 1;
  const int n_ops = replayed ? 0 : static_cast<int>(plan.ops.size());
  std::vector<TaskArg> args(static_cast<size_t>(n_ops));
  for (int i = 0; i < n_ops; ++i) {
    args[static_cast<size_t>(i)] = TaskArg{&im, i};
    const PlannedOp& p = plan.ops[static_cast<size_t>(i)];
    std::vector<int64_t> reads(p.deps.begin(), p.deps.end());
    const int64_t own = i;
    if (ofc_executor_submit(im.executor, p.stream, task_trampoline, &args[static_cast<size_t>(i)], reads.data(), static_cast<int>(reads.size()), &own, 1) != 0)
      throw std::runtime_error(std::string("executor: ") + ofc_last_error());
  }
  if (ofc_executor_wait_all(im.executor, 600000) != 0) throw std::runtime_error(std::string("executor: ") + ofc_last_error());
  if (im.device >= 0) {
    check_cuda(cudaSetDevice(im.device), "cudaSetDevice");
    for (auto s : im.streams) check_cuda(cudaStreamSynchronize(s), "cudaStreamSynchronize");
  }
  if (im.failed()) throw std::runtime_error(im.error);
  std::vector<Tensor> outs;
  if (update_only) return outs;
  for (int t : im.ir.outputs) {
    const TensorDef& def = im.ir.tensors[static_cast<size_t>(t)];
    Tensor o = Tensor::empty(Shape(plan.shape[static_cast<size_t>(t)]), im.device, def.dtype);
    const size_t bytes = static_cast<size_t>(numel(plan.shape[static_cast<size_t>(t)]) * SizeOf(def.dtype));
    if (im.device < 0) std::memcpy(o.data(), im.addr(t), bytes);
    else check_cuda(cudaMemcpy(o.data(), im.addr(t), bytes, cudaMemcpyDeviceToDevice), "cudaMemcpy");
    outs.push_back(std::move(o));
  }
  return outs;
}

}  // namespace oneflow_api
