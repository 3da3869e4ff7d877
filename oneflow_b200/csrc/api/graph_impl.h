// Shared definitions of the graph compiler and executor behind oneflow_api::Graph: the operator IR, the compiled plan and
// the implementation object. Included by graph_runtime.cpp (parser, plan compiler, forward operators, execution),
// graph_autodiff.cpp (the pass that appends backward and optimizer operators) and graph_train_ops.cpp (their kernels).
#pragma once
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "../core/ofc_core.h"
#include "graph_runtime.h"

namespace oneflow_api {

using namespace detail;

// ------------------------------------------------------------------------------------------------ IR
struct TensorDef {
  DType dtype = DType::kBFloat16;
  std::vector<int64_t> shape;
  int kind = 2;   // 0 input, 1 param, 2 activation, 3 optimizer state (persistent, written by the update operator)
  std::string file;
  int alias_of = -1;
  int64_t alias_off = 0;   // elements into the aliased tensor
  std::string name;        // parameters the exporter found among the module's named parameters: these are trainable
  int init_from = -1;      // state tensors: starts as a copy of this parameter (fp32 master weights); else zeros
};
struct OpDef {
  std::string type;
  std::vector<int> in, out;
  std::map<std::string, std::string> attr;
};
struct IR {
  std::vector<TensorDef> tensors;
  std::vector<OpDef> ops;
  std::vector<int> inputs, outputs;
  bool dynamic_rows = false;
  // training graphs (filled by append_training_ops)
  bool training = false;
  std::vector<int> trainable;   // parameter roots that get updated, in export order
  std::vector<int> masters;     // their fp32 master-weight state tensors
  std::vector<int> grad_tensors;  // their fp32 gradient buffers (persistent only with accumulation or external reduction)
  int n_forward_ops = 0;        // operators before the first backward one
  bool recompute_cheap = false; // asks the recompute pass to run
  bool recompute_full = false;  // ... for every operator off the residual stream
  std::vector<std::pair<std::string, int>> pass_report;   // rewriting passes that ran and how often each fired
};

// The rewriting passes (graph_passes.cpp), in their fixed order; returns (pass name, times it fired).
std::vector<std::pair<std::string, int>> run_graph_passes(IR& ir);
// d fn(x) / dx for the unary function codes (graph_train_ops.cpp).
float host_unary_grad(float x, int fn, float alpha);

// Appends to a forward IR whose first output is a scalar loss: the backward operators, gradient buffers and one optimizer
// update operator (graph_autodiff.cpp). Throws std::runtime_error with the offending operator for anything it cannot
// differentiate.
void append_training_ops(IR& ir, const TrainOptions& options);
// Shape / dtype checks and scratch sizes of the operators only training graphs contain (graph_train_ops.cpp);
// check_train_op returns false for a type it does not know.
struct Plan;
bool check_train_op(const OpDef& op, const IR& ir, const Plan& plan);
int64_t train_workspace_for(const OpDef& op, const Plan& plan);
// The IR in its text format (tensors, operators, inputs, outputs).
std::string ir_to_text(const IR& ir);

inline std::vector<std::string> split(const std::string& s, char sep) {
  std::vector<std::string> out;
  std::string cur;
  for (char c : s) {
    if (c == sep) { out.push_back(cur); cur.clear(); }
    else cur.push_back(c);
  }
  out.push_back(cur);
  return out;
}
inline std::vector<int64_t> int_list(const std::string& s) {
  std::vector<int64_t> out;
  if (s.empty()) return out;
  for (auto& t : split(s, ',')) out.push_back(std::stoll(t));
  return out;
}
inline int64_t attr_int(const OpDef& op, const char* k, int64_t dflt) {
  auto it = op.attr.find(k);
  return it == op.attr.end() ? dflt : std::stoll(it->second);
}
inline double attr_float(const OpDef& op, const char* k, double dflt) {
  auto it = op.attr.find(k);
  return it == op.attr.end() ? dflt : std::stod(it->second);
}
inline std::string attr_str(const OpDef& op, const char* k, const std::string& dflt) {
  auto it = op.attr.find(k);
  return it == op.attr.end() ? dflt : it->second;
}
inline int act_code(const std::string& a) { return a == "gelu" ? 1 : a == "gelu_tanh" ? 2 : a == "relu" ? 3 : 0; }

// ------------------------------------------------------------------------------------------------ plan
struct Range {
  int64_t key, bytes;
};
inline bool overlaps(const Range& a, const Range& b) { return a.key < b.key + b.bytes && b.key < a.key + a.bytes; }

struct PlannedOp {
  const OpDef* def = nullptr;
  std::vector<int> deps;        // indices of earlier operators this one must follow
  int stream = 0;
  int64_t workspace_bytes = 0;
  void* workspace = nullptr;
  std::vector<Range> reads, writes;
};

struct Plan {
  int64_t rows = 0;
  std::vector<std::vector<int64_t>> shape;     // resolved shapes per tensor
  std::vector<int> root;                       // storage root per tensor
  std::vector<int64_t> byte_off;               // byte offset of the tensor inside its root's storage
  std::vector<void*> base;                     // per root: planned address (activations); null for inputs (bound per call)
  std::vector<PlannedOp> ops;
  PlanStats stats;
};

inline int64_t numel(const std::vector<int64_t>& s) {
  int64_t n = 1;
  for (auto d : s) n *= d;
  return n;
}

struct Graph::Impl {
  IR ir;
  std::string dir;
  std::string graph_text;   // graph.txt as loaded (Save writes it back unchanged)
  int device = 0;
  int n_streams = 2;
  std::vector<std::shared_ptr<void>> params;   // per tensor id (params only)
  std::vector<void*> allocators;              // one pool per stream of the plan
  void* executor = nullptr;
  std::vector<cudaStream_t> streams;
  std::vector<cudaEvent_t> events;             // one per planned operator
  std::unique_ptr<Plan> plan;
  // GPU only: the plan replayed as one CUDA graph. The first Forward of a plan runs through the scheduler (it also performs
  // every one-time initialisation the kernels do on first use); the second one records the same launches (same streams,
  // cross-stream edges as events) into a graph on the calling thread, and from then on a Forward is: copy the inputs into
  // the plan's own input buffers, one graph launch, copy the outputs out.
  std::vector<std::shared_ptr<void>> input_bufs;   // per graph input, static addresses
  // One recorded graph per kind of call: bit 0 = first micro-batch of an optimizer step, bit 1 = last one (operators marked
  // when=first / when=last only run then). Without gradient accumulation every call is kind 3.
  cudaGraphExec_t graph_exec[4] = {nullptr, nullptr, nullptr, nullptr};
  cudaEvent_t fork_event = nullptr;
  std::vector<cudaEvent_t> join_events;
  int runs_of_plan[4] = {0, 0, 0, 0};
  int micro_step = 0;     // position inside the current optimizer step
  int call_kind = 3;      // of the running call; 4 = evaluation (forward operators only), 8 = update only; neither is recorded
  enum RunMode { kStep = 0, kEvaluate = 1, kUpdateOnly = 2 };
  std::vector<Tensor> run(const std::vector<Tensor>& inputs, int mode, const Graph& self);
  int64_t graph_replays = 0;
  bool graph_disabled = false;
  // training graphs: hyper-parameters read by the update operator at launch time, steps taken so far
  TrainOptions train;
  int64_t train_steps = 0;
  // GPU: {learning rate, 1 - beta1^t, 1 - beta2^t} of the running step, refreshed before every step through pinned host
  // memory; the update operator reads them on the device, so a recorded step stays valid from one step to the next
  float* step_scalars = nullptr;
  float* step_scalars_host = nullptr;
  // dropout: number of Forward calls so far; on the GPU it follows the four floats above as one 64-bit value
  uint64_t call_counter = 0;
  const unsigned long long* call_counter_device() const { return reinterpret_cast<const unsigned long long*>(step_scalars + 4); }
  std::mutex run_mu;
  // per call
  std::vector<void*> bound;                    // per root: address of inputs for the running call
  std::mutex err_mu;
  std::string error;

  ~Impl() {
    if (executor) ofc_executor_destroy(executor);
    if (device >= 0) cudaSetDevice(device);   // the streams, events and graphs below belong to that device
    if (step_scalars) cudaFree(step_scalars);
    if (step_scalars_host) cudaFreeHost(step_scalars_host);
    for (auto ge : graph_exec)
      if (ge) cudaGraphExecDestroy(ge);
    if (fork_event) cudaEventDestroy(fork_event);
    for (auto e : join_events) cudaEventDestroy(e);
    for (auto e : events) cudaEventDestroy(e);
    for (auto s : streams) cudaStreamDestroy(s);
    for (void* al : allocators) ofc_allocator_destroy(al);
  }

  void fail(const std::string& msg) {
    std::lock_guard<std::mutex> g(err_mu);
    if (error.empty()) error = msg;
  }
  bool failed() {
    std::lock_guard<std::mutex> g(err_mu);
    return !error.empty();
  }

  void compile(int64_t rows);
  void* addr(int tensor) const {
    const int r = plan->root[static_cast<size_t>(tensor)];
    char* b = static_cast<char*>(plan->base[static_cast<size_t>(r)] ? plan->base[static_cast<size_t>(r)] : bound[static_cast<size_t>(r)]);
    return b + plan->byte_off[static_cast<size_t>(tensor)];
  }
  // learning rate of optimizer step t (1-based) under the schedule of `train`
  float scheduled_lr(int64_t t) const {
    float lr = train.lr;
    if (train.warmup_steps > 0 && t <= train.warmup_steps) return lr * static_cast<float>(t) / static_cast<float>(train.warmup_steps);
    if (train.lr_schedule == "constant" || train.decay_steps <= train.warmup_steps) return lr;
    const double span = static_cast<double>(train.decay_steps - train.warmup_steps);
    const double x = std::min(1.0, static_cast<double>(t - train.warmup_steps) / span);
    const double shape = train.lr_schedule == "cosine" ? 0.5 * (1.0 + std::cos(3.14159265358979323846 * x)) : 1.0 - x;
    return lr * static_cast<float>(train.min_lr_ratio + (1.0 - train.min_lr_ratio) * shape);
  }
  // operators marked when=first / when=last are skipped on the other micro-batches
  bool op_enabled(const OpDef& op) const {
    if (call_kind == 4) return op.attr.count("fwd") != 0;
    auto it = op.attr.find("when");
    if (call_kind == 8) return it != op.attr.end() && it->second == "last";
    if (it == op.attr.end()) return true;
    return it->second == "first" ? (call_kind & 1) != 0 : (call_kind & 2) != 0;
  }
  void run_op(int index);
  bool capture_plan();
  void run_op_device(const PlannedOp& p, cudaStream_t s);
  void run_op_host(const PlannedOp& p);
  // operators that only training graphs contain (graph_train_ops.cpp); false = not one of them
  bool run_train_op_device(const PlannedOp& p, cudaStream_t s);
  bool run_train_op_host(const PlannedOp& p);
};

}  // namespace oneflow_api
