// C++ graph API: load an exported network and run it, or train it, without Python.
//
//   #include "oneflow_api.h"
//   auto graph = oneflow_api::Graph::Load("model_dir");            // reads graph.txt + raw weight files, compiles a plan
//   oneflow_api::Tensor x = oneflow_api::Tensor::from_buffer(host_floats, {batch, features});
//   oneflow_api::Tensor y = graph.Forward(x);                      // or Forward(std::vector<Tensor>) -> std::vector<Tensor>
//   std::vector<float> out = y.to_host();
//
// The directory is written by oneflow_b200.utils.export: `export_graph(module, example_inputs, dir)` records the operator
// graph of any module built from the supported operators (linear with fused bias / activation / residual, batched matmul,
// LayerNorm, embedding, element-wise unary and binary ops with row broadcasting, softmax, fused attention, reshapes as
// aliases, permute / slice / concatenation as strided copies) with static shapes; `export_inference_graph` is the older
// layer-list form, still read. Loading compiles the operator graph into a plan (graph_runtime.cpp):
//   * reshapes become aliases of their source's storage;
//   * every activation gets an address from the caching allocator of libofb_core (bin_allocator) by walking the
//     operators in order, allocating at the first write and freeing after the last read, so that buffers with disjoint
//     lifetimes share memory;
//   * dependencies are derived from the address ranges each operator reads and writes (true, anti and output
//     dependencies, including the ones memory sharing introduces);
//   * operators are spread over the streams of the instruction scheduler of libofb_core (task_executor): a chain stays
//     on its producer's stream, independent branches go to other streams; on the GPU each stream is a CUDA stream and
//     cross-stream dependencies are CUDA events.
// `device` >= 0 runs the sm_100a kernels of libofb_kernels on that GPU; device = -1 runs a plain host implementation of
// the same operators (fp32 arithmetic, bf16 storage), which is what the tests without a GPU use. From its second run on a
// plan on the GPU is replayed as one CUDA graph.
//
// Training: `Graph::LoadTraining(dir, options)` takes a graph whose first output is a scalar loss, appends the backward and
// optimizer operators (graph_autodiff.cpp), rewrites the result (graph_passes.cpp: activation and activation-gradient into
// GEMM epilogues, optional recomputation, dead operators) and compiles forward + backward + update into one plan; every
// Forward call is then one training step (TrainOptions below: optimizer, clipping, accumulation, checkpointing, dropout
// seed, learning-rate schedule; Evaluate, Save / Restore, parameter read-back on Graph).
//
// Reference counterpart: oneflow/api/cpp/ (oneflow_api::Tensor, Shape, Graph::Load(dir) running a saved nn.Graph through
// the job -> plan compiler and the actor runtime).
#pragma once
#include <cstdint>
#include <memory>
#include <string>
#include <vector>

namespace oneflow_api {

class Shape {
 public:
  Shape() = default;
  Shape(std::initializer_list<int64_t> d) : dims_(d) {}
  explicit Shape(std::vector<int64_t> d) : dims_(std::move(d)) {}
  int64_t At(int i) const { return dims_.at(i); }
  int NumAxes() const { return static_cast<int>(dims_.size()); }
  int64_t elem_cnt() const {
    int64_t n = 1;
    for (auto d : dims_) n *= d;
    return n;
  }
  const std::vector<int64_t>& dims() const { return dims_; }
  bool operator==(const Shape& o) const { return dims_ == o.dims_; }

 private:
  std::vector<int64_t> dims_;
};

enum class DType { kBFloat16 = 0, kInt64 = 1, kFloat = 2 };
inline int64_t SizeOf(DType t) { return t == DType::kBFloat16 ? 2 : (t == DType::kInt64 ? 8 : 4); }

// A tensor in device memory (device >= 0) or host memory (device = -1), shared ownership.
class Tensor {
 public:
  Tensor() = default;
  static Tensor from_buffer(const float* host, const Shape& shape, int device = 0);      // stored as bf16
  static Tensor from_int64(const int64_t* host, const Shape& shape, int device = 0);     // stored as int64 (token ids)
  static Tensor empty(const Shape& shape, int device = 0, DType dtype = DType::kBFloat16);
  std::vector<float> to_host() const;
  const Shape& shape() const { return shape_; }
  DType dtype() const { return dtype_; }
  void* data() const { return data_.get(); }
  int device() const { return device_; }

 private:
  Shape shape_;
  std::shared_ptr<void> data_;
  int device_ = 0;
  DType dtype_ = DType::kBFloat16;
};

// Device blocks of dropped tensors are kept for the next tensor of the same size (up to 1 GiB in blocks of at most
// 64 MiB each); this returns them to the driver.
void EmptyCache();

struct PlanStats {
  int64_t n_ops = 0, n_tensors = 0;
  int64_t activation_bytes = 0;   // sum of all activation sizes
  int64_t arena_bytes = 0;        // peak bytes in use at once after sharing (activations + operator workspaces)
  int64_t n_dependencies = 0;
  int n_streams_used = 0;
  int64_t graph_replays = 0;      // GPU: runs of the current plan that were one CUDA-graph launch
};

// Optimizer of a training graph (Graph::LoadTraining). "adamw" keeps fp32 master weights and both moments per parameter,
// "sgd" fp32 master weights and, with momentum > 0, a momentum buffer; the bf16 parameters the forward operators read are
// rewritten from the master weights by the same update operator.
struct TrainOptions {
  std::string optimizer = "adamw";
  float lr = 1e-3f;
  float beta1 = 0.9f, beta2 = 0.999f, eps = 1e-8f;
  float weight_decay = 0.f;
  // true: weight decay only on parameters used with two or more axes (weight matrices, tables); biases and LayerNorm
  // scales / shifts go into a second update operator without decay.
  bool decay_matrices_only = false;
  float momentum = 0.f;
  // > 0: the gradients are scaled by min(1, clip_grad_norm / (global L2 norm + 1e-6)) before the update.
  float clip_grad_norm = 0.f;
  // k > 1: every Forward call is one micro-batch; its gradients (of loss / k) are added to persistent fp32 buffers and the
  // optimizer runs on every k-th call.
  int accumulation_steps = 1;
  // Activation checkpointing for the cheap operators: outputs of element-wise operators and LayerNorms that only the
  // backward pass still needs are not kept; the backward pass recomputes them from their (kept) inputs.
  bool recompute_cheap_activations = false;
  // Full activation checkpointing: only the residual stream (tensors with more than one forward reader), the inputs and the
  // loss operator's results are kept; every other forward operator whose result the backward pass needs, GEMMs and attention
  // included, runs again right before that part of the backward pass.
  bool recompute_all_but_residual_stream = false;
  // Seed of the dropout operators (graphs exported in training mode). The mask of an operator is a function of (seed,
  // number of the call, operator): every call draws new masks, a run with the same seed draws the same sequence.
  uint64_t seed = 0;
  // Data parallelism (or any other treatment of the gradients) outside the graph: Forward runs forward and backward only
  // and adds into persistent fp32 gradient buffers (cleared on the first call after an update); the caller reads them with
  // gradient(i), reduces them across ranks, writes them back with set_gradient(i, ...) and calls ApplyUpdate(), which runs
  // clipping and the optimizer. accumulation_steps still scales the loss gradient (micro-batches per update).
  bool external_gradient_reduction = false;
  // Learning-rate schedule evaluated by the runtime before every optimizer step t = 1, 2, ...: linear warm-up from 0 over
  // warmup_steps, then "constant", or "cosine" / "linear" decay to min_lr_ratio * lr at decay_steps (and flat after it).
  // set_learning_rate changes the base rate the schedule scales.
  std::string lr_schedule = "constant";
  int64_t warmup_steps = 0;
  int64_t decay_steps = 0;
  float min_lr_ratio = 0.f;
};

class Graph {
 public:
  static Graph Load(const std::string& dir, int device = 0, int n_streams = 2);
  // The same exported graph as a TRAINING step. Its first output must be a scalar loss (a cross_entropy or mse operator).
  // Loading appends the backward operators of everything between the named (trainable) parameters and the loss, and one
  // optimizer update operator; the whole step is then compiled like an inference graph (liveness, memory sharing across
  // forward and backward, dependencies, streams). Each Forward call runs one step: forward, backward, update; it returns
  // the graph's outputs (the loss first) as computed BEFORE the update.
  static Graph LoadTraining(const std::string& dir, const TrainOptions& options, int device = 0, int n_streams = 2);
  Tensor Forward(const Tensor& input) const;
  std::vector<Tensor> Forward(const std::vector<Tensor>& inputs) const;
  // Training graphs: the forward operators only, dropout switched off, nothing updated and no counter advanced (a
  // validation loss between steps). On an inference graph it is Forward.
  std::vector<Tensor> Evaluate(const std::vector<Tensor>& inputs) const;
  // Graphs loaded with external_gradient_reduction: the accumulated gradient of trainable parameter i (fp32), and the
  // optimizer step on whatever the gradient buffers hold now.
  std::vector<float> gradient(int i) const;
  void set_gradient(int i, const float* values, int64_t count);
  void ApplyUpdate();
  int64_t in_features() const;    // last axis of the first input
  int64_t out_features() const;   // last axis of the first output
  int num_inputs() const;
  int num_outputs() const;
  Shape input_shape(int i) const;
  Shape output_shape(int i) const;
  DType input_dtype(int i) const;
  int device() const;
  // Graphs exported without a batch size (the layer-list form) are compiled for a row count on first use, or here.
  void BindRows(int64_t rows);
  PlanStats stats() const;
  // Training graphs: the trainable parameters in export order, their current values (fp32 master weights), the learning
  // rate of the following steps, the number of steps taken, and the operator list after the backward pass was appended
  // (the IR text format, for inspection).
  int num_parameters() const;
  std::string parameter_name(int i) const;
  int64_t parameter_numel(int i) const;
  std::vector<float> parameter(int i) const;
  // Save writes a directory that loads again (graph.txt and every parameter file, the trainable ones with their current
  // values) plus, for training graphs, train_state.bin: step count, fp32 master weights and optimizer state. Restore reads
  // train_state.bin back into a training graph loaded from such a directory, so that training continues bit for bit.
  void Save(const std::string& dir) const;
  void Restore(const std::string& dir);
  void set_learning_rate(float lr);
  void set_lr_schedule(const std::string& kind, int64_t warmup_steps, int64_t decay_steps, float min_lr_ratio);
  float learning_rate() const;   // the rate the next optimizer step will use
  void set_seed(uint64_t seed);
  int64_t steps() const;
  std::string dump() const;
  struct Impl;

 private:
  std::shared_ptr<Impl> impl_;
};

}  // namespace oneflow_api

extern "C" {
void* ofb_api_graph_load(const char* dir, int device);
void* ofb_api_graph_load_ex(const char* dir, int device, int n_streams);
long long ofb_api_graph_in_features(void* graph);
long long ofb_api_graph_out_features(void* graph);
// x: host fp32 [rows, in_features]; y: host fp32 [rows, out_features]. Returns 0 on success. For graphs with one bf16 input
// whose leading axes multiply to `rows` as exported.
int ofb_api_graph_forward(void* graph, const float* x, long long rows, float* y);
// General form: n_in host buffers (fp32 for bf16 inputs, int64 for id inputs) in the graph's input order with the exported
// shapes; n_out host fp32 buffers sized by ofb_api_graph_output_numel.
int ofb_api_graph_run(void* graph, const void* const* inputs, int n_in, float* const* outputs, int n_out);
int ofb_api_graph_num_inputs(void* graph);
int ofb_api_graph_num_outputs(void* graph);
long long ofb_api_graph_input_numel(void* graph, int i);
int ofb_api_graph_input_is_int64(void* graph, int i);
long long ofb_api_graph_output_numel(void* graph, int i);
// stats_out[7]: ops, tensors, activation bytes, arena bytes, dependencies, streams used, CUDA-graph replays of the current plan
int ofb_api_graph_stats(void* graph, long long* stats_out);
// As ofb_api_graph_run, through Graph::Evaluate.
int ofb_api_graph_evaluate(void* graph, const void* const* inputs, int n_inputs, float* const* outputs, int n_outputs);
// Training graphs (oneflow_api::Graph::LoadTraining); optimizer: "adamw" or "sgd".
void* ofb_api_graph_load_training(const char* dir, int device, int n_streams, const char* optimizer, float lr, float beta1, float beta2,
                                  float eps, float weight_decay, float momentum);
void* ofb_api_graph_load_training_ex(const char* dir, int device, int n_streams, const char* optimizer, float lr, float beta1, float beta2,
                                     float eps, float weight_decay, float momentum, float clip_grad_norm, int accumulation_steps);
// flags: bit 0 recompute cheap activations in the backward pass, bit 1 recompute everything but the residual stream, bit 3
// weight decay on matrices only,
// bit 2 external gradient reduction (ofb_api_graph_gradient_read / _write / ofb_api_graph_apply_update)
void* ofb_api_graph_load_training_flags(const char* dir, int device, int n_streams, const char* optimizer, float lr, float beta1, float beta2,
                                        float eps, float weight_decay, float momentum, float clip_grad_norm, int accumulation_steps, int flags);
int ofb_api_graph_num_parameters(void* graph);
const char* ofb_api_graph_parameter_name(void* graph, int i);
long long ofb_api_graph_parameter_numel(void* graph, int i);
int ofb_api_graph_parameter_read(void* graph, int i, float* out);
int ofb_api_graph_gradient_read(void* graph, int i, float* out);
int ofb_api_graph_gradient_write(void* graph, int i, const float* values, long long count);
int ofb_api_graph_apply_update(void* graph);
int ofb_api_graph_set_lr(void* graph, float lr);
int ofb_api_graph_set_seed(void* graph, unsigned long long seed);
int ofb_api_graph_set_lr_schedule(void* graph, const char* kind, long long warmup_steps, long long decay_steps, float min_lr_ratio);
float ofb_api_graph_lr(void* graph);
int ofb_api_graph_save(void* graph, const char* dir);
int ofb_api_graph_restore(void* graph, const char* dir);
long long ofb_api_graph_steps(void* graph);
// Writes the operator list (IR text) into buf (at most cap bytes, zero-terminated); returns the full length.
long long ofb_api_graph_dump(void* graph, char* buf, long long cap);
void ofb_api_graph_free(void* graph);
const char* ofb_api_last_error(void);
}
