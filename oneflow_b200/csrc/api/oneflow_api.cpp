// Tensor type and C ABI of the C++ inference API; the graph compiler and executor are in graph_runtime.cpp.
#include "oneflow_api.h"

#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <stdexcept>
#include <vector>

#include "graph_runtime.h"

namespace oneflow_api {

namespace detail {

thread_local std::string g_error;

void check_cuda(int e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(static_cast<cudaError_t>(e)));
}

uint16_t to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);  // NaN
  u += 0x7fffu + ((u >> 16) & 1u);                                                       // round to nearest even
  return static_cast<uint16_t>(u >> 16);
}
float from_bf16(uint16_t h) {
  const uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

namespace {
// Free device blocks by (device, size). Lives until the process exits (never destroyed: tensors with static lifetime may
// return blocks during shutdown). Holds at most kMaxCachedBytes; beyond that a returned block goes back to the driver.
class DevicePool {
 public:
  static constexpr size_t kMaxCachedBytes = size_t(1) << 30;
  static constexpr size_t kMaxCachedBlock = size_t(64) << 20;   // larger blocks (weights, big arenas) go straight back
  void* take(int device, size_t bytes) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = free_.find({device, bytes});
    if (it == free_.end() || it->second.empty()) return nullptr;
    void* p = it->second.back();
    it->second.pop_back();
    cached_ -= bytes;
    return p;
  }
  void give(int device, size_t bytes, void* p) {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (bytes <= kMaxCachedBlock && cached_ + bytes <= kMaxCachedBytes) {
        free_[{device, bytes}].push_back(p);
        cached_ += bytes;
        return;
      }
    }
    cudaFree(p);
  }
  void release_all() {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& kv : free_)
      for (void* p : kv.second) cudaFree(p);
    free_.clear();
    cached_ = 0;
  }

 private:
  std::mutex mu_;
  std::map<std::pair<int, size_t>, std::vector<void*>> free_;
  size_t cached_ = 0;
};
DevicePool& device_pool() {
  static DevicePool* pool = new DevicePool();
  return *pool;
}
}  // namespace

std::shared_ptr<void> storage_alloc(size_t bytes, int device) {
  if (bytes == 0) bytes = 16;
  if (device < 0) {
    void* p = nullptr;
    if (posix_memalign(&p, 64, (bytes + 63) / 64 * 64) != 0) throw std::runtime_error("out of host memory");
    return std::shared_ptr<void>(p, [](void* q) { std::free(q); });
  }
  check_cuda(cudaSetDevice(device), "cudaSetDevice");
  // Device blocks are recycled: a serving loop allocates the same input and output sizes on every request, and a
  // cudaMalloc / cudaFree pair costs more than a small graph takes to run. Every user of a block is synchronous with the
  // host when the block is dropped (Forward returns after its streams are idle, the copies block), so a returned block can
  // be handed out again at once.
  DevicePool& pool = device_pool();
  bytes = (bytes + 511) / 512 * 512;
  void* p = pool.take(device, bytes);
  if (!p) {
    cudaError_t rc = cudaMalloc(&p, bytes);
    if (rc != cudaSuccess) {
      cudaGetLastError();
      pool.release_all();
      check_cuda(cudaMalloc(&p, bytes), "cudaMalloc");
    }
  }
  return std::shared_ptr<void>(p, [device, bytes](void* q) { device_pool().give(device, bytes, q); });
}

}  // namespace detail

void EmptyCache() { detail::device_pool().release_all(); }

namespace detail {

void copy_in(void* dst, const void* host, size_t bytes, int device) {
  if (bytes == 0) return;
  if (device < 0) std::memcpy(dst, host, bytes);
  else check_cuda(cudaMemcpy(dst, host, bytes, cudaMemcpyHostToDevice), "cudaMemcpy");
}
void copy_out(void* host, const void* src, size_t bytes, int device) {
  if (bytes == 0) return;
  if (device < 0) std::memcpy(host, src, bytes);
  else check_cuda(cudaMemcpy(host, src, bytes, cudaMemcpyDeviceToHost), "cudaMemcpy");
}

}  // namespace detail

using namespace detail;

Tensor Tensor::empty(const Shape& shape, int device, DType dtype) {
  Tensor t;
  t.shape_ = shape;
  t.device_ = device;
  t.dtype_ = dtype;
  t.data_ = storage_alloc(static_cast<size_t>(shape.elem_cnt() * SizeOf(dtype)), device);
  return t;
}

Tensor Tensor::from_buffer(const float* host, const Shape& shape, int device) {
  Tensor t = empty(shape, device, DType::kBFloat16);
  const int64_t n = shape.elem_cnt();
  std::vector<uint16_t> tmp(static_cast<size_t>(n));
  for (int64_t i = 0; i < n; ++i) tmp[static_cast<size_t>(i)] = to_bf16(host[i]);
  copy_in(t.data(), tmp.data(), static_cast<size_t>(n) * 2, device);
  return t;
}

Tensor Tensor::from_int64(const int64_t* host, const Shape& shape, int device) {
  Tensor t = empty(shape, device, DType::kInt64);
  copy_in(t.data(), host, static_cast<size_t>(shape.elem_cnt()) * 8, device);
  return t;
}

std::vector<float> Tensor::to_host() const {
  const int64_t n = shape_.elem_cnt();
  std::vector<float> out(static_cast<size_t>(n));
  if (device_ >= 0) check_cuda(cudaSetDevice(device_), "cudaSetDevice");
  if (dtype_ == DType::kBFloat16) {
    std::vector<uint16_t> tmp(static_cast<size_t>(n));
    copy_out(tmp.data(), data(), static_cast<size_t>(n) * 2, device_);
    for (int64_t i = 0; i < n; ++i) out[static_cast<size_t>(i)] = from_bf16(tmp[static_cast<size_t>(i)]);
  } else if (dtype_ == DType::kFloat) {
    copy_out(out.data(), data(), static_cast<size_t>(n) * 4, device_);
  } else {
    std::vector<int64_t> tmp(static_cast<size_t>(n));
    copy_out(tmp.data(), data(), static_cast<size_t>(n) * 8, device_);
    for (int64_t i = 0; i < n; ++i) out[static_cast<size_t>(i)] = static_cast<float>(tmp[static_cast<size_t>(i)]);
  }
  return out;
}

}  // namespace oneflow_api

// ------------------------------------------------------------------------------------------------ C ABI
extern "C" {

using oneflow_api::Graph;
using oneflow_api::Shape;
using oneflow_api::Tensor;

const char* ofb_api_last_error(void) { return oneflow_api::detail::g_error.c_str(); }

void* ofb_api_graph_load_ex(const char* dir, int device, int n_streams) {
  try {
    return new Graph(Graph::Load(dir, device, n_streams));
  } catch (const std::exception& e) {
    oneflow_api::detail::g_error = e.what();
    return nullptr;
  }
}
void* ofb_api_graph_load(const char* dir, int device) { return ofb_api_graph_load_ex(dir, device, 2); }
long long ofb_api_graph_in_features(void* g) { return static_cast<Graph*>(g)->in_features(); }
long long ofb_api_graph_out_features(void* g) { return static_cast<Graph*>(g)->out_features(); }
int ofb_api_graph_num_inputs(void* g) { return static_cast<Graph*>(g)->num_inputs(); }
int ofb_api_graph_num_outputs(void* g) { return static_cast<Graph*>(g)->num_outputs(); }
long long ofb_api_graph_input_numel(void* g, int i) { return static_cast<Graph*>(g)->input_shape(i).elem_cnt(); }
long long ofb_api_graph_output_numel(void* g, int i) { return static_cast<Graph*>(g)->output_shape(i).elem_cnt(); }
int ofb_api_graph_input_is_int64(void* g, int i) { return oneflow_api::graph_input_is_int64(*static_cast<Graph*>(g), i) ? 1 : 0; }

static int run_or_evaluate(void* g, const void* const* inputs, int n_in, float* const* outputs, int n_out, bool evaluate);
int ofb_api_graph_run(void* g, const void* const* inputs, int n_in, float* const* outputs, int n_out) {
  return run_or_evaluate(g, inputs, n_in, outputs, n_out, false);
}
int ofb_api_graph_evaluate(void* g, const void* const* inputs, int n_in, float* const* outputs, int n_out) {
  return run_or_evaluate(g, inputs, n_in, outputs, n_out, true);
}
static int run_or_evaluate(void* g, const void* const* inputs, int n_in, float* const* outputs, int n_out, bool evaluate) {
  try {
    auto* graph = static_cast<Graph*>(g);
    if (n_in != graph->num_inputs() || n_out != graph->num_outputs()) throw std::runtime_error("run: wrong number of inputs or outputs");
    const int device = oneflow_api::graph_device(*graph);
    std::vector<Tensor> in;
    for (int i = 0; i < n_in; ++i) {
      if (oneflow_api::graph_input_is_int64(*graph, i))
        in.push_back(Tensor::from_int64(static_cast<const int64_t*>(inputs[i]), graph->input_shape(i), device));
      else
        in.push_back(Tensor::from_buffer(static_cast<const float*>(inputs[i]), graph->input_shape(i), device));
    }
    auto out = evaluate ? graph->Evaluate(in) : graph->Forward(in);
    for (int i = 0; i < n_out; ++i) {
      auto h = out[static_cast<size_t>(i)].to_host();
      std::memcpy(outputs[i], h.data(), h.size() * sizeof(float));
    }
    return 0;
  } catch (const std::exception& e) {
    oneflow_api::detail::g_error = e.what();
    return -1;
  }
}

int ofb_api_graph_forward(void* g, const float* x, long long rows, float* y) {
  try {
    auto* graph = static_cast<Graph*>(g);
    if (graph->num_inputs() != 1 || graph->num_outputs() != 1) throw std::runtime_error("forward: the graph has several inputs or outputs; use ofb_api_graph_run");
    const Shape want = graph->input_shape(0);
    if (want.elem_cnt() != rows * graph->in_features()) {
      // layer-list graphs are exported without a batch size: bind it now
      oneflow_api::graph_rebind_rows(*graph, rows);
    }
    const void* in[1] = {x};
    float* out[1] = {y};
    return ofb_api_graph_run(g, in, 1, out, 1);
  } catch (const std::exception& e) {
    oneflow_api::detail::g_error = e.what();
    return -1;
  }
}

int ofb_api_graph_stats(void* g, long long* s) {
  const auto st = static_cast<Graph*>(g)->stats();
  s[0] = st.n_ops; s[1] = st.n_tensors; s[2] = st.activation_bytes; s[3] = st.arena_bytes; s[4] = st.n_dependencies; s[5] = st.n_streams_used; s[6] = st.graph_replays;
  return 0;
}
void ofb_api_graph_free(void* g) { delete static_cast<Graph*>(g); }

void* ofb_api_graph_load_training_ex(const char* dir, int device, int n_streams, const char* optimizer, float lr, float beta1, float beta2, float eps,
                                     float weight_decay, float momentum, float clip_grad_norm, int accumulation_steps) {
  return ofb_api_graph_load_training_flags(dir, device, n_streams, optimizer, lr, beta1, beta2, eps, weight_decay, momentum, clip_grad_norm,
                                           accumulation_steps, 0);
}
void* ofb_api_graph_load_training_flags(const char* dir, int device, int n_streams, const char* optimizer, float lr, float beta1, float beta2, float eps,
                                        float weight_decay, float momentum, float clip_grad_norm, int accumulation_steps, int flags) {
  try {
    oneflow_api::TrainOptions o;
    o.optimizer = optimizer ? optimizer : "adamw";
    o.lr = lr; o.beta1 = beta1; o.beta2 = beta2; o.eps = eps; o.weight_decay = weight_decay; o.momentum = momentum;
    o.clip_grad_norm = clip_grad_norm;
    o.accumulation_steps = accumulation_steps;
    o.recompute_cheap_activations = (flags & 1) != 0;
    o.recompute_all_but_residual_stream = (flags & 2) != 0;
    o.external_gradient_reduction = (flags & 4) != 0;
    o.decay_matrices_only = (flags & 8) != 0;
    return new Graph(Graph::LoadTraining(dir, o, device, n_streams));
  } catch (const std::exception& e) {
    oneflow_api::detail::g_error = e.what();
    return nullptr;
  }
}
void* ofb_api_graph_load_training(const char* dir, int device, int n_streams, const char* optimizer, float lr, float beta1, float beta2, float eps,
                                  float weight_decay, float momentum) {
  return ofb_api_graph_load_training_ex(dir, device, n_streams, optimizer, lr, beta1, beta2, eps, weight_decay, momentum, 0.f, 1);
}
int ofb_api_graph_num_parameters(void* g) { return static_cast<Graph*>(g)->num_parameters(); }
const char* ofb_api_graph_parameter_name(void* g, int i) {
  static thread_local std::string name;
  try {
    name = static_cast<Graph*>(g)->parameter_name(i);
  } catch (const std::exception& e) {
    oneflow_api::detail::g_error = e.what();
    return nullptr;
  }
  return name.c_str();
}
long long ofb_api_graph_parameter_numel(void* g, int i) {
  try {
    return static_cast<Graph*>(g)->parameter_numel(i);
  } catch (const std::exception& e) {
    oneflow_api::detail::g_error = e.what();
    return -1;
  }
}
int ofb_api_graph_parameter_read(void* g, int i, float* out) {
  try {
    const auto v = static_cast<Graph*>(g)->parameter(i);
    std::memcpy(out, v.data(), v.size() * sizeof(float));
    return 0;
  } catch (const std::exception& e) {
    oneflow_api::detail::g_error = e.what();
    return -1;
  }
}
int ofb_api_graph_gradient_read(void* g, int i, float* out) {
  try {
    const auto v = static_cast<Graph*>(g)->gradient(i);
    std::memcpy(out, v.data(), v.size() * sizeof(float));
    return 0;
  } catch (const std::exception& e) {
    oneflow_api::detail::g_error = e.what();
    return -1;
  }
}
int ofb_api_graph_gradient_write(void* g, int i, const float* values, long long count) {
  try {
    static_cast<Graph*>(g)->set_gradient(i, values, count);
    return 0;
  } catch (const std::exception& e) {
    oneflow_api::detail::g_error = e.what();
    return -1;
  }
}
int ofb_api_graph_apply_update(void* g) {
  try {
    static_cast<Graph*>(g)->ApplyUpdate();
    return 0;
  } catch (const std::exception& e) {
    oneflow_api::detail::g_error = e.what();
    return -1;
  }
}
int ofb_api_graph_set_lr(void* g, float lr) {
  static_cast<Graph*>(g)->set_learning_rate(lr);
  return 0;
}
int ofb_api_graph_save(void* g, const char* dir) {
  try {
    static_cast<Graph*>(g)->Save(dir);
    return 0;
  } catch (const std::exception& e) {
    oneflow_api::detail::g_error = e.what();
    return -1;
  }
}
int ofb_api_graph_restore(void* g, const char* dir) {
  try {
    static_cast<Graph*>(g)->Restore(dir);
    return 0;
  } catch (const std::exception& e) {
    oneflow_api::detail::g_error = e.what();
    return -1;
  }
}
int ofb_api_graph_set_lr_schedule(void* g, const char* kind, long long warmup_steps, long long decay_steps, float min_lr_ratio) {
  try {
    static_cast<Graph*>(g)->set_lr_schedule(kind ? kind : "constant", warmup_steps, decay_steps, min_lr_ratio);
    return 0;
  } catch (const std::exception& e) {
    oneflow_api::detail::g_error = e.what();
    return -1;
  }
}
float ofb_api_graph_lr(void* g) { return static_cast<Graph*>(g)->learning_rate(); }
int ofb_api_graph_set_seed(void* g, unsigned long long seed) {
  static_cast<Graph*>(g)->set_seed(seed);
  return 0;
}
long long ofb_api_graph_steps(void* g) { return static_cast<Graph*>(g)->steps(); }
long long ofb_api_graph_dump(void* g, char* buf, long long cap) {
  const std::string text = static_cast<Graph*>(g)->dump();
  if (buf && cap > 0) {
    const size_t n = std::min(static_cast<size_t>(cap - 1), text.size());
    std::memcpy(buf, text.data(), n);
    buf[n] = 0;
  }
  return static_cast<long long>(text.size());
}
}
