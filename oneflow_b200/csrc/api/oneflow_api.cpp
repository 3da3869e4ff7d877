// Implementation of the C++ inference API on top of the C ABI of libofb_kernels.so.
#include "oneflow_api.h"

#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <fstream>
#include <sstream>
#include <stdexcept>

#include "../kernels/ofb_kernels.h"

extern "C" int ofb_layer_norm_fwd(const void* x, const void* gamma, const void* beta, void* y, float* mean, float* rstd, int rows,
                                  int cols, float eps, void* stream);
extern "C" int ofb_bias_act_fwd(const void* x, const void* bias, void* y, long long n, int cols, int act, void* stream);

namespace oneflow_api {

namespace {

thread_local std::string g_error;

void check_cuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
void check_ofb(int rc, const char* what) {
  if (rc != 0) throw std::runtime_error(std::string(what) + ": " + ofb_last_error());
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

std::shared_ptr<void> device_alloc(size_t bytes, int device) {
  check_cuda(cudaSetDevice(device), "cudaSetDevice");
  void* p = nullptr;
  check_cuda(cudaMalloc(&p, bytes ? bytes : 16), "cudaMalloc");
  return std::shared_ptr<void>(p, [](void* q) { cudaFree(q); });
}

std::shared_ptr<void> load_bf16_file(const std::string& path, size_t elems, int device) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot open " + path);
  std::vector<uint16_t> host(elems);
  f.read(reinterpret_cast<char*>(host.data()), static_cast<std::streamsize>(elems * 2));
  if (static_cast<size_t>(f.gcount()) != elems * 2) throw std::runtime_error("short read: " + path);
  auto dev = device_alloc(elems * 2, device);
  check_cuda(cudaMemcpy(dev.get(), host.data(), elems * 2, cudaMemcpyHostToDevice), "cudaMemcpy");
  return dev;
}

struct Layer {
  int kind = 0;  // 0 linear, 1 layer_norm, 2 activation only
  int64_t in = 0, out = 0;
  int act = 0;
  float eps = 1e-5f;
  std::shared_ptr<void> w, b;
};

}  // namespace

Tensor Tensor::empty(const Shape& shape, int device) {
  Tensor t;
  t.shape_ = shape;
  t.device_ = device;
  t.data_ = device_alloc(static_cast<size_t>(shape.elem_cnt()) * 2, device);
  return t;
}

Tensor Tensor::from_buffer(const float* host, const Shape& shape, int device) {
  Tensor t = empty(shape, device);
  const int64_t n = shape.elem_cnt();
  std::vector<uint16_t> tmp(static_cast<size_t>(n));
  for (int64_t i = 0; i < n; ++i) tmp[static_cast<size_t>(i)] = to_bf16(host[i]);
  check_cuda(cudaMemcpy(t.data(), tmp.data(), static_cast<size_t>(n) * 2, cudaMemcpyHostToDevice), "cudaMemcpy");
  return t;
}

std::vector<float> Tensor::to_host() const {
  const int64_t n = shape_.elem_cnt();
  std::vector<uint16_t> tmp(static_cast<size_t>(n));
  check_cuda(cudaSetDevice(device_), "cudaSetDevice");
  check_cuda(cudaMemcpy(tmp.data(), data(), static_cast<size_t>(n) * 2, cudaMemcpyDeviceToHost), "cudaMemcpy");
  std::vector<float> out(static_cast<size_t>(n));
  for (int64_t i = 0; i < n; ++i) out[static_cast<size_t>(i)] = from_bf16(tmp[static_cast<size_t>(i)]);
  return out;
}

struct Graph::Impl {
  std::vector<Layer> layers;
  int device = 0;
  int64_t in_features = 0, out_features = 0;
};

Graph Graph::Load(const std::string& dir, int device) {
  std::ifstream f(dir + "/graph.txt");
  if (!f) throw std::runtime_error("cannot open " + dir + "/graph.txt");
  std::string line;
  std::getline(f, line);
  if (line.rfind("oneflow_b200 inference graph v1", 0) != 0) throw std::runtime_error("not an inference graph: " + dir);
  auto impl = std::make_shared<Impl>();
  impl->device = device;
  int64_t width = -1;
  while (std::getline(f, line)) {
    if (line.empty() || line[0] == '#') continue;
    std::istringstream ss(line);
    std::string op;
    ss >> op;
    Layer l;
    if (op == "linear") {
      std::string wf, bf, act;
      ss >> l.in >> l.out >> wf >> bf >> act;
      if (l.in % 8 || l.out % 8) throw std::runtime_error("linear: features must be multiples of 8");
      if (width >= 0 && width != l.in) throw std::runtime_error("linear: input width does not match the previous layer");
      l.kind = 0;
      l.act = act == "gelu" ? 1 : act == "gelu_tanh" ? 2 : act == "relu" ? 3 : 0;
      l.w = load_bf16_file(dir + "/" + wf, static_cast<size_t>(l.in * l.out), device);
      if (bf != "-") l.b = load_bf16_file(dir + "/" + bf, static_cast<size_t>(l.out), device);
      if (impl->layers.empty()) impl->in_features = l.in;
      width = l.out;
    } else if (op == "layer_norm") {
      std::string gf, bf;
      ss >> l.in >> gf >> bf >> l.eps;
      l.out = l.in;
      l.kind = 1;
      if (width >= 0 && width != l.in) throw std::runtime_error("layer_norm: width does not match the previous layer");
      l.w = load_bf16_file(dir + "/" + gf, static_cast<size_t>(l.in), device);
      l.b = load_bf16_file(dir + "/" + bf, static_cast<size_t>(l.in), device);
      if (impl->layers.empty()) impl->in_features = l.in;
      width = l.in;
    } else if (op == "activation") {
      std::string act;
      ss >> l.in >> act;
      l.out = l.in;
      l.kind = 2;
      l.act = act == "gelu" ? 1 : act == "gelu_tanh" ? 2 : act == "relu" ? 3 : 0;
      if (impl->layers.empty()) impl->in_features = l.in;
      width = l.in;
    } else {
      throw std::runtime_error("unknown layer type: " + op);
    }
    impl->layers.push_back(std::move(l));
  }
  if (impl->layers.empty()) throw std::runtime_error("empty graph");
  impl->out_features = width;
  Graph g;
  g.impl_ = impl;
  return g;
}

int64_t Graph::in_features() const { return impl_->in_features; }
int64_t Graph::out_features() const { return impl_->out_features; }

Tensor Graph::Forward(const Tensor& input) const {
  if (input.shape().NumAxes() != 2 || input.shape().At(1) != impl_->in_features)
    throw std::runtime_error("Forward: input must be [rows, in_features]");
  check_cuda(cudaSetDevice(impl_->device), "cudaSetDevice");
  const int64_t rows = input.shape().At(0);
  Tensor cur = input;
  for (const Layer& l : impl_->layers) {
    Tensor next = Tensor::empty(Shape{rows, l.out}, impl_->device);
    if (l.kind == 0) {
      OfbGemmArgs a;
      std::memset(&a, 0, sizeof(a));
      a.A = cur.data(); a.lda = l.in;
      a.B = l.w.get(); a.ldb = l.in;
      a.C = next.data(); a.ldc = l.out;
      a.bias = l.b ? l.b.get() : nullptr;
      a.M = static_cast<int>(rows); a.N = static_cast<int>(l.out); a.K = static_cast<int>(l.in);
      a.act = l.act;
      a.alpha = 1.f;
      check_ofb(ofb_gemm_bf16(&a, nullptr), "gemm");
    } else if (l.kind == 1) {
      auto stats = device_alloc(static_cast<size_t>(rows) * 8, impl_->device);
      float* mean = static_cast<float*>(stats.get());
      check_ofb(ofb_layer_norm_fwd(cur.data(), l.w.get(), l.b.get(), next.data(), mean, mean + rows, static_cast<int>(rows),
                                   static_cast<int>(l.in), l.eps, nullptr), "layer_norm");
      check_cuda(cudaDeviceSynchronize(), "layer_norm");   // the statistics buffer is released right after
    } else {
      check_ofb(ofb_bias_act_fwd(cur.data(), nullptr, next.data(), rows * l.in, static_cast<int>(l.in), l.act, nullptr), "activation");
    }
    cur = next;
  }
  check_cuda(cudaDeviceSynchronize(), "Forward");
  return cur;
}

}  // namespace oneflow_api

// ------------------------------------------------------------------------------------------------ C ABI
extern "C" {

const char* ofb_api_last_error(void) { return oneflow_api::g_error.c_str(); }

void* ofb_api_graph_load(const char* dir, int device) {
  try {
    return new oneflow_api::Graph(oneflow_api::Graph::Load(dir, device));
  } catch (const std::exception& e) {
    oneflow_api::g_error = e.what();
    return nullptr;
  }
}
long long ofb_api_graph_in_features(void* g) { return static_cast<oneflow_api::Graph*>(g)->in_features(); }
long long ofb_api_graph_out_features(void* g) { return static_cast<oneflow_api::Graph*>(g)->out_features(); }

int ofb_api_graph_forward(void* g, const float* x, long long rows, float* y) {
  try {
    auto* graph = static_cast<oneflow_api::Graph*>(g);
    auto in = oneflow_api::Tensor::from_buffer(x, oneflow_api::Shape{rows, graph->in_features()});
    auto out = graph->Forward(in).to_host();
    std::memcpy(y, out.data(), out.size() * sizeof(float));
    return 0;
  } catch (const std::exception& e) {
    oneflow_api::g_error = e.what();
    return -1;
  }
}
void ofb_api_graph_free(void* g) { delete static_cast<oneflow_api::Graph*>(g); }
}
