// C++ inference API: load an exported network and run it on the GPU without Python.
//
//   #include "oneflow_api.h"
//   auto graph = oneflow_api::Graph::Load("model_dir");            // reads graph.txt + raw bf16 weight files
//   oneflow_api::Tensor x = oneflow_api::Tensor::from_buffer(host_floats, {batch, features});
//   oneflow_api::Tensor y = graph.Forward(x);                      // tcgen05 GEMMs with fused bias/activation, LayerNorm
//   std::vector<float> out = y.to_host();
//
// The directory is written by oneflow_b200.utils.export.export_inference_graph (feed-forward stacks of Linear,
// ReLU / GELU and LayerNorm). A C ABI (ofb_api_*) wraps the same objects for other languages.
//
// Reference counterpart: oneflow/api/cpp/ (oneflow_api::Tensor, Shape, Graph::Load(dir) running a saved nn.Graph).
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

 private:
  std::vector<int64_t> dims_;
};

// A bf16 tensor in device memory (shared ownership).
class Tensor {
 public:
  Tensor() = default;
  static Tensor from_buffer(const float* host, const Shape& shape, int device = 0);
  static Tensor empty(const Shape& shape, int device = 0);
  std::vector<float> to_host() const;
  const Shape& shape() const { return shape_; }
  void* data() const { return data_.get(); }
  int device() const { return device_; }

 private:
  Shape shape_;
  std::shared_ptr<void> data_;
  int device_ = 0;
};

class Graph {
 public:
  static Graph Load(const std::string& dir, int device = 0);
  Tensor Forward(const Tensor& input) const;
  int64_t in_features() const;
  int64_t out_features() const;
  struct Impl;

 private:
  std::shared_ptr<Impl> impl_;
};

}  // namespace oneflow_api

extern "C" {
void* ofb_api_graph_load(const char* dir, int device);
long long ofb_api_graph_in_features(void* graph);
long long ofb_api_graph_out_features(void* graph);
// x: host fp32 [rows, in_features]; y: host fp32 [rows, out_features]. Returns 0 on success.
int ofb_api_graph_forward(void* graph, const float* x, long long rows, float* y);
void ofb_api_graph_free(void* graph);
const char* ofb_api_last_error(void);
}
