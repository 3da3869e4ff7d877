// Minimal C++ program on the inference API: load an exported graph directory, feed inputs read from raw files, print the
// outputs. Built by the tests against libofb_api.so:
//     g++ -std=c++17 run_graph.cpp -I<csrc/api> -L<lib> -lofb_api -Wl,-rpath,<lib> -o run_graph
//     ./run_graph <graph dir> <device: -1 host, >= 0 GPU> <input file per graph input ...>
// An input file holds little-endian float32 values (for bf16 graph inputs) or int64 values (for id inputs) in the
// exported shape. Every output is printed as one line of numbers.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <vector>

#include "oneflow_api.h"

template <typename T>
static std::vector<T> read_file(const std::string& path, int64_t n) {
  std::ifstream f(path, std::ios::binary);
  std::vector<T> v(static_cast<size_t>(n));
  f.read(reinterpret_cast<char*>(v.data()), static_cast<std::streamsize>(n * sizeof(T)));
  if (static_cast<int64_t>(f.gcount()) != static_cast<int64_t>(n * sizeof(T))) {
    std::cerr << "short read: " << path << "\n";
    std::exit(2);
  }
  return v;
}

int main(int argc, char** argv) {
  if (argc < 4) {
    std::cerr << "usage: run_graph <dir> <device> <input files...>\n";
    return 2;
  }
  try {
    const int device = std::atoi(argv[2]);
    oneflow_api::Graph graph = oneflow_api::Graph::Load(argv[1], device, 2);
    if (argc - 3 != graph.num_inputs()) {
      std::cerr << "the graph takes " << graph.num_inputs() << " inputs\n";
      return 2;
    }
    std::vector<oneflow_api::Tensor> inputs;
    for (int i = 0; i < graph.num_inputs(); ++i) {
      const oneflow_api::Shape shape = graph.input_shape(i);
      if (graph.input_dtype(i) == oneflow_api::DType::kInt64) {
        auto v = read_file<int64_t>(argv[3 + i], shape.elem_cnt());
        inputs.push_back(oneflow_api::Tensor::from_int64(v.data(), shape, device));
      } else {
        auto v = read_file<float>(argv[3 + i], shape.elem_cnt());
        inputs.push_back(oneflow_api::Tensor::from_buffer(v.data(), shape, device));
      }
    }
    const std::vector<oneflow_api::Tensor> outputs = graph.Forward(inputs);
    const oneflow_api::PlanStats st = graph.stats();
    std::cerr << "ops " << st.n_ops << " streams " << st.n_streams_used << " peak bytes " << st.arena_bytes << "\n";
    for (const auto& t : outputs) {
      const std::vector<float> host = t.to_host();
      for (size_t k = 0; k < host.size(); ++k) std::printf(k ? " %.6g" : "%.6g", host[k]);
      std::printf("\n");
    }
  } catch (const std::exception& e) {
    std::cerr << "error: " << e.what() << "\n";
    return 1;
  }
  return 0;
}
