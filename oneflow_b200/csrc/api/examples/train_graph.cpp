// Minimal C++ training program on the graph API: load an exported graph whose first output is a loss as a training step,
// run a number of steps on inputs read from raw files, print the loss of every step, save the result as a directory that
// loads again (for inference, or to continue training). Built by the tests against libofb_api.so:
//     g++ -std=c++17 train_graph.cpp -I<csrc/api> -L<lib> -lofb_api -Wl,-rpath,<lib> -o train_graph
//     ./train_graph [--recompute=cheap|full] <graph dir> <device: -1 host, >= 0 GPU> <steps> <learning rate> <save dir or -> <input file per graph input ...>
// An input file holds little-endian float32 values (for bf16 graph inputs) or int64 values (for id inputs) in the exported
// shape; the same batch is used for every step.
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <iostream>
#include <string>
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
  std::string recompute;
  if (argc > 1 && std::string(argv[1]).rfind("--recompute=", 0) == 0) {
    recompute = std::string(argv[1]).substr(12);
    --argc;
    ++argv;
  }
  if (argc < 7) {
    std::cerr << "usage: train_graph <dir> <device> <steps> <lr> <save dir or -> <input files...>\n";
    return 2;
  }
  try {
    const int device = std::atoi(argv[2]), steps = std::atoi(argv[3]);
    oneflow_api::TrainOptions options;
    options.optimizer = "adamw";
    options.lr = static_cast<float>(std::atof(argv[4]));
    options.recompute_cheap_activations = recompute == "cheap";
    options.recompute_all_but_residual_stream = recompute == "full";
    oneflow_api::Graph graph = oneflow_api::Graph::LoadTraining(argv[1], options, device, 2);
    if (argc - 6 != graph.num_inputs()) {
      std::cerr << "the graph takes " << graph.num_inputs() << " inputs\n";
      return 2;
    }
    std::vector<oneflow_api::Tensor> inputs;
    for (int i = 0; i < graph.num_inputs(); ++i) {
      const oneflow_api::Shape shape = graph.input_shape(i);
      if (graph.input_dtype(i) == oneflow_api::DType::kInt64) {
        auto v = read_file<int64_t>(argv[6 + i], shape.elem_cnt());
        inputs.push_back(oneflow_api::Tensor::from_int64(v.data(), shape, device));
      } else {
        auto v = read_file<float>(argv[6 + i], shape.elem_cnt());
        inputs.push_back(oneflow_api::Tensor::from_buffer(v.data(), shape, device));
      }
    }
    std::cerr << graph.num_parameters() << " trainable parameters, first: " << graph.parameter_name(0) << " (" << graph.parameter_numel(0)
              << " elements)\n";
    for (int s = 0; s < steps; ++s) {
      const std::vector<oneflow_api::Tensor> outputs = graph.Forward(inputs);   // forward, backward and update
      std::printf("%.6g\n", outputs.at(0).to_host().at(0));
    }
    const oneflow_api::PlanStats st = graph.stats();
    std::cerr << "steps " << graph.steps() << " ops " << st.n_ops << " streams " << st.n_streams_used << " peak bytes " << st.arena_bytes
              << " graph replays " << st.graph_replays << "\n";
    if (std::string(argv[5]) != "-") graph.Save(argv[5]);
  } catch (const std::exception& e) {
    std::cerr << "error: " << e.what() << "\n";
    return 1;
  }
  return 0;
}
