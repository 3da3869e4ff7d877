// Internal interface between the Tensor / C ABI part (oneflow_api.cpp) and the graph compiler + executor
// (graph_runtime.cpp).
#pragma once
#include <cstdint>
#include <memory>
#include <string>

#include "oneflow_api.h"

namespace oneflow_api {

namespace detail {
extern thread_local std::string g_error;
void check_cuda(int e, const char* what);
uint16_t to_bf16(float f);
float from_bf16(uint16_t h);
std::shared_ptr<void> storage_alloc(size_t bytes, int device);
void copy_in(void* dst, const void* host, size_t bytes, int device);
void copy_out(void* host, const void* src, size_t bytes, int device);
}  // namespace detail

inline bool graph_input_is_int64(const Graph& g, int i) { return g.input_dtype(i) == DType::kInt64; }
inline int graph_device(const Graph& g) { return g.device(); }
inline void graph_rebind_rows(Graph& g, int64_t rows) { g.BindRows(rows); }

}  // namespace oneflow_api
