// Placement / SBP geometry shared with the Python layer (oneflow_b200/framework/{balanced_splitter,nd_sbp}.py).
// Reference behaviour: BalancedSplitter (oneflow/core/common/balanced_splitter.cpp:19-43),
// GetTensorSliceView4ParallelId (oneflow/core/job/nd_sbp_util.cpp:58-109), copy cost
// (oneflow/core/framework/sbp_infer_util.cpp:75-150).
#include <vector>

#include "common.h"
#include "ofc_core.h"

OFC_API const char* ofc_last_error(void) { return ofc::last_error().c_str(); }

OFC_API void ofc_balanced_split(int64_t total, int64_t parts, int64_t idx, int64_t* begin, int64_t* end) {
  const int64_t base = total / parts, rem = total % parts;
  const int64_t b = idx * base + (idx < rem ? idx : rem);
  *begin = b;
  *end = b + base + (idx < rem ? 1 : 0);
}

OFC_API int ofc_slice_view(const int64_t* logical_shape, int ndim, const int64_t* hierarchy, int mesh_ndim, const int* sbp_kind,
                           const int* sbp_axis, const int64_t* coords, int64_t* ranges_out) {
  for (int d = 0; d < ndim; ++d) {
    ranges_out[2 * d] = 0;
    ranges_out[2 * d + 1] = logical_shape[d];
  }
  for (int a = 0; a < mesh_ndim; ++a) {
    if (sbp_kind[a] != 2) continue;
    const int d = sbp_axis[a];
    if (d < 0 || d >= ndim) return ofc::fail("split axis out of range");
    const int64_t b = ranges_out[2 * d], e = ranges_out[2 * d + 1];
    int64_t lo, hi;
    ofc_balanced_split(e - b, hierarchy[a], coords[a], &lo, &hi);
    ranges_out[2 * d] = b + lo;
    ranges_out[2 * d + 1] = b + hi;
  }
  return 0;
}

OFC_API double ofc_copy_cost(int in_kind, int in_axis, int out_kind, int out_axis, double nbytes, int n, int same_placement) {
  if (!same_placement) {
    double c = nbytes;
    if (out_kind == 0) c += (n - 1) * nbytes;
    if (in_kind == 1) c += (n - 1) * nbytes;
    return c;
  }
  if (in_kind == out_kind && (in_kind != 2 || in_axis == out_axis)) return 0.0;
  if (out_kind == 1) return 1.0;
  if (in_kind == 0 && out_kind == 2) return 1.0;
  if (in_kind == 2 && out_kind == 2) return nbytes * (n - 1) / n;
  if (in_kind == 1 && out_kind == 2) return nbytes * (n - 1);
  if (in_kind == 2 && out_kind == 0) return nbytes * (n - 1);
  if (in_kind == 1 && out_kind == 0) return 2 * nbytes * (n - 1);
  return nbytes;
}
