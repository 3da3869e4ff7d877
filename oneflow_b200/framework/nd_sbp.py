"""Geometry of n-D SBP: which slice of the logical tensor a rank holds, local shapes, and the copy-cost
model used to choose between SBP signatures.

Reference: GetTensorSliceView4ParallelId / GetPhysicalShape (oneflow/core/job/nd_sbp_util.cpp:58-109),
copy-cost rules (oneflow/core/framework/sbp_infer_util.cpp:75-150).
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

from .balanced_splitter import BalancedSplitter


def slice_view(logical_shape: Sequence[int], hierarchy: Sequence[int], nd_sbp, coords: Sequence[int]) -> List[Tuple[int, int]]:
    """[begin, end) per dimension of the part of the logical tensor held at mesh coordinates `coords`.
    Splits on the same tensor dimension by several mesh axes nest in mesh-axis order."""
    ranges = [(0, int(s)) for s in logical_shape]
    for axis, s in enumerate(nd_sbp):
        if s.kind != "S":
            continue
        d = s.axis
        if d >= len(ranges):
            raise ValueError(f"split axis {d} out of range for a {len(ranges)}-d tensor")
        b, e = ranges[d]
        lo, hi = BalancedSplitter(e - b, hierarchy[axis]).at(coords[axis])
        ranges[d] = (b + lo, b + hi)
    return ranges


def local_shape(logical_shape, hierarchy, nd_sbp, coords):
    return tuple(e - b for b, e in slice_view(logical_shape, hierarchy, nd_sbp, coords))


def logical_shape_from_local(local_shapes_by_coord, hierarchy, nd_sbp, my_coords, my_local_shape):
    """Logical shape implied by this rank's local shape under even splits (used when check_meta is off)."""
    shape = list(my_local_shape)
    for axis, s in enumerate(nd_sbp):
        if s.kind == "S":
            shape[s.axis] *= hierarchy[axis]
    return tuple(shape)


def copy_cost(in_sbp, out_sbp, nbytes: float, n: int, same_placement: bool = True) -> float:
    """Bytes-moved estimate for converting one mesh axis from in_sbp to out_sbp over n ranks."""
    if not same_placement:
        cost = nbytes
        if out_sbp.kind == "B":
            cost += (n - 1) * nbytes
        if in_sbp.kind == "P":
            cost += (n - 1) * nbytes
        return cost
    if in_sbp == out_sbp:
        return 0.0
    if out_sbp.kind == "P":
        return 1.0  # small penalty: produces zeros on all ranks but one
    if in_sbp.kind == "B" and out_sbp.kind == "S":
        return 1.0
    if in_sbp.kind == "S" and out_sbp.kind == "S":
        return nbytes * (n - 1) / n
    if in_sbp.kind == "P" and out_sbp.kind == "S":
        return nbytes * (n - 1)
    if in_sbp.kind == "S" and out_sbp.kind == "B":
        return nbytes * (n - 1)
    if in_sbp.kind == "P" and out_sbp.kind == "B":
        return 2 * nbytes * (n - 1)
    return nbytes


def nd_copy_cost(in_nd, out_nd, nbytes, hierarchy):
    return sum(copy_cost(a, b, nbytes, n) for a, b, n in zip(in_nd, out_nd, hierarchy))
