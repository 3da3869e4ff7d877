"""bf16 GEMM with fused epilogues on the tcgen05 kernel (csrc/kernels/gemm_tcgen05.cuh).

``gemm`` is the single entry point: forward Linear (x[M,K] @ w[N,K]^T), data gradient
(dy[M,N] @ w[N,K], w read "MN-major") and weight gradient (dy^T @ x, both operands
"MN-major") all map onto it without materialising a transpose. CPU tensors take a plain
PyTorch fp32 path with identical semantics so that host-only tests exercise the same
call sites; CUDA tensors always run the native kernel.

Counterpart in the reference: ``oneflow/user/kernels/matmul_kernels.cpp`` (matmul :185),
``cublas_fused_mlp_kernel.cu`` and ``fused_matmul_bias_kernel.cu`` epilogues.
"""
from __future__ import annotations

import torch

from . import _native

ACT_NONE, ACT_GELU, ACT_GELU_TANH, ACT_RELU = 0, 1, 2, 3
_ACT_NAMES = {None: 0, "none": 0, "gelu": 1, "gelu_tanh": 2, "relu": 3}


def _act_code(act):
    return act if isinstance(act, int) else _ACT_NAMES[act]


def _act_ref(v, act):
    if act == ACT_GELU:
        return torch.nn.functional.gelu(v)
    if act == ACT_GELU_TANH:
        return torch.nn.functional.gelu(v, approximate="tanh")
    if act == ACT_RELU:
        return torch.relu(v)
    return v


def _act_grad_ref(h, act):
    h = h.detach().clone().requires_grad_(True)
    with torch.enable_grad():
        y = _act_ref(h, act).sum()
    (g,) = torch.autograd.grad(y, h)
    return g


def gemm_reference(a, b, a_layout="mk", b_layout="nk", bias=None, act=0, residual=None, aux_in=None,
                   want_aux=False, out=None, out_dtype=torch.bfloat16, accumulate=False, alpha=1.0):
    """fp32 PyTorch statement of what the kernel computes (oracle for tests, CPU path)."""
    act = _act_code(act)
    A = a.float() if a_layout == "mk" else a.float().t()
    B = b.float() if b_layout == "nk" else b.float().t()
    v = alpha * (A @ B.t())
    if bias is not None:
        v = v + bias.float()
    aux = v.to(torch.bfloat16) if want_aux else None
    if aux_in is not None:
        v = v * _act_grad_ref(aux_in.float(), act)
    elif act:
        v = _act_ref(v, act)
    if residual is not None:
        v = v + residual.float()
    if accumulate and out is not None:
        v = v + out.float()
    res = v.to(out_dtype)
    if out is not None:
        out.copy_(res)
        res = out
    return (res, aux) if want_aux else res


def _check_operand(t, name):
    if t.dtype != torch.bfloat16:
        raise TypeError(f"gemm: {name} must be bfloat16, got {t.dtype}")
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"gemm: {name} must be 2-D with a contiguous last dimension")
    if t.stride(0) % 8 != 0 or t.data_ptr() % 16 != 0:
        raise ValueError(f"gemm: {name} needs a 16-byte aligned base and a leading dimension that is a multiple of 8")


def gemm(a, b, *, a_layout="mk", b_layout="nk", bias=None, act=0, residual=None, aux_in=None, want_aux=False,
         out=None, out_dtype=torch.bfloat16, accumulate=False, alpha=1.0, bn=0, max_ctas=0):
    """``out = epilogue(alpha * A @ B^T)`` with A logical [M,K] and B logical [N,K].

    a_layout: "mk" (a is [M,K]) or "km" (a is [K,M]);  b_layout: "nk" (b is [N,K]) or "kn" (b is [K,N]).
    Epilogue order: +bias -> (aux_out = pre-activation) -> act  (or  *act'(aux_in))  -> +residual -> (+out).
    Returns ``out`` or ``(out, aux)`` when ``want_aux``.
    """
    act = _act_code(act)
    if not a.is_cuda:
        return gemm_reference(a, b, a_layout, b_layout, bias, act, residual, aux_in, want_aux, out, out_dtype,
                              accumulate, alpha)
    _check_operand(a, "a")
    _check_operand(b, "b")
    M, K = (a.shape if a_layout == "mk" else (a.shape[1], a.shape[0]))
    N, Kb = (b.shape if b_layout == "nk" else (b.shape[1], b.shape[0]))
    if K != Kb:
        raise ValueError(f"gemm: reduction sizes differ ({K} vs {Kb})")
    if N % 8 != 0:
        raise ValueError("gemm: N must be a multiple of 8")
    if out is None:
        if accumulate:
            raise ValueError("gemm: accumulate needs `out`")
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    else:
        if out.shape != (M, N) or out.stride(1) != 1:
            raise ValueError("gemm: bad `out`")
        out_dtype = out.dtype
    if out_dtype not in (torch.bfloat16, torch.float32):
        raise TypeError("gemm: output must be bfloat16 or float32")
    aux = torch.empty((M, N), dtype=torch.bfloat16, device=a.device) if want_aux else None
    args = _native.GemmArgs()
    args.A, args.B, args.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.bias = bias.data_ptr() if bias is not None else None
    args.residual = residual.data_ptr() if residual is not None else None
    args.aux_in = aux_in.data_ptr() if aux_in is not None else None
    args.aux_out = aux.data_ptr() if aux is not None else None
    args.lda, args.ldb, args.ldc = a.stride(0), b.stride(0), out.stride(0)
    args.ldr = residual.stride(0) if residual is not None else 0
    args.ld_aux = aux_in.stride(0) if aux_in is not None else (aux.stride(0) if aux is not None else 0)
    args.M, args.N, args.K = M, N, K
    args.a_mn_major = 0 if a_layout == "mk" else 1
    args.b_mn_major = 0 if b_layout == "nk" else 1
    args.act, args.out_fp32, args.accumulate = act, int(out_dtype == torch.float32), int(bool(accumulate))
    args.bn, args.max_ctas, args.alpha = bn, max_ctas, float(alpha)
    for t, nm in ((bias, "bias"), (residual, "residual"), (aux_in, "aux_in")):
        if t is not None and (t.dtype != torch.bfloat16 or t.data_ptr() % 16 != 0):
            raise TypeError(f"gemm: {nm} must be 16-byte aligned bfloat16")
    lib = _native.kernels()
    if _native._recorder is not None:
        for t in (a, b, out, bias, residual, aux_in, aux):
            if t is not None:
                _native._recorder.saw_tensor(t)
        _native._recorder.note(flops=2.0 * M * N * K, attrs=f"act={act} a={a_layout} b={b_layout}")
    _native.check(lib.ofb_gemm_bf16(args, _native.stream_ptr()), "ofb_gemm_bf16")
    from . import kernels as _k
    _k._count()
    return (out, aux) if want_aux else out
