"""Export of networks for the C++ inference API (csrc/api/oneflow_api.h).

``export_graph(module, example_inputs, directory)`` records the operator graph of ``module`` on the example inputs (static
shapes) and writes ``graph.txt`` (tensors, operators, inputs, outputs) plus one raw file per parameter; the C++ side compiles
it into a plan (memory sharing, dependencies, streams) and runs it on the sm_100a kernels or on its host implementation.
``export_inference_graph(module, directory)`` is the older layer-list form: it walks an ``nn.Sequential`` (nested ones are flattened) of Linear, ReLU,
GELU and LayerNorm layers and writes ``graph.txt`` plus one raw bf16 file per parameter; an activation that follows a
Linear is folded into that layer's GEMM epilogue. ``InferenceGraph`` loads such a directory through the C ABI of
``libofb_api.so`` (what a C++ program does with ``oneflow_api::Graph::Load``).

A module whose forward returns a scalar loss (``F.cross_entropy`` / ``F.mse_loss`` or the loss modules) exports the same way
(use ``fuse=False``); ``TrainingGraph`` loads it as a training step: the C++ side appends the backward and optimizer operators
and compiles forward, backward and update into one plan.

Reference: oneflow/api/cpp (Graph::Load of a saved nn.Graph), python/oneflow/framework/check_point_v2.py save(..., save_as_external_data)."""
from __future__ import annotations

import ctypes
import os

import numpy as np
import torch


def _flatten(module):
    if isinstance(module, torch.nn.Sequential):
        for m in module:
            yield from _flatten(m)
    else:
        yield module


def _act_name(m):
    if isinstance(m, torch.nn.ReLU):
        return "relu"
    if isinstance(m, torch.nn.GELU):
        return "gelu_tanh" if getattr(m, "approximate", "none") == "tanh" else "gelu"
    return None


def _write_bf16(path, t):
    t.detach().to(torch.bfloat16).contiguous().cpu().view(torch.int16).numpy().tofile(path)


def export_inference_graph(module, directory):
    os.makedirs(directory, exist_ok=True)
    layers = list(_flatten(module))
    lines = ["oneflow_b200 inference graph v1"]
    i, width = 0, None
    while i < len(layers):
        m = layers[i]
        if isinstance(m, torch.nn.Linear):
            act = _act_name(layers[i + 1]) if i + 1 < len(layers) else None
            wf = f"p{i}.weight.bin"
            _write_bf16(os.path.join(directory, wf), m.weight)
            bf = "-"
            if m.bias is not None:
                bf = f"p{i}.bias.bin"
                _write_bf16(os.path.join(directory, bf), m.bias)
            lines.append(f"linear {m.in_features} {m.out_features} {wf} {bf} {act or 'none'}")
            width = m.out_features
            i += 2 if act else 1
        elif isinstance(m, torch.nn.LayerNorm):
            if len(m.normalized_shape) != 1:
                raise ValueError("only LayerNorm over the last dimension can be exported")
            n = m.normalized_shape[0]
            gf, bf = f"p{i}.gamma.bin", f"p{i}.beta.bin"
            _write_bf16(os.path.join(directory, gf), m.weight if m.weight is not None else torch.ones(n))
            _write_bf16(os.path.join(directory, bf), m.bias if m.bias is not None else torch.zeros(n))
            lines.append(f"layer_norm {n} {gf} {bf} {m.eps}")
            width = n
            i += 1
        elif _act_name(m) is not None:
            if width is None:
                raise ValueError("an activation cannot be the first layer (its width is unknown)")
            lines.append(f"activation {width} {_act_name(m)}")
            i += 1
        elif isinstance(m, (torch.nn.Dropout, torch.nn.Identity)):
            i += 1
        else:
            raise ValueError(f"cannot export layer of type {type(m).__name__}")
    with open(os.path.join(directory, "graph.txt"), "w") as f:
        f.write("\n".join(lines) + "\n")
    return directory


# ------------------------------------------------------------------------------------------------ operator-graph export
import math
import operator

import torch.fx
import torch.nn.functional as F


_UNARY = {"scale": 0, "gelu": 1, "gelu_tanh": 2, "relu": 3, "tanh": 4, "sigmoid": 5, "silu": 6, "add_scalar": 7, "exp": 8, "rsqrt": 9,
          "square": 10}
_BINARY = {"add": 0, "sub": 1, "mul": 2, "div": 3, "maximum": 4, "minimum": 5}
_INPLACE = {"iadd": "add", "imul": "mul", "isub": "sub", "itruediv": "div", "add_": "add", "mul_": "mul", "sub_": "sub", "div_": "div",
            "relu_": "relu", "tanh_": "tanh", "sigmoid_": "sigmoid"}


class _GraphEmitter(torch.fx.Interpreter):
    """Runs the traced module on the example inputs and writes one IR operator per computing node.

    Invariant: every tensor the interpreter holds is laid out in its torch storage exactly as in the IR tensor that stands for
    that storage (a flat "root" tensor per storage). View operations therefore need no IR at all: a consumer reads the view's
    shape, strides and offset off the torch tensor. Where torch would hand back a result in another layout (an element-wise
    op on a permuted input keeps the permutation; attention returns [B, H, S, D]) the node's value is replaced by an equal
    tensor in the layout the IR operator writes."""

    def __init__(self, gm, directory):
        super().__init__(gm)
        self.dir = directory
        self.tensors = []          # IR tensor records (without the leading "tensor <id>")
        self.ops = []              # dicts: type, in, out, attr
        self.inputs, self.outputs = [], []
        self.roots = {}            # torch storage pointer -> IR id of the flat tensor standing for that storage
        self.keep = []             # tensors kept alive so that storage pointers stay unique
        self.alias_cache = {}
        self.copy_cache = {}
        # parameters that own their whole storage and take gradients: named in the IR, which makes them trainable there
        self.n_dropout = 0
        self.pending_log_softmax = {}     # storage of a log_softmax result -> the logits it was computed from
        self.param_names = {}
        for name, prm in gm.named_parameters():
            if prm.requires_grad and prm.dtype.is_floating_point and prm.storage_offset() == 0 and \
                    prm.untyped_storage().nbytes() == prm.numel() * prm.element_size():
                self.param_names.setdefault(prm.untyped_storage().data_ptr(), name)

    # ---- IR helpers
    @staticmethod
    def _dtype(t):
        if t.dtype.is_floating_point:
            return "bf16"
        if t.dtype in (torch.int64, torch.int32):
            return "i64"
        raise ValueError(f"cannot export tensors of dtype {t.dtype}")

    def _new_tensor(self, dtype, kind, shape, extra=""):
        self.tensors.append(f"{dtype} {kind} {len(shape)} " + " ".join(str(int(d)) for d in shape) + (" " + extra if extra else ""))
        return len(self.tensors) - 1

    def _kind(self, tid):
        return self.tensors[tid].split()[1]

    def _register(self, real, kind, extra=""):
        """``real`` owns a fresh storage that it fills contiguously: a new flat IR tensor stands for it."""
        assert real.is_contiguous() and real.storage_offset() == 0
        rid = self._new_tensor(self._dtype(real), kind, [max(real.numel(), 1)], extra)
        self.keep.append(real)
        self.roots[real.untyped_storage().data_ptr()] = rid
        return rid

    def _root(self, real):
        if real.untyped_storage().data_ptr() in self.pending_log_softmax:
            raise ValueError("log_softmax is exported only as the input of nll_loss (the pair becomes one cross_entropy operator)")
        rid = self.roots.get(real.untyped_storage().data_ptr())
        if rid is None:
            rid = self._constant(real)
        return rid

    def _constant(self, real):
        """A tensor that does not depend on the inputs (a parameter, a buffer, a table built in forward): saved as a file."""
        n_storage = real.untyped_storage().nbytes() // real.element_size()
        whole = torch.as_strided(real.detach(), (n_storage,), (1,), 0)       # the storage in its own order
        name = f"t{len(self.tensors)}.bin"
        if self._dtype(real) == "bf16":
            _write_bf16(os.path.join(self.dir, name), whole)
        else:
            whole.to(torch.int64).cpu().numpy().tofile(os.path.join(self.dir, name))
        pname = self.param_names.get(real.untyped_storage().data_ptr())
        rid = self._new_tensor(self._dtype(real), "param", [n_storage], f"file={name}" + (f" name={pname}" if pname else ""))
        self.keep.append(real)
        self.roots[real.untyped_storage().data_ptr()] = rid
        return rid

    def _alias(self, root, offset, shape):
        shape = tuple(int(d) for d in shape)
        key = (root, int(offset), shape)
        if key not in self.alias_cache:
            self.alias_cache[key] = self._new_tensor(self.tensors[root].split()[0], self._kind(root), shape, f"alias={root} offset={int(offset)}")
        return self.alias_cache[key]

    def _operand(self, real):
        """IR id of a contiguous tensor holding ``real``: an alias of its storage, or a strided copy when it is not contiguous."""
        root = self._root(real)
        if real.is_contiguous():
            return self._alias(root, real.storage_offset(), real.shape)
        key = (root, real.storage_offset(), tuple(real.shape), tuple(real.stride()))
        if key not in self.copy_cache:
            if real.dim() > 5:
                raise ValueError("strided copies support at most 5 axes")
            n = real.numel()
            rid = self._new_tensor(self._dtype(real), "act", [n])
            out_strides = torch.empty(real.shape, device="meta").stride()
            self.ops.append({"type": "copy", "in": [root], "out": [rid],
                             "attr": {"shape": ",".join(map(str, real.shape)), "in_strides": ",".join(map(str, real.stride())),
                                      "in_offset": int(real.storage_offset()), "out_strides": ",".join(map(str, out_strides)),
                                      "out_offset": 0}})
            self.copy_cache[key] = (rid, len(self.ops))
        rid, _ = self.copy_cache[key]
        return self._alias(rid, 0, real.shape)

    def _result(self, real):
        """Fresh activation for an operator's result: (IR id to write, the tensor to hand on), laid out contiguously."""
        real = real.contiguous() if not (real.is_contiguous() and real.storage_offset() == 0) else real
        if real.untyped_storage().data_ptr() in self.roots:
            real = real.clone()
        rid = self._register(real, "act")
        return self._alias(rid, 0, real.shape), real

    def _emit(self, type_, ins, out, **attr):
        self.copy_cache.clear()       # a cached copy is only valid until something may have rewritten its source
        self.ops.append({"type": type_, "in": list(ins), "out": [out], "attr": attr})

    # ---- operators: each returns the tensor that stands for the node from here on
    def _unary(self, x, y, fn, alpha=1.0, inplace=False):
        ix = self._operand(x)
        if inplace:
            if not x.is_contiguous():
                raise ValueError("an in-place operator on a strided view cannot be exported")
            self._emit("unary", [ix], ix, fn=_UNARY[fn], alpha=repr(float(alpha)))
            return y
        out, y = self._result(y)
        self._emit("unary", [ix], out, fn=_UNARY[fn], alpha=repr(float(alpha)))
        return y

    def _binary(self, a, b, y, fn, inplace=False):
        if not torch.is_tensor(b) or not torch.is_tensor(a):
            t, c = (a, b) if torch.is_tensor(a) else (b, a)
            c = float(c)
            if fn == "add":
                return self._unary(t, y, "add_scalar", c, inplace)
            if fn == "mul":
                return self._unary(t, y, "scale", c, inplace)
            if fn == "sub" and torch.is_tensor(a):
                return self._unary(t, y, "add_scalar", -c, inplace)
            if fn == "div" and torch.is_tensor(a):
                return self._unary(t, y, "scale", 1.0 / c, inplace)
            if fn == "sub" and not inplace:                      # c - t = (-t) + c
                return self._unary(self._unary(t, -t, "scale", -1.0), y, "add_scalar", c)
            raise ValueError(f"cannot export scalar {fn} with the tensor on the right")
        if tuple(a.shape) != tuple(y.shape):
            if not inplace and fn in ("add", "mul", "maximum", "minimum") and tuple(b.shape) == tuple(y.shape):
                a, b = b, a
            else:
                raise ValueError(f"cannot export {fn}: the first operand {tuple(a.shape)} is broadcast to {tuple(y.shape)}")
        cols = 1
        bs = list(b.shape)
        while bs and bs[0] == 1:
            bs.pop(0)                                   # leading broadcast axes
        tail = list(bs)
        while tail and tail[-1] == 1:
            tail.pop()                                  # trailing broadcast axes
        if tuple(b.shape) == tuple(y.shape):
            mode = 0
        elif bs and tuple(y.shape[y.dim() - len(bs):]) == tuple(bs):
            mode, cols = 1, b.numel()                   # b repeats over the leading axes: y as [rows, cols] with cols = |b|
        elif b.dim() == y.dim() and tail and tuple(b.shape[:len(tail)]) == tuple(y.shape[:len(tail)]) and b.numel() == math.prod(tail):
            mode, cols = 2, y.numel() // b.numel()      # one value of b per leading index
        else:
            # any other broadcast (axes of length 1 in the middle, ...): the expanded operand is materialised by a strided copy
            try:
                b = b.expand(y.shape)
            except RuntimeError:
                raise ValueError(f"cannot export {fn} of shapes {tuple(a.shape)} and {tuple(b.shape)}") from None
            mode = 0
        ia, ib = self._operand(a), self._operand(b)
        if inplace:
            if not a.is_contiguous():
                raise ValueError("an in-place operator on a strided view cannot be exported")
            self._emit("binary", [ia, ib], ia, fn=_BINARY[fn], bmode=mode, cols=cols)
            return y
        out, y = self._result(y)
        self._emit("binary", [ia, ib], out, fn=_BINARY[fn], bmode=mode, cols=cols)
        return y

    def _linear(self, x, w, b, y):
        ins = [self._operand(x), self._operand(w), self._operand(b) if b is not None else -1, -1]
        out, y = self._result(y)
        self._emit("linear", ins, out, act="none")
        return y

    def _layer_norm(self, x, shape, w, b, eps, y):
        if len(shape) != 1:
            raise ValueError("only LayerNorm over the last dimension can be exported")
        n = int(shape[0])
        w = w if w is not None else torch.ones(n)
        b = b if b is not None else torch.zeros(n)
        ins = [self._operand(x), self._operand(w), self._operand(b)]
        out, y = self._result(y)
        self._emit("layer_norm", ins, out, eps=repr(float(eps)))
        return y

    def _rms_norm(self, x, shape, w, eps, y):
        """RMSNorm on the LayerNorm kernels: over [x, -x] the mean is zero and the variance is mean(x^2), so the first half of
        LayerNorm([x, -x]) with unit scale and zero shift is x / sqrt(mean(x^2) + eps); the learned scale is a broadcast
        multiplication afterwards (its gradient a column sum). Twice the row length through the normalisation, no new kernel."""
        if len(shape) != 1:
            raise ValueError("only RMSNorm over the last dimension can be exported")
        n = int(shape[0])
        eps = float(eps) if eps is not None else float(torch.finfo(x.dtype).eps)
        with torch.no_grad():
            neg = self._unary(x, -x, "scale", -1.0)
            both = self._cat([x, neg], x.dim() - 1, torch.cat([x, neg], dim=-1))
            normed = self._layer_norm(both, (2 * n,), torch.ones(2 * n), torch.zeros(2 * n), eps, F.layer_norm(both, (2 * n,), None, None, eps))
            half = normed[..., :n]
            if w is None:
                return self._unary(half, y, "scale", 1.0)
            return self._binary(half, w, y, "mul")

    def _embedding(self, ids, table, y):
        ins = [self._operand(ids), self._operand(table)]
        out, y = self._result(y)
        self._emit("embedding", ins, out)
        return y

    def _matmul(self, a, b, y):
        if a.dim() < 2 or b.dim() < 2:
            raise ValueError("matmul of vectors cannot be exported")
        if b.dim() > 2 and tuple(b.shape[:-2]) != tuple(a.shape[:-2]):
            raise ValueError("matmul with broadcast batch axes cannot be exported")
        ia = self._operand(a)
        # a right operand whose transpose is contiguous ([.., N, K] in memory) is read in place as a K-major matrix
        if not b.is_contiguous() and b.transpose(-1, -2).is_contiguous():
            ib, tb = self._operand(b.transpose(-1, -2)), 1
        else:
            ib, tb = self._operand(b), 0
        out, y = self._result(y)
        self._emit("matmul", [ia, ib], out, tb=tb, alpha="1.0")
        return y

    def _softmax(self, x, dim, y):
        if dim % x.dim() != x.dim() - 1:
            raise ValueError("softmax over an inner axis cannot be exported")
        ix = self._operand(x)
        out, y = self._result(y)
        self._emit("softmax", [ix], out, scale="1.0")
        return y

    def _token_major(self, t):
        """[B, heads, S, D] -> (IR id of a [B, S, heads, D] tensor, token stride): read in place when the heads of one token are
        adjacent (a slice of a packed projection), else through a copy."""
        tt = t.transpose(1, 2)
        B, S, H, D = tt.shape
        st = tt.stride()
        if st[3] == 1 and st[2] == D and st[1] >= H * D and (B == 1 or st[0] == S * st[1]) and tt.storage_offset() % 8 == 0 and st[1] % 8 == 0:
            return self._alias(self._root(tt), tt.storage_offset(), (B, S, H, D)), int(st[1])
        return self._operand(tt), int(H * D)

    def _sdpa(self, q, k, v, y, causal, scale):
        B, H, Sq, D = q.shape
        Sk = k.shape[2]
        if causal and Sq != Sk:
            raise ValueError("torch aligns the causal mask top-left when Sq != Sk; the fused kernel aligns it bottom-right")
        iq, qs = self._token_major(q)
        ik, ks = self._token_major(k)
        iv, vs = self._token_major(v)
        if ks != vs:
            ik, ks = self._operand(k.transpose(1, 2)), int(k.shape[1] * D)
            iv, vs = self._operand(v.transpose(1, 2)), ks
        # the operator writes [B, Sq, H, D]; the node's value becomes the [B, H, Sq, D] view of exactly that memory
        y_ir = y.transpose(1, 2).contiguous()
        rid = self._register(y_ir, "act")
        sc = scale if scale is not None else 1.0 / math.sqrt(D)
        self._emit("attention", [iq, ik, iv], self._alias(rid, 0, y_ir.shape), causal=int(bool(causal)), scale=repr(float(sc)), q_stride=qs,
                   kv_stride=ks)
        return y_ir.transpose(1, 2)

    def _dropout(self, x, y, p):
        """Only reached when the module is traced in training mode: in evaluation mode dropout hands its input through."""
        ix = self._operand(x)
        out, y = self._result(y)
        self._emit("dropout", [ix], out, p=repr(float(p)), index=self.n_dropout)
        self.n_dropout += 1
        return y

    def _reduce(self, x, dim, y, mean):
        """Sum or mean over one axis that is not the last: per leading index a column sum of a [reduced, rest] matrix into an
        fp32 buffer, then one cast (with 1 / reduced for the mean) to the bf16 result."""
        if isinstance(dim, (tuple, list)):
            if len(dim) != 1:
                raise ValueError("reductions over several axes cannot be exported")
            dim = dim[0]
        dim = dim % x.dim()
        if dim == x.dim() - 1:
            raise ValueError("reductions over the last axis cannot be exported")
        outer, red, rest = math.prod(x.shape[:dim]), x.shape[dim], math.prod(x.shape[dim + 1:])
        if outer > 64:
            raise ValueError("reductions with more than 64 leading indices cannot be exported")
        ix = self._operand(x)                                         # contiguous [outer, red, rest]
        root = int(self.tensors[ix].split("alias=")[1].split()[0]) if "alias=" in self.tensors[ix] else ix
        base = int(self.tensors[ix].split("offset=")[1].split()[0]) if "offset=" in self.tensors[ix] else 0
        acc = self._new_tensor("f32", "act", [outer * rest])
        self.copy_cache.clear()
        self.ops.append({"type": "fill", "in": [], "out": [acc], "attr": {"value": 0}})
        for b in range(outer):
            src = self._alias(root, base + b * red * rest, (red, rest))
            dst = self._new_tensor("f32", "act", [rest], f"alias={acc} offset={b * rest}")
            self.ops.append({"type": "column_sum", "in": [src], "out": [dst], "attr": {}})
        out, y = self._result(y)
        self.ops.append({"type": "cast", "in": [acc], "out": [out], "attr": {"scale": repr(1.0 / red if mean else 1.0)}})
        return y

    def _multihead_attention(self, m, a, kw):
        """nn.MultiheadAttention as packed projection -> fused attention -> output projection: self-attention (query is key is
        value: one GEMM for q, k, v) or cross-attention (key is value: one GEMM for q, one for k and v, both reading row slices
        of the packed weight in place). Batch-first inputs, no masks, no averaged attention weights (``need_weights=False``)."""
        q, k, v = a[0], (a[1] if len(a) > 1 else kw.get("key")), (a[2] if len(a) > 2 else kw.get("value"))
        if k is not v or not m.batch_first or not m._qkv_same_embed_dim or m.bias_k is not None or m.add_zero_attn:
            raise ValueError("MultiheadAttention is exported for batch-first inputs with key is value (self- or cross-attention)")
        if kw.get("need_weights", a[4] if len(a) > 4 else True) or kw.get("attn_mask") is not None or kw.get("key_padding_mask") is not None:
            raise ValueError("MultiheadAttention is exported with need_weights=False and without masks (is_causal is honoured)")
        if m.training and m.dropout > 0:
            raise ValueError("attention dropout inside MultiheadAttention cannot be exported")
        B, S, E = q.shape
        H, D = m.num_heads, E // m.num_heads
        with torch.no_grad():
            w, bias = m.in_proj_weight, m.in_proj_bias
            part = lambda t, lo, hi: None if t is None else t[lo:hi]
            if q is k:
                packed = self._linear(q, w, bias, F.linear(q, w, bias))
                qh, kh, vh = (t.transpose(1, 2) for t in packed.view(B, S, 3, H, D).unbind(2))
            else:
                Sk = k.shape[1]
                qp = self._linear(q, w[:E], part(bias, 0, E), F.linear(q, w[:E], part(bias, 0, E)))
                kv = self._linear(k, w[E:], part(bias, E, 3 * E), F.linear(k, w[E:], part(bias, E, 3 * E)))
                qh = qp.view(B, S, H, D).transpose(1, 2)
                kh, vh = (t.transpose(1, 2) for t in kv.view(B, Sk, 2, H, D).unbind(2))
            causal = bool(kw.get("is_causal", False))
            att = self._sdpa(qh, kh, vh, F.scaled_dot_product_attention(qh, kh, vh, is_causal=causal), causal, None)
            merged = att.transpose(1, 2)
            merged = self._handle("reshape", (merged, (B, S, E)), {}, merged.reshape(B, S, E))
            out = self._linear(merged, m.out_proj.weight, m.out_proj.bias, F.linear(merged, m.out_proj.weight, m.out_proj.bias))
        return out, None

    def _encoder_layer(self, m, x, causal=False):
        """nn.TransformerEncoderLayer written out with the emitter's own operators (its forward cannot be traced: fast-path
        checks on concrete tensors). Batch-first, no masks, relu / gelu feed-forward; pre- or post-norm."""
        if not m.self_attn.batch_first:
            raise ValueError("TransformerEncoderLayer is exported with batch_first=True")
        act = m.activation
        name = "relu" if act in (F.relu, torch.relu) or isinstance(act, torch.nn.ReLU) else \
            "gelu" if act is F.gelu or isinstance(act, torch.nn.GELU) else None
        if name is None:
            raise ValueError("TransformerEncoderLayer is exported with relu or gelu as its activation")
        drop = lambda d, h: self._dropout(h, F.dropout(h, d.p, True), d.p) if m.training and d.p > 0 else h
        norm = lambda n, h: self._layer_norm(h, n.normalized_shape, n.weight, n.bias, n.eps, n(h))
        add = lambda p, q: self._binary(p, q, p + q, "add")

        def attend(h):
            return drop(m.dropout1, self._multihead_attention(m.self_attn, (h, h, h), {"need_weights": False, "is_causal": causal})[0])

        def feed_forward(h):
            h1 = self._linear(h, m.linear1.weight, m.linear1.bias, F.linear(h, m.linear1.weight, m.linear1.bias))
            h2 = drop(m.dropout, self._unary(h1, F.relu(h1) if name == "relu" else F.gelu(h1), name))
            return drop(m.dropout2, self._linear(h2, m.linear2.weight, m.linear2.bias, F.linear(h2, m.linear2.weight, m.linear2.bias)))

        with torch.no_grad():
            if m.norm_first:
                x = add(x, attend(norm(m.norm1, x)))
                return add(x, feed_forward(norm(m.norm2, x)))
            x = norm(m.norm1, add(x, attend(x)))
            return norm(m.norm2, add(x, feed_forward(x)))

    def _decoder_layer(self, m, x, memory, causal):
        """nn.TransformerDecoderLayer: (causal) self-attention, cross-attention over ``memory``, feed-forward."""
        if not m.self_attn.batch_first:
            raise ValueError("TransformerDecoderLayer is exported with batch_first=True")
        act = m.activation
        name = "relu" if act in (F.relu, torch.relu) or isinstance(act, torch.nn.ReLU) else \
            "gelu" if act is F.gelu or isinstance(act, torch.nn.GELU) else None
        if name is None:
            raise ValueError("TransformerDecoderLayer is exported with relu or gelu as its activation")
        drop = lambda d, h: self._dropout(h, F.dropout(h, d.p, True), d.p) if m.training and d.p > 0 else h
        norm = lambda n, h: self._layer_norm(h, n.normalized_shape, n.weight, n.bias, n.eps, n(h))
        add = lambda p, q: self._binary(p, q, p + q, "add")
        own = lambda h: drop(m.dropout1, self._multihead_attention(m.self_attn, (h, h, h), {"need_weights": False, "is_causal": causal})[0])
        cross = lambda h: drop(m.dropout2, self._multihead_attention(m.multihead_attn, (h, memory, memory), {"need_weights": False})[0])

        def feed_forward(h):
            h1 = self._linear(h, m.linear1.weight, m.linear1.bias, F.linear(h, m.linear1.weight, m.linear1.bias))
            h2 = drop(m.dropout, self._unary(h1, F.relu(h1) if name == "relu" else F.gelu(h1), name))
            return drop(m.dropout3, self._linear(h2, m.linear2.weight, m.linear2.bias, F.linear(h2, m.linear2.weight, m.linear2.bias)))

        with torch.no_grad():
            if m.norm_first:
                x = add(x, own(norm(m.norm1, x)))
                x = add(x, cross(norm(m.norm2, x)))
                return add(x, feed_forward(norm(m.norm3, x)))
            x = norm(m.norm1, add(x, own(x)))
            x = norm(m.norm2, add(x, cross(x)))
            return norm(m.norm3, add(x, feed_forward(x)))

    def _decoder(self, m, a, kw):
        x, memory = a[0], (a[1] if len(a) > 1 else kw.get("memory"))
        causal = bool(kw.get("tgt_is_causal", False))
        tgt_mask = kw.get("tgt_mask", a[2] if len(a) > 2 else None)
        # torch wants the square mask beside the tgt_is_causal hint; the hint is what is exported (the fused kernel masks itself)
        if (tgt_mask is not None and not causal) or any(kw.get(key) is not None for key in ("memory_mask", "tgt_key_padding_mask", "memory_key_padding_mask")) \
                or (len(a) > 3 and any(t is not None for t in a[3:])):
            raise ValueError("transformer decoders are exported without explicit masks (tgt_mask together with tgt_is_causal=True is the causal mask)")
        if isinstance(m, torch.nn.TransformerDecoderLayer):
            return self._decoder_layer(m, x, memory, causal)
        for layer in m.layers:
            x = self._decoder_layer(layer, x, memory, causal)
        if m.norm is not None:
            with torch.no_grad():
                x = self._layer_norm(x, m.norm.normalized_shape, m.norm.weight, m.norm.bias, m.norm.eps, m.norm(x))
        return x

    def _encoder(self, m, a, kw):
        causal = bool(kw.get("is_causal", False))
        mask = kw.get("mask", kw.get("src_mask", a[1] if len(a) > 1 else None))
        if (mask is not None and not causal) or kw.get("src_key_padding_mask") is not None or (len(a) > 2 and a[2] is not None):
            raise ValueError("transformer encoders are exported without explicit masks (a mask together with is_causal=True is the causal mask)")
        x = a[0]
        if isinstance(m, torch.nn.TransformerEncoderLayer):
            return self._encoder_layer(m, x, causal)
        for layer in m.layers:
            x = self._encoder_layer(layer, x, causal)
        if m.norm is not None:
            with torch.no_grad():
                x = self._layer_norm(x, m.norm.normalized_shape, m.norm.weight, m.norm.bias, m.norm.eps, m.norm(x))
        return x

    def _scalar_result(self, y):
        """A fresh fp32 scalar activation (loss values): (IR id, the tensor that stands for the node)."""
        real = y.detach().to(torch.float32).reshape(1).clone()
        rid = self._new_tensor("f32", "act", [1])
        self.keep.append(real)
        self.roots[real.untyped_storage().data_ptr()] = rid
        return rid, real.reshape(())

    def _cross_entropy(self, logits, target, y, weight=None, ignore_index=-100, reduction="mean", label_smoothing=0.0):
        if logits.dim() != 2 or target.dim() != 1 or target.dtype != torch.int64:
            raise ValueError("cross_entropy is exported for [rows, classes] logits and int64 class targets [rows]")
        if weight is not None or reduction != "mean" or label_smoothing:
            raise ValueError("cross_entropy is exported with mean reduction, no class weights and no label smoothing")
        ins = [self._operand(logits), self._operand(target)]
        out, y = self._scalar_result(y)
        # the mean runs over all rows; a row whose target is ignore_index adds nothing to the loss or the gradient
        self._emit("cross_entropy", ins, out, ignore_index=int(ignore_index))
        return y

    def _mse(self, a, b, y, reduction="mean"):
        if tuple(a.shape) != tuple(b.shape) or reduction != "mean":
            raise ValueError("mse_loss is exported for equal shapes and mean reduction")
        ins = [self._operand(a), self._operand(b)]
        out, y = self._scalar_result(y)
        self._emit("mse", ins, out)
        return y

    def _cat(self, tensors, dim, y):
        y = y.contiguous()
        if y.untyped_storage().data_ptr() in self.roots:
            y = y.clone()
        rid = self._register(y, "act")
        out_strides = list(y.stride())
        off = 0
        for t in tensors:
            if t.dim() > 5:
                raise ValueError("concatenation supports at most 5 axes")
            root = self._root(t)
            self.copy_cache.clear()
            self.ops.append({"type": "copy", "in": [root], "out": [rid],
                             "attr": {"shape": ",".join(map(str, t.shape)), "in_strides": ",".join(map(str, t.stride())),
                                      "in_offset": int(t.storage_offset()), "out_strides": ",".join(map(str, out_strides)),
                                      "out_offset": int(off * out_strides[dim])}})
            off += t.shape[dim]
        return y

    # ---- interpreter hooks
    def placeholder(self, target, args, kwargs):
        real = super().placeholder(target, args, kwargs)
        if torch.is_tensor(real):
            real = real.contiguous().clone()
            self._register(real, "input")
            self.inputs.append(self._operand(real))
        return real

    def output(self, target, args, kwargs):
        res = super().output(target, args, kwargs)
        outs = res if isinstance(res, (tuple, list)) else (res,)
        for o in outs:
            if not torch.is_tensor(o):
                raise ValueError("graph outputs must be tensors")
            self.outputs.append(self._operand(o))
        return res

    def _handle(self, name, a, kw, y, module=None):
        """After a call node ran on concrete values: emit IR for it and return the value that stands for the node."""
        flat = []
        for x in list(a) + list(kw.values()):
            flat += [t for t in (x if isinstance(x, (tuple, list)) else (x,)) if torch.is_tensor(t)]
        inplace = name in _INPLACE or bool(getattr(module, "inplace", False))
        if isinstance(module, torch.nn.MultiheadAttention):
            return self._multihead_attention(module, a, kw)          # returns (output, None)
        if isinstance(module, (torch.nn.TransformerEncoderLayer, torch.nn.TransformerEncoder)):
            return self._encoder(module, a, kw)
        if isinstance(module, (torch.nn.TransformerDecoderLayer, torch.nn.TransformerDecoder)):
            return self._decoder(module, a, kw)
        if isinstance(module, torch.nn.Transformer):                 # encoder over src, decoder over tgt and the encoder's output
            if not module.batch_first:
                raise ValueError("nn.Transformer is exported with batch_first=True")
            src, tgt = a[0], (a[1] if len(a) > 1 else kw.get("tgt"))
            memory = self._encoder(module.encoder, (src,), {"mask": kw.get("src_mask"), "is_causal": kw.get("src_is_causal", False),
                                                             "src_key_padding_mask": kw.get("src_key_padding_mask")})
            return self._decoder(module.decoder, (tgt, memory), {k: kw.get(k) for k in ("tgt_mask", "memory_mask", "tgt_key_padding_mask",
                                                                                         "memory_key_padding_mask", "tgt_is_causal")})
        if not torch.is_tensor(y):
            if isinstance(y, (tuple, list)):
                for r in y:
                    if torch.is_tensor(r) and not any(r.untyped_storage().data_ptr() == t.untyped_storage().data_ptr() for t in flat):
                        raise ValueError(f"cannot export {name}: it returns several new tensors")
            return y
        if not inplace and any(y.untyped_storage().data_ptr() == t.untyped_storage().data_ptr() for t in flat):
            return y                    # a view of a traced tensor (or the tensor itself: dropout in eval mode, .to of the same dtype)
        if isinstance(module, torch.nn.Dropout) or (module is None and name == "dropout"):
            p = module.p if module is not None else (a[1] if len(a) > 1 else kw.get("p", 0.5))
            training = module.training if module is not None else (a[2] if len(a) > 2 else kw.get("training", True))
            return self._dropout(a[0], y, p) if training and p > 0 else a[0]
        if module is not None:
            m = module
            if isinstance(m, torch.nn.Linear):
                return self._linear(a[0], m.weight, m.bias, y)
            if isinstance(m, torch.nn.LayerNorm):
                return self._layer_norm(a[0], m.normalized_shape, m.weight, m.bias, m.eps, y)
            if isinstance(m, torch.nn.Embedding):
                return self._embedding(a[0], m.weight, y)
            if isinstance(m, torch.nn.RMSNorm):
                return self._rms_norm(a[0], m.normalized_shape, m.weight, m.eps, y)
            if isinstance(m, torch.nn.GELU):
                return self._unary(a[0], y, "gelu_tanh" if m.approximate == "tanh" else "gelu")
            for cls, fn in ((torch.nn.ReLU, "relu"), (torch.nn.Tanh, "tanh"), (torch.nn.Sigmoid, "sigmoid"), (torch.nn.SiLU, "silu")):
                if isinstance(m, cls):
                    return self._unary(a[0], y, fn, inplace=inplace)
            if isinstance(m, torch.nn.Softmax):
                return self._softmax(a[0], m.dim, y)
            if isinstance(m, torch.nn.CrossEntropyLoss):
                return self._cross_entropy(a[0], a[1], y, m.weight, m.ignore_index, m.reduction, m.label_smoothing)
            if isinstance(m, torch.nn.MSELoss):
                return self._mse(a[0], a[1], y, m.reduction)
            raise ValueError(f"cannot export module of type {type(m).__name__}")
        n = name
        if n in _INPLACE:
            fn = _INPLACE[n]
            return self._unary(a[0], y, fn, inplace=True) if fn in _UNARY else self._binary(a[0], a[1], y, fn, inplace=True)
        if n == "linear":
            return self._linear(a[0], a[1], a[2] if len(a) > 2 else kw.get("bias"), y)
        if n == "layer_norm":
            return self._layer_norm(a[0], a[1], a[2] if len(a) > 2 else kw.get("weight"), a[3] if len(a) > 3 else kw.get("bias"),
                                    a[4] if len(a) > 4 else kw.get("eps", 1e-5), y)
        if n == "embedding":
            return self._embedding(a[0], a[1], y)
        if n == "rms_norm":
            return self._rms_norm(a[0], a[1], a[2] if len(a) > 2 else kw.get("weight"), a[3] if len(a) > 3 else kw.get("eps"), y)
        if n == "gelu":
            return self._unary(a[0], y, "gelu_tanh" if kw.get("approximate", "none") == "tanh" else "gelu")
        if n in ("relu", "tanh", "sigmoid", "silu", "exp", "rsqrt", "square"):
            return self._unary(a[0], y, n)
        if n == "neg":
            return self._unary(a[0], y, "scale", -1.0)
        if n == "sqrt":                                          # sqrt(x) = x * rsqrt(x)
            return self._binary(a[0], self._unary(a[0], torch.rsqrt(a[0]), "rsqrt"), y, "mul")
        if n == "clamp" and (a[1] if len(a) > 1 else kw.get("min")) == 0 and (a[2] if len(a) > 2 else kw.get("max")) is None:
            return self._unary(a[0], y, "relu")
        if n == "pow" and not torch.is_tensor(a[1] if len(a) > 1 else kw.get("exponent")):
            p = a[1] if len(a) > 1 else kw.get("exponent")
            if p == 2:
                return self._unary(a[0], y, "square")
            if p == 1:
                return self._unary(a[0], y, "scale", 1.0)
            if p == -0.5:
                return self._unary(a[0], y, "rsqrt")
            if p == 3:                                           # x^3 = x^2 * x
                return self._binary(self._unary(a[0], a[0] * a[0], "square"), a[0], y, "mul")
            raise ValueError(f"cannot export pow with exponent {p} (2, 3, 1 and -0.5 are)")
        if n in ("add", "sub", "mul", "truediv", "div", "maximum", "minimum"):
            return self._binary(a[0], a[1], y, "div" if n == "truediv" else n)
        if n in ("matmul", "bmm", "mm"):
            return self._matmul(a[0], a[1], y)
        if n == "softmax":
            return self._softmax(a[0], a[1] if len(a) > 1 else kw.get("dim", -1), y)
        if n == "scaled_dot_product_attention":
            if (a[3] if len(a) > 3 else kw.get("attn_mask")) is not None:
                raise ValueError("attention with an explicit mask cannot be exported")
            if (a[4] if len(a) > 4 else kw.get("dropout_p", 0.0)):
                raise ValueError("attention dropout has no place in an inference graph")
            return self._sdpa(a[0], a[1], a[2], y, a[5] if len(a) > 5 else kw.get("is_causal", False), kw.get("scale"))
        if n in ("mean", "sum") and torch.is_tensor(y) and y.dim() > 0 and (len(a) > 1 or "dim" in kw):
            return self._reduce(a[0], a[1] if len(a) > 1 else kw["dim"], y, n == "mean")
        if n == "log_softmax":
            x, dim = a[0], (a[1] if len(a) > 1 else kw.get("dim", -1))
            if x.dim() != 2 or dim % 2 != 1:
                raise ValueError("log_softmax is exported over the class axis of [rows, classes] logits, as the input of nll_loss")
            self.keep.append(y)
            self.pending_log_softmax[y.untyped_storage().data_ptr()] = x
            return y
        if n == "nll_loss":
            logits = self.pending_log_softmax.get(a[0].untyped_storage().data_ptr())   # stays registered: any other reader is refused
            if logits is None:
                raise ValueError("nll_loss is exported on the result of log_softmax only")
            return self._cross_entropy(logits, a[1], y, a[2] if len(a) > 2 else kw.get("weight"), kw.get("ignore_index", -100),
                                       kw.get("reduction", "mean"), 0.0)
        if n == "cross_entropy":
            return self._cross_entropy(a[0], a[1], y, a[2] if len(a) > 2 else kw.get("weight"), kw.get("ignore_index", -100),
                                       kw.get("reduction", "mean"), kw.get("label_smoothing", 0.0))
        if n == "mse_loss":
            return self._mse(a[0], a[1], y, kw.get("reduction", "mean"))
        if n in ("cat", "concat"):
            return self._cat(list(a[0]), int(a[1] if len(a) > 1 else kw.get("dim", 0)) % y.dim(), y)
        if n in ("reshape", "contiguous", "clone", "flatten", "to", "float", "type_as", "dropout", "expand_as"):
            # torch copied because the source view is not contiguous: a strided copy, then the new shape as an alias
            src = a[0]
            rid = self._operand(src)
            root = int(self.tensors[rid].split("alias=")[1].split()[0]) if "alias=" in self.tensors[rid] else rid
            flat_copy = src.contiguous()
            self.keep.append(flat_copy)
            self.roots[flat_copy.untyped_storage().data_ptr()] = root
            return flat_copy.reshape(y.shape)
        if any(t.untyped_storage().data_ptr() in self.pending_log_softmax for t in flat):
            raise ValueError("log_softmax is exported only as the input of nll_loss (the pair becomes one cross_entropy operator)")
        if all(t.untyped_storage().data_ptr() not in self.roots or self._kind(self.roots[t.untyped_storage().data_ptr()]) == "param" for t in flat):
            y = y.contiguous()
            self._constant(y)           # built from constants only (position ids, tables of fixed shape, ...)
            return y
        raise ValueError(f"cannot export operator {n}")

    def call_module(self, target, args, kwargs):
        m = self.fetch_attr(target)
        return self._handle(type(m).__name__, args, kwargs, super().call_module(target, args, kwargs), module=m)

    def call_function(self, target, args, kwargs):
        return self._handle(getattr(target, "__name__", str(target)), args, kwargs, super().call_function(target, args, kwargs))

    def call_method(self, target, args, kwargs):
        return self._handle(target, args, kwargs, super().call_method(target, args, kwargs))


class _LeafTracer(torch.fx.Tracer):
    """Layers the emitter knows by type stay whole, whatever package their class lives in: the flow API's layers subclass the
    torch ones and dispatch on the tensor kind in ``forward``, which cannot be traced symbolically (and need not be)."""

    _LEAVES = (torch.nn.Linear, torch.nn.LayerNorm, torch.nn.RMSNorm, torch.nn.Embedding, torch.nn.GELU, torch.nn.ReLU, torch.nn.Tanh, torch.nn.Sigmoid,
               torch.nn.SiLU, torch.nn.Softmax, torch.nn.Dropout, torch.nn.CrossEntropyLoss, torch.nn.MSELoss, torch.nn.MultiheadAttention,
               torch.nn.TransformerEncoderLayer, torch.nn.TransformerEncoder, torch.nn.TransformerDecoderLayer, torch.nn.TransformerDecoder)

    def is_leaf_module(self, m, qualname):
        return isinstance(m, self._LEAVES) or super().is_leaf_module(m, qualname)


def _fold(ops, outputs, tensor_lines):
    """Peephole fusion: an activation, then a residual addition, that are the only consumer of a linear's result move into its
    GEMM epilogue (bias -> activation -> + residual is the order the kernel applies). The fused operator takes the consumer's
    place in the order, where all of its inputs exist."""
    def root_of(t):
        rec = tensor_lines[t]
        return root_of(int(rec.split("alias=")[1].split()[0])) if "alias=" in rec else t

    out_roots = {root_of(t) for t in outputs}
    changed = True
    while changed:
        changed = False
        readers = {}
        for i, op in enumerate(ops):
            for t in op["in"]:
                if t >= 0:
                    readers.setdefault(root_of(t), []).append(i)
        for i, op in enumerate(ops):
            if op["type"] != "linear" or op["in"][3] != -1:
                continue
            r = root_of(op["out"][0])
            if r in out_roots or len(readers.get(r, [])) != 1:
                continue
            j = readers[r][0]
            nxt = ops[j]
            mine = {root_of(t) for t in op["in"] if t >= 0}
            if any(root_of(o) in mine for k in range(i + 1, j) for o in ops[k]["out"]):
                continue            # something rewrites one of the linear's inputs in between
            if root_of(nxt["out"][0]) == r:
                continue            # an in-place consumer: leave it alone
            if nxt["type"] == "unary" and int(nxt["attr"]["fn"]) in (1, 2, 3) and op["attr"]["act"] == "none":
                op["attr"]["act"] = {1: "gelu", 2: "gelu_tanh", 3: "relu"}[int(nxt["attr"]["fn"])]
            elif nxt["type"] == "binary" and int(nxt["attr"]["fn"]) == 0 and int(nxt["attr"]["bmode"]) == 0:
                other = [t for t in nxt["in"] if root_of(t) != r]
                if len(other) != 1:
                    continue
                op["in"][3] = other[0]
            else:
                continue
            op["out"] = nxt["out"]
            ops[j] = op
            del ops[i]
            changed = True
            break
    return ops


def export_graph(module, example_inputs, directory, fuse=True, train_mode=False):
    """Records ``module(*example_inputs)`` as an operator graph with the example's shapes and writes it for the C++ runtime.
    Parameters are stored as bf16 (integer tables as int64). Returns the directory. The module is traced in evaluation mode
    unless ``train_mode`` is set; in training mode dropout layers become dropout operators (a training graph draws a new mask
    on every step; loaded for inference they hand their input through)."""
    os.makedirs(directory, exist_ok=True)
    if torch.is_tensor(example_inputs):
        example_inputs = (example_inputs,)
    was_training = module.training
    module.train(bool(train_mode))
    try:
        if isinstance(module, torch.fx.GraphModule):
            gm = module
        else:
            tracer = _LeafTracer()
            gm = torch.fx.GraphModule(module, tracer.trace(module))
        em = _GraphEmitter(gm, directory)
        with torch.no_grad():
            em.run(*[t.detach().cpu() for t in example_inputs])
    finally:
        module.train(was_training)
    ops = _fold(em.ops, em.outputs, em.tensors) if fuse else em.ops
    lines = ["oneflow_b200 graph v2"]
    lines += [f"tensor {i} {t}" for i, t in enumerate(em.tensors)]
    for op in ops:
        attrs = " ".join(f"{k}={v}" for k, v in op["attr"].items())
        lines.append(f"op {op['type']} in={','.join(map(str, op['in']))} out={','.join(map(str, op['out']))} {attrs}".rstrip())
    lines += [f"input {t}" for t in em.inputs] + [f"output {t}" for t in em.outputs]
    with open(os.path.join(directory, "graph.txt"), "w") as f:
        f.write("\n".join(lines) + "\n")
    return directory


class InferenceGraph:
    """ctypes face of the C ABI of the C++ inference API. ``device`` -1 runs the host implementation of the operators."""

    def __init__(self, directory, device=0, n_streams=2):
        lib_dir = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib")
        for dep in ("libofb_core.so", "libofb_kernels.so"):
            ctypes.CDLL(os.path.join(lib_dir, dep), mode=ctypes.RTLD_GLOBAL)
        self.lib = lib = ctypes.CDLL(os.path.join(lib_dir, "libofb_api.so"))
        lib.ofb_api_graph_load_ex.restype = ctypes.c_void_p
        lib.ofb_api_last_error.restype = ctypes.c_char_p
        for fn in ("ofb_api_graph_in_features", "ofb_api_graph_out_features", "ofb_api_graph_input_numel", "ofb_api_graph_output_numel"):
            getattr(lib, fn).restype = ctypes.c_longlong
        lib.ofb_api_graph_load_training_flags.restype = ctypes.c_void_p
        load = getattr(self, "_load", None)
        self.h = load(lib) if load else lib.ofb_api_graph_load_ex(directory.encode(), ctypes.c_int(device), ctypes.c_int(n_streams))
        if not self.h:
            raise RuntimeError(lib.ofb_api_last_error().decode())
        h = ctypes.c_void_p(self.h)
        self.in_features = lib.ofb_api_graph_in_features(h)
        self.out_features = lib.ofb_api_graph_out_features(h)
        self.num_inputs = lib.ofb_api_graph_num_inputs(h)
        self.num_outputs = lib.ofb_api_graph_num_outputs(h)

    def forward(self, x):
        """One bf16 input [rows, in_features] -> [rows, out_features] (fp32 numpy arrays on the host)."""
        x = np.ascontiguousarray(np.asarray(x, dtype=np.float32))
        rows = x.size // self.in_features
        y = np.empty((rows, self.out_features), dtype=np.float32)
        rc = self.lib.ofb_api_graph_forward(ctypes.c_void_p(self.h), x.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(rows),
                                            y.ctypes.data_as(ctypes.c_void_p))
        if rc != 0:
            raise RuntimeError(self.lib.ofb_api_last_error().decode())
        return y

    def run(self, *inputs):
        """Any number of inputs (float arrays for bf16 inputs, integer arrays for id inputs) -> list of flat fp32 outputs."""
        return self._call(self.lib.ofb_api_graph_run, inputs)

    def _call(self, entry, inputs):
        h = ctypes.c_void_p(self.h)
        if len(inputs) != self.num_inputs:
            raise ValueError(f"the graph takes {self.num_inputs} inputs")
        bufs = []
        for i, x in enumerate(inputs):
            dt = np.int64 if self.lib.ofb_api_graph_input_is_int64(h, ctypes.c_int(i)) else np.float32
            a = np.ascontiguousarray(np.asarray(x, dtype=dt))
            if a.size != self.lib.ofb_api_graph_input_numel(h, ctypes.c_int(i)):
                raise ValueError(f"input {i} has {a.size} elements, the graph was exported for "
                                 f"{self.lib.ofb_api_graph_input_numel(h, ctypes.c_int(i))}")
            bufs.append(a)
        outs = [np.empty(self.lib.ofb_api_graph_output_numel(h, ctypes.c_int(i)), dtype=np.float32) for i in range(self.num_outputs)]
        in_ptrs = (ctypes.c_void_p * len(bufs))(*[b.ctypes.data for b in bufs])
        out_ptrs = (ctypes.c_void_p * len(outs))(*[o.ctypes.data for o in outs])
        rc = entry(h, in_ptrs, ctypes.c_int(len(bufs)), out_ptrs, ctypes.c_int(len(outs)))
        if rc != 0:
            raise RuntimeError(self.lib.ofb_api_last_error().decode())
        return outs

    def stats(self):
        s = (ctypes.c_longlong * 7)()
        self.lib.ofb_api_graph_stats(ctypes.c_void_p(self.h), s)
        return dict(zip(("ops", "tensors", "activation_bytes", "arena_bytes", "dependencies", "streams_used", "graph_replays"), list(s)))

    def close(self):
        if getattr(self, "h", None):
            self.lib.ofb_api_graph_free(ctypes.c_void_p(self.h))
            self.h = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class TrainingGraph(InferenceGraph):
    """An exported graph whose first output is a scalar loss, loaded as a training step (``oneflow_api::Graph::LoadTraining``):
    reverse-mode differentiation of the operator IR, gradient buffers planned together with the activations, one fused
    optimizer operator ("adamw" or "sgd") over fp32 master weights. ``step(*inputs)`` runs forward, backward and update and
    returns the loss (computed before the update); ``parameters()`` reads the fp32 master weights back by parameter name.
    ``clip_grad_norm`` > 0 scales the gradients to that global L2 norm at most; with ``accumulation_steps`` = k every call is
    one micro-batch whose gradients (of loss / k) are accumulated, and the optimizer runs on every k-th call.
    ``recompute_cheap_activations`` drops the outputs of element-wise operators and LayerNorms after the forward pass and
    recomputes them in the backward pass (less activation memory, a few more memory-bound kernels);
    ``recompute_all_but_residual_stream`` keeps only the residual stream and runs every other forward operator again in the
    backward pass (full activation checkpointing: about a third more compute for the smallest activation footprint).
    ``decay_matrices_only`` keeps weight decay off biases and LayerNorm parameters (a second update operator).
    With ``external_gradient_reduction`` a ``step`` runs forward and backward only; ``gradients()`` / ``set_gradients()`` give
    access to the accumulated fp32 gradients, ``all_reduce_gradients()`` averages them over a torch.distributed group (data
    parallelism), ``apply_update()`` runs clipping and the optimizer."""

    def __init__(self, directory, device=0, n_streams=2, optimizer="adamw", lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0,
                 momentum=0.0, clip_grad_norm=0.0, accumulation_steps=1, recompute_cheap_activations=False, seed=0,
                 recompute_all_but_residual_stream=False, external_gradient_reduction=False, decay_matrices_only=False):
        self._load = lambda lib: lib.ofb_api_graph_load_training_flags(
            directory.encode(), ctypes.c_int(device), ctypes.c_int(n_streams), optimizer.encode(), ctypes.c_float(lr),
            ctypes.c_float(betas[0]), ctypes.c_float(betas[1]), ctypes.c_float(eps), ctypes.c_float(weight_decay), ctypes.c_float(momentum),
            ctypes.c_float(clip_grad_norm), ctypes.c_int(accumulation_steps), ctypes.c_int((1 if recompute_cheap_activations else 0) | (2 if recompute_all_but_residual_stream else 0) |
                         (4 if external_gradient_reduction else 0) | (8 if decay_matrices_only else 0)))
        super().__init__(directory, device, n_streams)
        lib = self.lib
        lib.ofb_api_graph_parameter_name.restype = ctypes.c_char_p
        lib.ofb_api_graph_parameter_numel.restype = ctypes.c_longlong
        lib.ofb_api_graph_steps.restype = ctypes.c_longlong
        lib.ofb_api_graph_dump.restype = ctypes.c_longlong
        if seed:
            self.set_seed(seed)

    def step(self, *inputs):
        outs = self.run(*inputs)
        return float(outs[0][0])

    def evaluate(self, *inputs):
        """The loss (first output) of the current weights on ``inputs``: forward operators only, dropout off, nothing updated."""
        return float(self._call(self.lib.ofb_api_graph_evaluate, inputs)[0][0])

    @property
    def steps(self):
        return int(self.lib.ofb_api_graph_steps(ctypes.c_void_p(self.h)))

    def set_lr_schedule(self, kind="cosine", warmup_steps=0, decay_steps=0, min_lr_ratio=0.0):
        """Linear warm-up over ``warmup_steps`` optimizer steps, then "constant", or "cosine" / "linear" decay to
        ``min_lr_ratio`` times the base rate at ``decay_steps``; evaluated by the runtime before every optimizer step."""
        if self.lib.ofb_api_graph_set_lr_schedule(ctypes.c_void_p(self.h), kind.encode(), ctypes.c_longlong(warmup_steps),
                                                  ctypes.c_longlong(decay_steps), ctypes.c_float(min_lr_ratio)) != 0:
            raise RuntimeError(self.lib.ofb_api_last_error().decode())

    @property
    def lr(self):
        """The rate the next optimizer step will use."""
        self.lib.ofb_api_graph_lr.restype = ctypes.c_float
        return float(self.lib.ofb_api_graph_lr(ctypes.c_void_p(self.h)))

    def set_seed(self, seed):
        """Seed of the dropout operators: the mask is a function of (seed, number of the call, operator, element)."""
        self.lib.ofb_api_graph_set_seed(ctypes.c_void_p(self.h), ctypes.c_ulonglong(seed))

    def set_lr(self, lr):
        self.lib.ofb_api_graph_set_lr(ctypes.c_void_p(self.h), ctypes.c_float(lr))

    def save(self, directory):
        """Writes a directory that loads again (for inference, or with ``restore`` for training that continues bit for bit)."""
        os.makedirs(directory, exist_ok=True)
        if self.lib.ofb_api_graph_save(ctypes.c_void_p(self.h), directory.encode()) != 0:
            raise RuntimeError(self.lib.ofb_api_last_error().decode())
        return directory

    def restore(self, directory):
        """Step count, fp32 master weights and optimizer state from ``directory/train_state.bin`` (written by ``save``)."""
        if self.lib.ofb_api_graph_restore(ctypes.c_void_p(self.h), directory.encode()) != 0:
            raise RuntimeError(self.lib.ofb_api_last_error().decode())

    def _parameter_names(self):
        h = ctypes.c_void_p(self.h)
        return [self.lib.ofb_api_graph_parameter_name(h, ctypes.c_int(i)).decode() for i in range(self.lib.ofb_api_graph_num_parameters(h))]

    def gradients(self):
        """The accumulated fp32 gradients by parameter name (graphs loaded with ``external_gradient_reduction``)."""
        h = ctypes.c_void_p(self.h)
        out = {}
        for i, name in enumerate(self._parameter_names()):
            buf = np.empty(self.lib.ofb_api_graph_parameter_numel(h, ctypes.c_int(i)), dtype=np.float32)
            if self.lib.ofb_api_graph_gradient_read(h, ctypes.c_int(i), buf.ctypes.data_as(ctypes.c_void_p)) != 0:
                raise RuntimeError(self.lib.ofb_api_last_error().decode())
            out[name] = buf
        return out

    def set_gradients(self, grads):
        h = ctypes.c_void_p(self.h)
        for i, name in enumerate(self._parameter_names()):
            if name not in grads:
                continue
            a = np.ascontiguousarray(np.asarray(grads[name], dtype=np.float32).reshape(-1))
            if self.lib.ofb_api_graph_gradient_write(h, ctypes.c_int(i), a.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(a.size)) != 0:
                raise RuntimeError(self.lib.ofb_api_last_error().decode())

    def all_reduce_gradients(self, group=None):
        """Averages the gradients over the ranks of a torch.distributed group: one flat buffer, one collective."""
        import torch.distributed as dist
        grads = self.gradients()
        names = list(grads)
        flat = torch.from_numpy(np.concatenate([grads[n] for n in names]))
        dist.all_reduce(flat, group=group)
        flat /= dist.get_world_size(group)
        out, at = {}, 0
        for n in names:
            out[n] = flat[at:at + grads[n].size].numpy()
            at += grads[n].size
        self.set_gradients(out)

    def apply_update(self):
        if self.lib.ofb_api_graph_apply_update(ctypes.c_void_p(self.h)) != 0:
            raise RuntimeError(self.lib.ofb_api_last_error().decode())

    def parameters(self):
        h = ctypes.c_void_p(self.h)
        out = {}
        for i in range(self.lib.ofb_api_graph_num_parameters(h)):
            name = self.lib.ofb_api_graph_parameter_name(h, ctypes.c_int(i)).decode()
            buf = np.empty(self.lib.ofb_api_graph_parameter_numel(h, ctypes.c_int(i)), dtype=np.float32)
            if self.lib.ofb_api_graph_parameter_read(h, ctypes.c_int(i), buf.ctypes.data_as(ctypes.c_void_p)) != 0:
                raise RuntimeError(self.lib.ofb_api_last_error().decode())
            out[name] = buf
        return out

    def copy_parameters_to(self, module):
        """Writes the trained fp32 master weights back into ``module``'s parameters (matched by name), so that the module
        can go on in Python: evaluation, another export, a state_dict checkpoint."""
        trained = self.parameters()
        with torch.no_grad():
            for name, prm in module.named_parameters():
                if name in trained:
                    prm.copy_(torch.from_numpy(trained[name]).view_as(prm).to(prm.dtype))
        return module

    def dump(self):
        """The operator list after the backward pass was appended, in the IR text format."""
        h = ctypes.c_void_p(self.h)
        n = self.lib.ofb_api_graph_dump(h, None, ctypes.c_longlong(0))
        buf = ctypes.create_string_buffer(n + 1)
        self.lib.ofb_api_graph_dump(h, buf, ctypes.c_longlong(n + 1))
        return buf.value.decode()


def compile_training(module, example_inputs, directory=None, device=0, **options):
    """Export ``module`` (its forward returns the loss) in training mode and load it as a ``TrainingGraph``: the one call that
    takes a PyTorch / flow module to a natively compiled training step. ``options`` are ``TrainingGraph``'s."""
    import tempfile
    directory = directory or tempfile.mkdtemp(prefix="oneflow_graph_")
    export_graph(module, example_inputs, directory, fuse=False, train_mode=True)
    return TrainingGraph(directory, device=device, **options)
