"""``ArgsTree``: walk and rebuild nested tuples / lists / dicts of graph inputs and outputs
(reference: python/oneflow/framework/args_tree.py:33-300).  With ``gen_name`` every node gets a stable name
``<prefix>.<index or key>`` and a running index, which ``nn.Graph`` uses to label its inputs and outputs."""
from __future__ import annotations

from collections import OrderedDict

import torch


def _raw(value, t):
    return type(value) is t


def _container(value):
    return type(value) in (list, tuple, dict, OrderedDict)


class NamedArg:
    """One node of a named tree: a leaf value or a container whose children are NamedArgs."""

    def __init__(self, prefix="", name=None, global_index=0, tensor_type=torch.Tensor):
        self._name = name if name is not None else str(global_index)
        self._prefix, self._global_index, self._tensor_type = prefix, global_index, tensor_type
        self._value, self._is_value_set = None, False

    def prefix(self):
        return self._prefix

    def name(self):
        return self._name

    def global_index(self):
        return self._global_index

    def value(self):
        if not self._is_value_set:
            raise RuntimeError("NamedArg has no value yet")
        return self._value

    def is_leaf(self):
        return not _container(self._value)

    def set_value(self, value):
        if self._is_value_set:
            raise RuntimeError("NamedArg value is already set")
        self._value, self._is_value_set = value, True

    def __repr__(self):
        v = self._value
        shown = f"tensor{tuple(v.shape)}" if isinstance(v, self._tensor_type) else (
            type(v).__name__ if _container(v) else repr(v))
        return f"{self._prefix}_{self._name} (index {self._global_index}): {shown}"


class ArgsTree:
    def __init__(self, io_args, gen_name=False, root_prefix="", root_name=None, tensor_type=torch.Tensor):
        self._io_args, self._gen_name = io_args, gen_name
        self._tensor_type, self._next_index = tensor_type, 0
        self._named_io_args = self._name_tree(io_args, root_prefix, root_name) if gen_name else None

    def gen_name(self):
        return self._gen_name

    def _name_tree(self, value, prefix, name):
        arg = NamedArg(prefix, name, self._next_index, self._tensor_type)
        self._next_index += 1
        if _raw(value, list) or _raw(value, tuple):
            arg.set_value(type(value)(self._name_tree(v, prefix + ("." if prefix else "") + str(i), None)
                                      for i, v in enumerate(value)))
        elif _raw(value, dict) or _raw(value, OrderedDict):
            arg.set_value(type(value)((k, self._name_tree(v, prefix + ("." if prefix else "") + str(k), str(k) + "_" + str(i)))
                                      for i, (k, v) in enumerate(value.items())))
        else:
            arg.set_value(value)
        return arg

    def iter_nodes(self):
        """Depth-first, parents before children; NamedArgs when names were generated, the raw values otherwise."""
        stack = [iter([self._named_io_args if self._gen_name else self._io_args])]
        while stack:
            try:
                cur = next(stack[-1])
            except StopIteration:
                stack.pop()
                continue
            val = cur.value() if type(cur) is NamedArg else cur
            if _raw(val, list) or _raw(val, tuple):
                stack.append(iter(val))
            elif _raw(val, dict) or _raw(val, OrderedDict):
                stack.append(iter(val.values()))
            yield cur

    def iter_named_nodes(self):
        if not self._gen_name:
            raise RuntimeError("iter_named_nodes needs gen_name=True")
        for node in self.iter_nodes():
            yield node.prefix() + "_" + node.name(), node

    def map_leaf(self, fn):
        """A copy of the tree with ``fn`` applied to every leaf (to the NamedArg when names were generated)."""
        return self._map(self._named_io_args if self._gen_name else self._io_args, fn, leaves_only=True)

    def map_tuple_leaf(self, fn):
        """Like :meth:`map_leaf` for trees made of tuples / lists only, the common shape of graph inputs."""
        return self.map_leaf(fn)

    def _map(self, value, fn, leaves_only):
        inner = value.value() if type(value) is NamedArg else value
        if _raw(inner, list) or _raw(inner, tuple):
            return type(inner)(self._map(v, fn, leaves_only) for v in inner)
        if _raw(inner, dict) or _raw(inner, OrderedDict):
            return type(inner)((k, self._map(v, fn, leaves_only)) for k, v in inner.items())
        return fn(value)

    def __repr__(self):
        if self._named_io_args is not None:
            return "\n".join(repr(n) for n in self.iter_nodes())
        return repr(self._io_args)
