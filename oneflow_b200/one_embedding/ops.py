"""OneEmbedding as separate ops, with the reference's signatures (oneflow/core/functional/functional_api.yaml,
``one_embedding_*``; kernels: oneflow/user/kernels/{data_shuffle_kernel,one_embedding_kernels,
one_embedding_update_kernels}.cu).  ``Embedding.forward`` / ``backward`` run these stages fused (on CUDA in the device
engine); this module exposes the stages one by one for code that builds its own pipeline:

``id_shuffle`` -> ``lookup`` -> ``embedding_shuffle`` ... ``embedding_gradient_shuffle`` -> ``*_update`` -> ``embedding_put``

A key is ``id * num_tables + table_id``; its owner rank is a hash of the key.  ``num_unique_matrix[i * world + j]`` is
how many unique keys rank i sends to rank j.  Outputs have their exact sizes (no padding to a static shape).
"""
from __future__ import annotations

import weakref

import torch
import torch.distributed as dist

from .embedding import _all_to_all_v, _row_update, owner_of

_REGISTRY = weakref.WeakValueDictionary()


def register(embedding):
    _REGISTRY[embedding.name] = embedding


def embedding_by_name(name):
    emb = _REGISTRY.get(name)
    if emb is None:
        raise KeyError(f"no OneEmbedding named {name!r} is alive in this process")
    return emb


def _world():
    return (dist.get_world_size(), dist.get_rank()) if dist.is_initialized() else (1, 0)


def one_embedding_id_shuffle(ids, table_ids=None, num_tables=1, embedding_name=None):
    """-> (num_unique_matrix, inverse_unique_partition_indices, cur_rank_num_unique, cur_rank_unique_ids,
    cur_rank_unique_table_ids, cur_rank_inverse_indices)"""
    world, me = _world()
    flat = ids.reshape(-1).long()
    if table_ids is None:
        tids = (torch.arange(flat.numel(), device=flat.device) % num_tables) if num_tables > 1 else torch.zeros_like(flat)
    else:
        tids = table_ids.reshape(-1).long()
    keys = flat * num_tables + tids
    uniq, inverse = torch.unique(keys, return_inverse=True)
    owner = owner_of(uniq, world)
    order = torch.argsort(owner, stable=True)
    unperm = torch.empty_like(order)
    unperm[order] = torch.arange(order.numel(), device=order.device)
    send_counts = torch.bincount(owner, minlength=world)
    if world > 1:
        recv_keys, _ = _all_to_all_v(uniq[order], send_counts.tolist())
        rows = [torch.empty_like(send_counts) for _ in range(world)]
        dist.all_gather(rows, send_counts)
        matrix = torch.stack(rows).reshape(-1)
    else:
        recv_keys, matrix = uniq[order], send_counts.reshape(-1)
    cur_uniq, cur_inverse = torch.unique(recv_keys, return_inverse=True)
    n = torch.tensor([cur_uniq.numel()], dtype=torch.int32, device=flat.device)
    return (matrix.to(torch.int32), unperm[inverse].to(torch.int32), n, (cur_uniq // num_tables).to(ids.dtype),
            (cur_uniq % num_tables).to(torch.int32), cur_inverse.to(torch.int32))


def _counts(matrix):
    world, me = _world()
    m = matrix.reshape(world, world).long()
    return m[me, :].tolist(), m[:, me].tolist()      # (what I sent in the id shuffle, what I received)


def one_embedding_embedding_shuffle(cur_rank_embeddings, num_unique_matrix, cur_rank_inverse_indices,
                                    inverse_unique_partition_indices, embedding_name=None):
    """Rows of this rank's unique keys -> one row per original id position."""
    sent, received = _counts(num_unique_matrix)
    rows = cur_rank_embeddings[cur_rank_inverse_indices.long()]
    if _world()[0] > 1:
        rows, _ = _all_to_all_v(rows, received)
    return rows[inverse_unique_partition_indices.long()]


def one_embedding_embedding_gradient_shuffle(embedding_grad, num_unique_matrix, cur_rank_inverse_indices,
                                             inverse_unique_partition_indices, embedding_name=None):
    """One gradient row per id position -> summed gradient per unique key owned by this rank (fp32)."""
    sent, received = _counts(num_unique_matrix)
    D = embedding_grad.shape[-1]
    g = embedding_grad.reshape(-1, D)
    part = torch.zeros((sum(sent), D), dtype=torch.float32, device=g.device)
    part.index_add_(0, inverse_unique_partition_indices.long(), g.float())
    if _world()[0] > 1:
        part, _ = _all_to_all_v(part, sent)
    n_cur = int(cur_rank_inverse_indices.max().item()) + 1 if cur_rank_inverse_indices.numel() else 0
    out = torch.zeros((n_cur, D), dtype=torch.float32, device=g.device)
    return out.index_add_(0, cur_rank_inverse_indices.long(), part.float())


def one_embedding_lookup(num_unique_ids, unique_ids, table_ids, dtype=None, embedding_dtype=None, line_size=None,
                         embedding_size=None, embedding_name=None, embedding_tables=None, state_initializer=None, seed=0):
    """Full lines ``[embedding | optimizer state]`` of the keys, inserting and initialising the new ones."""
    emb = embedding_by_name(embedding_name)
    n = int(num_unique_ids.reshape(-1)[0])
    nt = max(len(emb.tables), 1)
    keys = unique_ids.reshape(-1)[:n].long() * nt + table_ids.reshape(-1)[:n].long()
    store = emb._ensure_store(unique_ids.device)
    emb._op_slots = store.lookup(keys, keys % nt)
    return store.rows(emb._op_slots)


def one_embedding_embedding_put(num_unique_ids, unique_ids, unique_embeddings, embedding_name=None, line_size=None):
    """Write updated lines back for the keys of the preceding :func:`one_embedding_lookup`."""
    emb = embedding_by_name(embedding_name)
    n = int(num_unique_ids.reshape(-1)[0])
    nt = max(len(emb.tables), 1)
    store = emb._ensure_store(unique_ids.device)
    slots = getattr(emb, "_op_slots", None)
    if slots is None or slots.numel() != n:
        keys = unique_ids.reshape(-1)[:n].long() * nt
        slots = store.lookup(keys, keys % nt)
    store.put(slots, unique_embeddings[:n].float())


def _update(kind, num_unique_ids, unique_embeddings, embedding_grad, learning_rate, down_scale_by_tensor, skip_if, lr_val,
            scale, embedding_size, hyper, step=1):
    n = int(num_unique_ids.reshape(-1)[0])
    rows = unique_embeddings.float().clone()
    if skip_if is not None and int(skip_if.reshape(-1)[0]) != 0:
        return rows
    s = float(scale)
    if down_scale_by_tensor is not None:
        s /= float(down_scale_by_tensor.reshape(-1)[0])
    hyper = dict(hyper, lr=float(learning_rate.reshape(-1)[0]) if learning_rate is not None else float(lr_val), scale=s)
    live = rows[:n]
    _row_update(kind, live, embedding_grad[:n].float(), int(embedding_size), hyper, step)
    return rows


def one_embedding_sgd_update(num_unique_ids, unique_embeddings, embedding_grad, learning_rate=None, down_scale_by_tensor=None,
                             skip_if=None, learning_rate_val=0.0, scale=1.0, weight_decay=0.0, momentum=0.0, line_size=None,
                             embedding_size=None, embedding_name=None):
    kind = "momentum" if momentum != 0 else "sgd"
    return _update(kind, num_unique_ids, unique_embeddings, embedding_grad, learning_rate, down_scale_by_tensor, skip_if,
                   learning_rate_val, scale, embedding_size, {"weight_decay": weight_decay, "momentum": momentum})


def one_embedding_adam_update(num_unique_ids, unique_embeddings, embedding_grad, learning_rate=None, down_scale_by_tensor=None,
                              skip_if=None, bias_correction1=None, bias_correction2=None, learning_rate_val=0.0, scale=1.0,
                              weight_decay=0.0, beta1=0.9, beta2=0.999, bias_correction1_val=1.0, bias_correction2_val=1.0,
                              epsilon=1e-8, do_bias_correction=True, line_size=None, embedding_size=None, embedding_name=None):
    """The bias corrections ``1 - beta^t`` are inputs (tensor or value); they are turned back into the step count the
    row update expects."""
    import math
    bc1 = float(bias_correction1.reshape(-1)[0]) if bias_correction1 is not None else bias_correction1_val
    step = max(int(round(math.log(max(1.0 - bc1, 1e-300)) / math.log(beta1))), 1) if do_bias_correction and 0 < bc1 < 1 else 1
    return _update("adam", num_unique_ids, unique_embeddings, embedding_grad, learning_rate, down_scale_by_tensor, skip_if,
                   learning_rate_val, scale, embedding_size,
                   {"weight_decay": weight_decay, "beta1": beta1, "beta2": beta2, "eps": epsilon,
                    "do_bias_correction": do_bias_correction}, step)


def one_embedding_adagrad_update(num_unique_ids, unique_embeddings, embedding_grad, learning_rate=None, down_scale_by_tensor=None,
                                 skip_if=None, train_step=None, train_step_val=0, learning_rate_val=0.0, scale=1.0,
                                 weight_decay=0.0, lr_decay=0.0, epsilon=1e-10, line_size=None, embedding_size=None,
                                 embedding_name=None):
    step = int(train_step.reshape(-1)[0]) if train_step is not None else int(train_step_val)
    return _update("adagrad", num_unique_ids, unique_embeddings, embedding_grad, learning_rate, down_scale_by_tensor, skip_if,
                   learning_rate_val, scale, embedding_size, {"weight_decay": weight_decay, "lr_decay": lr_decay, "eps": epsilon},
                   step + 1)


def one_embedding_ftrl_update(num_unique_ids, unique_embeddings, embedding_grad, learning_rate=None, down_scale_by_tensor=None,
                              skip_if=None, learning_rate_val=0.0, scale=1.0, weight_decay=0.0, lr_power=-0.5, lambda1=0.0,
                              lambda2=0.0, beta=0.0, line_size=None, embedding_size=None, embedding_name=None):
    return _update("ftrl", num_unique_ids, unique_embeddings, embedding_grad, learning_rate, down_scale_by_tensor, skip_if,
                   learning_rate_val, scale, embedding_size,
                   {"weight_decay": weight_decay, "lr_power": lr_power, "lambda1": lambda1, "lambda2": lambda2, "beta": beta})


def one_embedding_fused_lookup(shadow, ids, table_ids=None, dtype=None, embedding_name=None, line_size=None, embedding_size=None,
                               is_full_cache=False, num_tables=1, embedding_tables=None, padding_idx=None, seed=0):
    """id shuffle + lookup + embedding shuffle of the named embedding in one call (its ``forward``)."""
    return embedding_by_name(embedding_name)(ids, table_ids)


def one_embedding_unique_key_value_pair(keys, values=None, num_tables=1, embedding_name=None):
    """-> (num_unique, unique_keys, unique_values, inverse_indices); without ``values`` the table id is the column
    index modulo ``num_tables``."""
    flat_k = keys.reshape(-1).long()
    flat_v = (values.reshape(-1).long() if values is not None
              else torch.arange(flat_k.numel(), device=keys.device) % num_tables)
    uniq, inverse = torch.unique(flat_k * num_tables + flat_v, return_inverse=True)
    n = torch.tensor([uniq.numel()], dtype=torch.int32, device=keys.device)
    return n, (uniq // num_tables).to(keys.dtype), (uniq % num_tables).to(torch.int32), inverse.to(torch.int32)


class OneEmbeddingHandler:
    """Snapshot handle of one embedding's key-value store, by embedding name
    (reference: oneflow/api/python/framework/one_embedding.cpp, ``OneEmbeddingHandler``)."""

    def __init__(self, key_value_store_options=None, local_rank_id=0, rank_id=0, world_size=1, embedding_name=None):
        self.options, self.rank_id, self.world_size = key_value_store_options, rank_id, world_size
        self.embedding_name = embedding_name

    def _emb(self):
        return embedding_by_name(self.embedding_name)

    def SaveSnapshot(self, snapshot_name):
        self._emb().save_snapshot(snapshot_name)

    def LoadSnapshot(self, snapshot_name):
        self._emb().load_snapshot(snapshot_name)
