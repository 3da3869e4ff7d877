"""Training through the native graph compiler: an exported forward graph that ends in a loss is differentiated in C++
(csrc/api/graph_autodiff.cpp), compiled into one plan with its backward and optimizer operators, and run by the same
executor as inference graphs. The host runtime is compared with PyTorch autograd; the GPU runtime with the host runtime."""
import os

import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from oneflow_b200.utils import export as E

from test_inference_api import Block, _bf16_weights


class Mlp(nn.Module):
    def __init__(self, d_in=32, d_h=64, classes=16):
        super().__init__()
        self.fc1, self.ln, self.fc2 = nn.Linear(d_in, d_h), nn.LayerNorm(d_h), nn.Linear(d_h, classes)

    def forward(self, x, y):
        return F.cross_entropy(self.fc2(self.ln(F.gelu(self.fc1(x)))), y)


class TiedLM(nn.Module):
    """Embedding + position table + one pre-LN transformer layer; the output projection shares the embedding table."""

    def __init__(self, **kw):
        super().__init__()
        self.block = Block(**kw)
        self.block.head.weight = self.block.emb.weight

    def forward(self, ids, targets):
        logits = self.block(ids)
        return F.cross_entropy(logits.view(-1, logits.shape[-1]), targets.view(-1))


def _grads_by_unit_sgd(module, inputs, directory, device=-1):
    """One SGD step with lr 1 and no momentum: parameter before - parameter after = the gradient the graph computed."""
    d = E.export_graph(module, inputs, directory, fuse=False)
    g = E.TrainingGraph(d, device=device, optimizer="sgd", lr=1.0)
    before = g.parameters()
    loss = g.step(*[t.numpy() for t in inputs])
    after = g.parameters()
    g.close()
    return loss, {k: before[k] - after[k] for k in before}


def _check_grads(module, grads, rel=3e-2):
    for name, p in module.named_parameters():
        ref = p.grad.detach().numpy().reshape(-1)
        scale = np.abs(ref).max() + 1e-6
        assert np.abs(grads[name] - ref).max() <= rel * scale, name


def test_mlp_gradients_and_sgd_trajectory_match_autograd(tmp_path):
    torch.manual_seed(0)
    m = _bf16_weights(Mlp())
    x, y = torch.randn(24, 32).bfloat16().float(), torch.randint(0, 16, (24,))
    loss, grads = _grads_by_unit_sgd(m, (x, y), str(tmp_path / "unit"))
    ref = m(x, y)
    ref.backward()
    assert abs(loss - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    _check_grads(m, grads)
    # several steps against torch.optim.SGD with momentum
    m.zero_grad()
    d = E.export_graph(m, (x, y), str(tmp_path / "run"), fuse=False)
    g = E.TrainingGraph(d, device=-1, optimizer="sgd", lr=0.1, momentum=0.9)
    opt = torch.optim.SGD(m.parameters(), lr=0.1, momentum=0.9)
    for _ in range(8):
        ref = m(x, y)
        opt.zero_grad()
        ref.backward()
        opt.step()
        assert abs(g.step(x.numpy(), y.numpy()) - float(ref.detach())) < 3e-2 * max(abs(float(ref.detach())), 0.1)
    assert g.steps == 8
    ps = g.parameters()
    for name, p in m.named_parameters():
        assert np.abs(ps[name] - p.detach().numpy().reshape(-1)).max() < 2e-2, name
    g.close()


def test_tied_transformer_block_gradients_match_autograd(tmp_path):
    """Attention backward through the packed projection, two embedding tables (one broadcast over the batch), residual
    streams with several consumers, and a table that is both looked up and used as the output projection."""
    torch.manual_seed(1)
    m = _bf16_weights(TiedLM(d=64, heads=1, vocab=96, seq=16))
    ids, tgt = torch.randint(0, 96, (2, 16)), torch.randint(0, 96, (2, 16))
    loss, grads = _grads_by_unit_sgd(m, (ids, tgt), str(tmp_path))
    ref = m(ids, tgt)
    ref.backward()
    assert abs(loss - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    assert "block.emb.weight" in grads and "block.head.weight" not in grads      # one parameter, two uses
    _check_grads(m, grads, rel=5e-2)


def test_adamw_loss_falls_like_torch(tmp_path):
    torch.manual_seed(2)
    m = _bf16_weights(TiedLM(d=64, heads=1, vocab=96, seq=16))
    ids, tgt = torch.randint(0, 96, (2, 16)), torch.randint(0, 96, (2, 16))
    d = E.export_graph(m, (ids, tgt), str(tmp_path), fuse=False)
    g = E.TrainingGraph(d, device=-1, optimizer="adamw", lr=1e-2, weight_decay=0.01)
    text = g.dump()
    assert text.count("op attention_bwd") == 1 and text.count("op adamw_update") == 1 and text.count("op embedding_bwd") == 2
    assert "dq_stride=192" in text            # the three gradients go straight into the packed projection's gradient
    st = g.stats()
    assert st["arena_bytes"] < st["activation_bytes"]          # forward activations, gradients and temporaries share memory
    opt = torch.optim.AdamW(m.parameters(), lr=1e-2, weight_decay=0.01)
    ours, theirs = [], []
    for _ in range(6):
        ref = m(ids, tgt)
        opt.zero_grad()
        ref.backward()
        opt.step()
        theirs.append(float(ref.detach()))
        ours.append(g.step(ids.numpy(), tgt.numpy()))
    assert ours[-1] < 0.05 * ours[0]
    for a, b in zip(ours[:4], theirs[:4]):
        assert abs(a - b) < 0.05 * max(abs(b), 1.0)
    g.set_lr(0.0)
    before = g.parameters()
    g.step(ids.numpy(), tgt.numpy())
    after = g.parameters()
    assert all(np.array_equal(before[k], after[k] * 1.0) or np.abs(before[k] - after[k]).max() < 1e-12 for k in before)
    g.close()


def test_mse_and_parameter_free_paths(tmp_path):
    class Reg(nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = nn.Linear(16, 32), nn.Linear(32, 8)

        def forward(self, x, t):
            return F.mse_loss(self.b(torch.tanh(self.a(x))) * 0.5, t)

    torch.manual_seed(3)
    m = _bf16_weights(Reg())
    x, t = torch.randn(8, 16).bfloat16().float(), torch.randn(8, 8).bfloat16().float()
    loss, grads = _grads_by_unit_sgd(m, (x, t), str(tmp_path))
    ref = m(x, t)
    ref.backward()
    assert abs(loss - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    _check_grads(m, grads)


def test_what_cannot_be_differentiated_is_refused_with_the_operator_named(tmp_path):
    class InPlace(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc = nn.Linear(16, 16)

        def forward(self, x, y):
            h = self.fc(x)
            h.relu_()
            return F.cross_entropy(h, y)

    m = _bf16_weights(InPlace())
    x, y = torch.randn(4, 16), torch.randint(0, 16, (4,))
    d = E.export_graph(m, (x, y), str(tmp_path / "inplace"), fuse=False)
    with pytest.raises(RuntimeError, match="in place"):
        E.TrainingGraph(d, device=-1)
    m2 = _bf16_weights(Mlp())
    x2, y2 = torch.randn(24, 32), torch.randint(0, 16, (24,))
    d2 = E.export_graph(m2, (x2, y2), str(tmp_path / "fused"), fuse=True)       # gelu folded into fc1's epilogue
    with pytest.raises(RuntimeError, match="fuse=False"):
        E.TrainingGraph(d2, device=-1)
    d3 = E.export_graph(_bf16_weights(nn.Sequential(nn.Linear(8, 8))), (torch.randn(2, 8),), str(tmp_path / "noloss"))
    with pytest.raises(RuntimeError, match="scalar fp32 loss"):
        E.TrainingGraph(d3, device=-1)
    # the same directories still load as inference graphs (the loss is just an output)
    out = E.InferenceGraph(d2, device=-1).run(x2.numpy(), y2.numpy())[0]
    assert abs(out[0] - float(m2(x2.bfloat16().float(), y2).detach())) < 5e-2


@pytest.mark.gpu
def test_training_step_on_the_gpu_runtime_matches_the_host_runtime(tmp_path):
    """The same plan on the sm_100a kernels: tcgen05 GEMMs for data and weight gradients (fp32 accumulation into the
    gradient buffers), fused attention backward writing into the packed projection gradient, LayerNorm backward, fused
    cross entropy, the multi-tensor AdamW; compared step by step with the host implementation of the same operators."""
    torch.manual_seed(4)
    m = _bf16_weights(TiedLM(d=128, heads=2, vocab=256, seq=128))
    ids, tgt = torch.randint(0, 256, (2, 128)), torch.randint(0, 256, (2, 128))
    d = E.export_graph(m, (ids, tgt), str(tmp_path), fuse=False)
    loss_h, grads_h = _grads_by_unit_sgd(m, (ids, tgt), str(tmp_path / "h"), device=-1)
    loss_d, grads_d = _grads_by_unit_sgd(m, (ids, tgt), str(tmp_path / "d"), device=0)
    assert abs(loss_h - loss_d) < 1e-2 * abs(loss_h)
    for k in grads_h:
        assert np.abs(grads_h[k] - grads_d[k]).max() <= 5e-2 * (np.abs(grads_h[k]).max() + 1e-6), k
    host = E.TrainingGraph(d, device=-1, optimizer="adamw", lr=3e-3)
    dev = E.TrainingGraph(d, device=0, optimizer="adamw", lr=3e-3)
    assert dev.stats()["streams_used"] == 2
    lh = [host.step(ids.numpy(), tgt.numpy()) for _ in range(5)]
    ld = [dev.step(ids.numpy(), tgt.numpy()) for _ in range(5)]
    assert ld[-1] < ld[0]
    assert dev.stats()["graph_replays"] == 4      # the whole step (forward, backward, update) is one CUDA-graph launch from the second on
    for a, b in zip(lh, ld):
        assert abs(a - b) < 5e-2 * max(abs(a), 1.0)
    host.close()
    dev.close()


def test_rewriting_passes_fuse_the_activation_into_both_gemms_and_keep_the_numbers(tmp_path, monkeypatch):
    """linear -> gelu becomes one GEMM that also stores the pre-activation; the next layer's data-gradient GEMM multiplies by
    gelu' of it in its epilogue, so neither the activation nor its derivative is a pass of its own. The unfused plan
    (passes switched off) is the reference."""
    torch.manual_seed(5)
    m = _bf16_weights(TiedLM(d=64, heads=1, vocab=96, seq=16))
    ids, tgt = torch.randint(0, 96, (2, 16)), torch.randint(0, 96, (2, 16))
    d = E.export_graph(m, (ids, tgt), str(tmp_path), fuse=False)
    fused = E.TrainingGraph(d, device=-1, optimizer="sgd", lr=0.5)
    text = fused.dump()
    assert "# pass fuse_activation_backward fired=1" in text and "# pass fuse_activation_forward fired=1" in text
    assert "act=gelu" in text and "act_grad=gelu" in text and "op unary" not in text
    monkeypatch.setenv("ONEFLOW_API_PASSES", "0")
    plain = E.TrainingGraph(d, device=-1, optimizer="sgd", lr=0.5)
    monkeypatch.delenv("ONEFLOW_API_PASSES")
    assert "op unary_bwd" in plain.dump() and "act_grad" not in plain.dump()
    assert fused.stats()["ops"] < plain.stats()["ops"]
    before = fused.parameters()
    a, b = fused.step(ids.numpy(), tgt.numpy()), plain.step(ids.numpy(), tgt.numpy())
    assert abs(a - b) < 1e-3 * max(abs(b), 1.0)                    # the forward pass computes the same numbers
    pf, pp = fused.parameters(), plain.parameters()
    for k in pf:                                                    # one step: the parameter deltas are lr * gradient
        gf, gp = before[k] - pf[k], before[k] - pp[k]
        assert np.abs(gf - gp).max() <= 3e-2 * (np.abs(gp).max() + 1e-6), k
    for _ in range(2):
        a, b = fused.step(ids.numpy(), tgt.numpy()), plain.step(ids.numpy(), tgt.numpy())
        assert abs(a - b) < 5e-2 * max(abs(b), 1.0)
    fused.close()
    plain.close()


def test_inference_graph_exported_unfused_is_fused_at_load_time(tmp_path):
    torch.manual_seed(6)
    m = _bf16_weights(nn.Sequential(nn.Linear(32, 64), nn.GELU(), nn.Linear(64, 16), nn.ReLU()))
    x = torch.randn(8, 32).bfloat16().float()
    d = E.export_graph(m, (x,), str(tmp_path), fuse=False)
    g = E.InferenceGraph(d, device=-1)
    assert g.stats()["ops"] == 2                      # two GEMMs, activations in their epilogues
    out = g.run(x.numpy())[0]
    assert np.abs(out - m(x).detach().numpy().reshape(-1)).max() < 3e-2
    g.close()


def test_save_and_restore_continue_training_bit_for_bit(tmp_path):
    torch.manual_seed(7)
    m = _bf16_weights(Mlp())
    x, y = torch.randn(24, 32).bfloat16().float(), torch.randint(0, 16, (24,))
    d = E.export_graph(m, (x, y), str(tmp_path / "export"), fuse=False)
    g = E.TrainingGraph(d, device=-1, optimizer="adamw", lr=1e-2, weight_decay=0.1)
    for _ in range(3):
        g.step(x.numpy(), y.numpy())
    saved = g.save(str(tmp_path / "ckpt"))
    after = [g.step(x.numpy(), y.numpy()) for _ in range(3)]
    final = g.parameters()
    g.close()
    # the saved directory is a graph of its own: as inference it computes the loss of the saved weights
    assert abs(E.InferenceGraph(saved, device=-1).run(x.numpy(), y.numpy())[0][0] - after[0]) < 1e-6
    r = E.TrainingGraph(saved, device=-1, optimizer="adamw", lr=1e-2, weight_decay=0.1)
    r.restore(saved)
    assert r.steps == 3
    assert [r.step(x.numpy(), y.numpy()) for _ in range(3)] == after
    again = r.parameters()
    assert all(np.array_equal(final[k], again[k]) for k in final)
    r.close()
    # without restore the moments start from zero and the master weights from the rounded bf16 files: another trajectory
    cold = E.TrainingGraph(saved, device=-1, optimizer="adamw", lr=1e-2, weight_decay=0.1)
    assert [cold.step(x.numpy(), y.numpy()) for _ in range(3)] != after
    # a state file of another optimizer is refused, and the graph stays usable
    sgd = E.TrainingGraph(saved, device=-1, optimizer="sgd", lr=1e-2)
    with pytest.raises(RuntimeError, match="another optimizer"):
        sgd.restore(saved)
    (tmp_path / "ckpt" / "train_state.bin").write_bytes((tmp_path / "ckpt" / "train_state.bin").read_bytes()[:-100])
    with pytest.raises(RuntimeError, match="truncated"):
        cold.restore(saved)
    cold.step(x.numpy(), y.numpy())
    cold.close()
    sgd.close()


def test_cpp_program_trains_through_the_api_and_saves_a_loadable_directory(tmp_path):
    """csrc/api/examples/train_graph.cpp compiled against oneflow_api.h: LoadTraining, Forward as a training step, Save."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no C++ compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    api = os.path.join(root, "oneflow_b200", "csrc", "api")
    lib = os.path.join(root, "oneflow_b200", "lib")
    exe = str(tmp_path / "train_graph")
    r = subprocess.run(["g++", "-std=c++17", "-O1", os.path.join(api, "examples", "train_graph.cpp"), "-I", api, "-L", lib, "-lofb_api",
                        "-lofb_kernels", "-lofb_core", f"-Wl,-rpath,{lib}", "-o", exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    torch.manual_seed(8)
    m = _bf16_weights(Mlp())
    x, y = torch.randn(24, 32).bfloat16().float(), torch.randint(0, 16, (24,))
    d = E.export_graph(m, (x, y), str(tmp_path / "g"), fuse=False)
    x.numpy().astype(np.float32).tofile(str(tmp_path / "x.bin"))
    y.numpy().astype(np.int64).tofile(str(tmp_path / "y.bin"))
    os.makedirs(str(tmp_path / "out"))
    r = subprocess.run([exe, d, "-1", "12", "0.01", str(tmp_path / "out"), str(tmp_path / "x.bin"), str(tmp_path / "y.bin")],
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    losses = [float(v) for v in r.stdout.split()]
    assert len(losses) == 12 and losses[-1] < 0.5 * losses[0]
    assert "6 trainable parameters, first: fc1.weight" in r.stderr and "steps 12" in r.stderr
    # the same steps through the Python binding give the same losses, and the saved directory evaluates to the next loss
    g = E.TrainingGraph(d, device=-1, optimizer="adamw", lr=0.01)
    ours = [g.step(x.numpy(), y.numpy()) for _ in range(13)]
    assert np.allclose(ours[:12], losses, rtol=1e-5, atol=1e-6)
    saved_loss = E.InferenceGraph(str(tmp_path / "out"), device=-1).run(x.numpy(), y.numpy())[0][0]
    assert abs(saved_loss - ours[12]) < 2e-2 * max(ours[12], 0.05)           # weights were stored as bf16
    g.close()


def test_gradient_clipping_matches_clip_grad_norm(tmp_path):
    torch.manual_seed(9)
    m = _bf16_weights(Mlp())
    x, y = torch.randn(24, 32).bfloat16().float() * 3, torch.randint(0, 16, (24,))
    d = E.export_graph(m, (x, y), str(tmp_path), fuse=False)
    g = E.TrainingGraph(d, device=-1, optimizer="sgd", lr=1.0, clip_grad_norm=0.25)
    assert "op grad_clip" in g.dump() and "clip=1" in g.dump()
    before = g.parameters()
    g.step(x.numpy(), y.numpy())
    after = g.parameters()
    m(x, y).backward()
    total = torch.nn.utils.clip_grad_norm_(m.parameters(), 0.25)
    assert float(total) > 0.25                                     # the clip is active
    ours = np.sqrt(sum(float(((before[k] - after[k]) ** 2).sum()) for k in before))
    assert abs(ours - 0.25) < 0.01                                 # the applied gradient has the clipped norm
    for name, p in m.named_parameters():
        ref = p.grad.numpy().reshape(-1)
        assert np.abs((before[name] - after[name]) - ref).max() <= 3e-2 * (np.abs(ref).max() + 1e-6), name
    g.close()


def test_gradient_accumulation_over_two_micro_batches_equals_one_large_batch(tmp_path):
    torch.manual_seed(10)
    m = _bf16_weights(Mlp())
    x, y = torch.randn(24, 32).bfloat16().float(), torch.randint(0, 16, (24,))
    d_full = E.export_graph(m, (x, y), str(tmp_path / "full"), fuse=False)
    d_half = E.export_graph(m, (x[:12], y[:12]), str(tmp_path / "half"), fuse=False)
    full = E.TrainingGraph(d_full, device=-1, optimizer="adamw", lr=1e-2)
    acc = E.TrainingGraph(d_half, device=-1, optimizer="adamw", lr=1e-2, accumulation_steps=2)
    text = acc.dump()
    assert "when=first" in text and "when=last" in text and "grad_scale=0.5" in text
    start = acc.parameters()
    for step in range(3):
        lf = full.step(x.numpy(), y.numpy())
        l0 = acc.step(x[:12].numpy(), y[:12].numpy())
        if step == 0:
            mid = acc.parameters()
            assert all(np.array_equal(start[k], mid[k]) for k in start)      # no update after the first micro-batch
            with pytest.raises(RuntimeError, match="save between steps"):
                acc.save(str(tmp_path / "never"))
        l1 = acc.step(x[12:].numpy(), y[12:].numpy())
        assert abs(0.5 * (l0 + l1) - lf) < 2e-2 * max(abs(lf), 0.1)
    assert acc.steps == 3 and full.steps == 3
    pf, pa = full.parameters(), acc.parameters()
    for k in pf:
        assert np.abs(pf[k] - pa[k]).max() < 1e-2, k
    full.close()
    acc.close()


@pytest.mark.gpu
def test_clipping_and_accumulation_on_the_gpu_runtime_match_the_host_runtime(tmp_path):
    """Every kind of call (first / last micro-batch of a step) is recorded as a CUDA graph of its own; the clip factor and the
    step scalars are read on the device, so the recordings stay valid from one step to the next."""
    torch.manual_seed(11)
    m = _bf16_weights(TiedLM(d=128, heads=2, vocab=256, seq=128))
    ids, tgt = torch.randint(0, 256, (4, 128)), torch.randint(0, 256, (4, 128))
    d = E.export_graph(m, (ids[:2], tgt[:2]), str(tmp_path), fuse=False)
    kw = dict(optimizer="adamw", lr=3e-3, clip_grad_norm=1.0, accumulation_steps=2)
    host, dev = E.TrainingGraph(d, device=-1, **kw), E.TrainingGraph(d, device=0, **kw)
    for _ in range(3):
        for lo in (0, 2):
            a = host.step(ids[lo:lo + 2].numpy(), tgt[lo:lo + 2].numpy())
            b = dev.step(ids[lo:lo + 2].numpy(), tgt[lo:lo + 2].numpy())
            assert abs(a - b) < 5e-2 * max(abs(a), 1.0)
    assert dev.steps == 3 and dev.stats()["graph_replays"] == 4          # calls 3..6: both kinds replay from their second run on
    ph, pd = host.parameters(), dev.parameters()
    for k in ph:
        assert np.abs(ph[k] - pd[k]).max() < 2e-2, k
    host.close()
    dev.close()


def test_recomputing_cheap_activations_saves_memory_and_keeps_the_trajectory(tmp_path):
    """The outputs of GELU and of the LayerNorms are dropped after their last forward reader and computed again in the
    backward pass from inputs that are kept anyway (the pre-activation, the LayerNorm input and its statistics)."""
    from oneflow_b200.utils.bench_graph_runtime import GPT
    torch.manual_seed(12)
    m = _bf16_weights(GPT(3, 64, 1, 96, 32))
    ids, tgt = torch.randint(0, 96, (4, 32)), torch.randint(0, 96, (4, 32))
    d = E.export_graph(m, (ids, tgt), str(tmp_path), fuse=False)
    plain = E.TrainingGraph(d, device=-1, optimizer="sgd", lr=2e-2)
    lean = E.TrainingGraph(d, device=-1, optimizer="sgd", lr=2e-2, recompute_cheap_activations=True)
    text = lean.dump()
    fired = int(text.split("# pass recompute_cheap_activations fired=")[1].split()[0])
    assert fired == 3 * 3 + 1            # per layer: two LayerNorms and the GELU; the final LayerNorm
    assert "act=gelu" in text            # the forward GELU still sits in its GEMM's epilogue
    assert lean.stats()["arena_bytes"] < 0.9 * plain.stats()["arena_bytes"]
    # the forward pass is the same plan; in the backward pass the recomputed GELU starts from the stored (bf16) pre-activation
    # where the fused epilogue started from the fp32 accumulator: the last bit of some activations differs
    assert lean.step(ids.numpy(), tgt.numpy()) == plain.step(ids.numpy(), tgt.numpy())
    for _ in range(3):
        a, b = lean.step(ids.numpy(), tgt.numpy()), plain.step(ids.numpy(), tgt.numpy())
        assert abs(a - b) < 2e-2 * max(abs(b), 1.0)
    pl, pp = lean.parameters(), plain.parameters()
    for k in pl:
        assert np.abs(pl[k] - pp[k]).max() < 2e-2 * (np.abs(pp[k]).max() + 1e-3), k
    plain.close()
    lean.close()


def _dropout_keep(seed, call, op_index, n, p):
    """The runtime's counter-based mask (csrc/common/dropout_hash.h) restated with numpy's wrapping 64-bit arithmetic."""
    u = np.uint64

    def mix(z):
        z = z + u(0x9E3779B97F4A7C15)
        z = (z ^ (z >> u(30))) * u(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> u(27))) * u(0x94D049BB133111EB)
        return z ^ (z >> u(31))

    with np.errstate(over="ignore"):
        base = mix(u(seed) ^ mix(u(call) * u(0xD1B54A32D192ED03) + u(op_index)))
        idx = np.arange(n, dtype=np.uint64)
        draw = mix(base + (idx >> u(2)) * u(0x9E3779B97F4A7C15))
        lane = (draw >> (u(16) * (idx & u(3)))) & u(0xFFFF)
    return lane >= u(int(p * 65536.0))


def test_dropout_draws_a_new_mask_every_call_and_backward_uses_the_same_one(tmp_path):
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1, self.drop, self.fc2 = nn.Linear(32, 64), nn.Dropout(0.25), nn.Linear(64, 16)

        def forward(self, x, y):
            return F.cross_entropy(self.fc2(F.gelu(self.drop(self.fc1(x)))), y)

    torch.manual_seed(13)
    m = _bf16_weights(Net())
    x, y = torch.randn(24, 32).bfloat16().float(), torch.randint(0, 16, (24,))
    d = E.export_graph(m, (x, y), str(tmp_path), fuse=False, train_mode=True)
    assert "op dropout" in open(os.path.join(d, "graph.txt")).read()
    assert m.training                                                   # the caller's mode is put back
    keep1 = _dropout_keep(77, 1, 0, 24 * 64, 0.25)
    assert 0.65 < keep1.mean() < 0.85 and not np.array_equal(keep1, _dropout_keep(77, 2, 0, 24 * 64, 0.25))
    g = E.TrainingGraph(d, device=-1, optimizer="sgd", lr=1.0, seed=77)
    assert g.dump().count("op dropout") == 2                             # forward, and the same operator on the gradient
    before = g.parameters()
    loss1 = g.step(x.numpy(), y.numpy())
    after = g.parameters()
    # the same computation in PyTorch with the mask of call 1 written out
    mask = torch.from_numpy(keep1.reshape(24, 64).astype(np.float32)) / 0.75
    ref = F.cross_entropy(m.fc2(F.gelu(m.fc1(x) * mask)), y)
    ref.backward()
    assert abs(loss1 - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    for name, p in m.named_parameters():
        r = p.grad.numpy().reshape(-1)
        assert np.abs((before[name] - after[name]) - r).max() <= 3e-2 * (np.abs(r).max() + 1e-6), name
    # the second call draws another mask: with lr 0 the weights stay, the loss changes
    g.set_lr(0.0)
    a, b = g.step(x.numpy(), y.numpy()), g.step(x.numpy(), y.numpy())
    assert a != b
    # loaded for inference the dropout operators hand their input through
    m.eval()
    saved = g.save(str(tmp_path / "saved"))
    out = E.InferenceGraph(saved, device=-1).run(x.numpy(), y.numpy())[0][0]
    with torch.no_grad():
        for name, p in m.named_parameters():
            p.copy_(torch.from_numpy(g.parameters()[name]).view_as(p))
        assert abs(out - float(m(x, y))) < 3e-2 * max(float(m(x, y)), 0.1)
    g.close()


@pytest.mark.gpu
def test_dropout_on_the_gpu_runtime_drops_the_same_elements_as_the_host_runtime(tmp_path):
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1, self.drop, self.fc2 = nn.Linear(128, 256), nn.Dropout(0.5), nn.Linear(256, 64)

        def forward(self, x, y):
            return F.cross_entropy(self.fc2(self.drop(F.gelu(self.fc1(x)))), y)

    torch.manual_seed(14)
    m = _bf16_weights(Net())
    x, y = torch.randn(256, 128).bfloat16().float(), torch.randint(0, 64, (256,))
    d = E.export_graph(m, (x, y), str(tmp_path), fuse=False, train_mode=True)
    host = E.TrainingGraph(d, device=-1, optimizer="sgd", lr=0.05, seed=5)
    dev = E.TrainingGraph(d, device=0, optimizer="sgd", lr=0.05, seed=5)
    other = E.TrainingGraph(d, device=0, optimizer="sgd", lr=0.05, seed=6)
    lh = [host.step(x.numpy(), y.numpy()) for _ in range(4)]
    ld = [dev.step(x.numpy(), y.numpy()) for _ in range(4)]
    lo = [other.step(x.numpy(), y.numpy()) for _ in range(4)]
    assert dev.stats()["graph_replays"] == 3                  # replays read the call number on the device: new masks each time
    for a, b in zip(lh, ld):
        assert abs(a - b) < 1e-2 * max(abs(a), 1.0)
    assert max(abs(a - b) for a, b in zip(ld, lo)) > 1e-3     # another seed, other masks
    for g in (host, dev, other):
        g.close()


def test_graph_compiler_runs_clean_under_address_ub_and_thread_sanitizers(tmp_path):
    """Parser, autodiff, the rewriting passes (default list, cheap recompute, full checkpointing), plan compiler, host
    operators and Save: the C++ training example built from the API's sources with -fsanitize=address,undefined trains a
    two-layer GPT with dropout on the host device."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no C++ compiler")
    from oneflow_b200 import build as B
    from oneflow_b200.utils.bench_graph_runtime import GPT
    exe = B.build_api_sanitized()
    torch.manual_seed(15)
    m = _bf16_weights(GPT(2, 64, 1, 96, 16))
    ids, tgt = torch.randint(0, 96, (2, 16)), torch.randint(0, 96, (2, 16))
    d = E.export_graph(m, (ids, tgt), str(tmp_path / "g"), fuse=False, train_mode=True)
    ids.numpy().astype(np.int64).tofile(str(tmp_path / "ids.bin"))
    tgt.numpy().astype(np.int64).tofile(str(tmp_path / "tgt.bin"))
    os.makedirs(str(tmp_path / "out"))
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=0 exitcode=67")
    runs = [(exe, mode) for mode in ([], ["--recompute=cheap"], ["--recompute=full"])]
    # and once under ThreadSanitizer with the scheduler's sources compiled in: two plan streams = two worker threads
    runs.append((B.build_api_thread_sanitized(), []))
    env["TSAN_OPTIONS"] = "halt_on_error=0 exitcode=66"
    for program, mode in runs:
        r = subprocess.run([program] + mode + [d, "-1", "4", "0.01", str(tmp_path / "out"), str(tmp_path / "ids.bin"), str(tmp_path / "tgt.bin")],
                           capture_output=True, text=True, timeout=600, env=env)
        out = r.stdout + r.stderr
        assert r.returncode == 0, out[-3000:]
        assert "AddressSanitizer" not in out and "ThreadSanitizer" not in out and "runtime error" not in out, out[-3000:]
        losses = [float(v) for v in r.stdout.split()]
        assert len(losses) == 4 and losses[-1] < losses[0]
        assert os.path.exists(str(tmp_path / "out" / "train_state.bin"))


def test_damaged_graph_files_are_refused_not_crashed_on(tmp_path):
    """Random damage to graph.txt (dropped or doubled records, dropped tokens, changed digits, negative and absurd numbers):
    the sanitized C++ program either trains or reports an error; it never reads or writes out of bounds."""
    import random
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no C++ compiler")
    from oneflow_b200 import build as B
    from oneflow_b200.utils.bench_graph_runtime import GPT
    exe = B.build_api_sanitized()
    torch.manual_seed(16)
    m = _bf16_weights(GPT(1, 64, 1, 96, 16))
    ids, tgt = torch.randint(0, 96, (2, 16)), torch.randint(0, 96, (2, 16))
    src = E.export_graph(m, (ids, tgt), str(tmp_path / "g"), fuse=False, train_mode=True)
    ids.numpy().astype(np.int64).tofile(str(tmp_path / "ids.bin"))
    tgt.numpy().astype(np.int64).tofile(str(tmp_path / "tgt.bin"))
    lines = open(os.path.join(src, "graph.txt")).read().splitlines()
    outcomes = {}
    for seed in range(80):
        rnd = random.Random(seed)
        damaged = list(lines)
        for _ in range(rnd.randint(1, 3)):
            i = rnd.randrange(1, len(damaged))
            toks = damaged[i].split()
            kind = rnd.randrange(6)
            if kind == 0 and len(toks) > 2:
                del toks[rnd.randrange(1, len(toks))]
            elif kind == 1:
                j = rnd.randrange(len(toks))
                toks[j] = "".join(c if not c.isdigit() else str(rnd.randrange(10)) for c in toks[j])
            elif kind == 2:
                j = rnd.randrange(len(toks))
                toks[j] = toks[j].replace("=", "=-", 1) if "=" in toks[j] else "-" + toks[j]
            elif kind == 3:
                del damaged[i]
                continue
            elif kind == 4:
                damaged.insert(i, damaged[rnd.randrange(1, len(damaged))])
                continue
            else:
                j = rnd.randrange(len(toks))
                toks[j] = toks[j] + "9999999999"
            damaged[i] = " ".join(toks)
        d = tmp_path / f"damaged{seed}"
        d.mkdir()
        for f in os.listdir(src):
            if f != "graph.txt":
                os.symlink(os.path.join(src, f), str(d / f))
        (d / "graph.txt").write_text("\n".join(damaged) + "\n")
        r = subprocess.run([exe, str(d), "-1", "1", "0.01", "-", str(tmp_path / "ids.bin"), str(tmp_path / "tgt.bin")], capture_output=True,
                           text=True, timeout=120, env=dict(os.environ, ASAN_OPTIONS="detect_leaks=0 exitcode=67"))
        assert r.returncode in (0, 1, 2) and "Sanitizer" not in r.stderr and "runtime error" not in r.stderr, (seed, r.stderr[-1500:])
        if r.returncode != 0:
            assert "error:" in r.stderr or "short read" in r.stderr or "takes" in r.stderr, (seed, r.stderr[-500:])
        outcomes[r.returncode] = outcomes.get(r.returncode, 0) + 1
    assert outcomes.get(1, 0) > 40           # most damage is detected and named


def test_layers_of_the_flow_api_export_and_train_natively(tmp_path):
    """flow.nn layers subclass the torch ones and dispatch on the tensor kind in forward; the exporter keeps them whole."""
    import oneflow as flow

    class Net(flow.nn.Module):
        def __init__(self):
            super().__init__()
            self.body = flow.nn.Sequential(flow.nn.Linear(32, 64), flow.nn.GELU(), flow.nn.LayerNorm(64), flow.nn.Linear(64, 16))

        def forward(self, x, y):
            return F.cross_entropy(self.body(x), y)

    torch.manual_seed(17)
    m = _bf16_weights(Net())
    x, y = torch.randn(24, 32).bfloat16().float(), torch.randint(0, 16, (24,))
    loss, grads = _grads_by_unit_sgd(m, (x, y), str(tmp_path))
    ref = m(x, y)
    ref.backward()
    assert abs(loss - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    assert set(grads) == {n for n, _ in m.named_parameters()}
    _check_grads(m, grads)


def test_learning_rate_schedule_follows_warmup_and_cosine(tmp_path):
    import math
    torch.manual_seed(18)
    m = _bf16_weights(Mlp())
    x, y = torch.randn(24, 32).bfloat16().float(), torch.randint(0, 16, (24,))
    d = E.export_graph(m, (x, y), str(tmp_path), fuse=False)
    g = E.TrainingGraph(d, device=-1, optimizer="sgd", lr=0.2)
    g.set_lr_schedule("cosine", warmup_steps=2, decay_steps=6, min_lr_ratio=0.1)
    want = []
    for t in range(1, 9):
        if t <= 2:
            want.append(0.2 * t / 2)
        else:
            xx = min(1.0, (t - 2) / 4)
            want.append(0.2 * (0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * xx))))
    got = []
    opt = torch.optim.SGD(m.parameters(), lr=0.2)
    for t in range(8):
        got.append(g.lr)
        for group in opt.param_groups:
            group["lr"] = want[t]
        ref = m(x, y)
        opt.zero_grad()
        ref.backward()
        opt.step()
        assert abs(g.step(x.numpy(), y.numpy()) - float(ref.detach())) < 3e-2 * max(abs(float(ref.detach())), 0.1)
    assert np.allclose(got, want, rtol=1e-5)
    ps = g.parameters()
    for name, p in m.named_parameters():
        assert np.abs(ps[name] - p.detach().numpy().reshape(-1)).max() < 2e-2, name
    with pytest.raises(RuntimeError, match="lr schedule"):
        g.set_lr_schedule("exponential")
    g.close()


def test_evaluation_calls_run_the_forward_pass_only(tmp_path):
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1, self.drop, self.fc2 = nn.Linear(32, 64), nn.Dropout(0.5), nn.Linear(64, 16)

        def forward(self, x, y):
            return F.cross_entropy(self.fc2(self.drop(F.gelu(self.fc1(x)))), y)

    torch.manual_seed(19)
    m = _bf16_weights(Net())
    x, y = torch.randn(24, 32).bfloat16().float(), torch.randint(0, 16, (24,))
    d = E.export_graph(m, (x, y), str(tmp_path), fuse=False, train_mode=True)
    g = E.TrainingGraph(d, device=-1, optimizer="adamw", lr=1e-2, accumulation_steps=2, recompute_cheap_activations=True, seed=3)
    m.eval()
    before = g.parameters()
    e0 = g.evaluate(x.numpy(), y.numpy())
    want = float(m(x, y).detach())
    assert abs(e0 - want) < 2e-2 * want                                  # dropout is off: the deterministic loss
    assert g.evaluate(x.numpy(), y.numpy()) == e0 and g.steps == 0
    assert all(np.array_equal(before[k], v) for k, v in g.parameters().items())
    # evaluation between the two micro-batches of a step disturbs neither the accumulated gradients nor the mask sequence
    ref = E.TrainingGraph(d, device=-1, optimizer="adamw", lr=1e-2, accumulation_steps=2, recompute_cheap_activations=True, seed=3)
    for _ in range(2):
        a0 = g.step(x.numpy(), y.numpy())
        g.evaluate(x.numpy(), y.numpy())
        a1 = g.step(x.numpy(), y.numpy())
        assert (a0, a1) == (ref.step(x.numpy(), y.numpy()), ref.step(x.numpy(), y.numpy()))
    pg, pr = g.parameters(), ref.parameters()
    assert all(np.array_equal(pg[k], pr[k]) for k in pg)
    assert g.evaluate(x.numpy(), y.numpy()) < e0
    g.close()
    ref.close()


def test_full_activation_checkpointing_keeps_only_the_residual_stream(tmp_path):
    """Every forward operator off the residual stream, GEMMs and attention included, runs again in the backward pass; the
    copies pull in their producers, each operator is copied once, and the losses stay those of the plain plan."""
    from oneflow_b200.utils.bench_graph_runtime import GPT
    torch.manual_seed(20)
    m = _bf16_weights(GPT(4, 64, 1, 96, 64))
    ids, tgt = torch.randint(0, 96, (8, 64)), torch.randint(0, 96, (8, 64))
    d = E.export_graph(m, (ids, tgt), str(tmp_path), fuse=False, train_mode=True)
    kw = dict(device=-1, optimizer="sgd", lr=2e-2, seed=9)
    plain = E.TrainingGraph(d, **kw)
    cheap = E.TrainingGraph(d, recompute_cheap_activations=True, **kw)
    full = E.TrainingGraph(d, recompute_all_but_residual_stream=True, **kw)
    assert full.stats()["arena_bytes"] < 0.6 * cheap.stats()["arena_bytes"] < 0.6 * plain.stats()["arena_bytes"]
    text = full.dump()
    count = lambda t: sum(1 for line in text.splitlines() if line.startswith("op " + t + " "))
    assert count("attention") == 2 * 4 and count("attention_bwd") == 4           # each attention once more, not more
    assert count("embedding") == 2                                                  # the first residual value is a checkpoint
    for _ in range(3):
        a, b = full.step(ids.numpy(), tgt.numpy()), plain.step(ids.numpy(), tgt.numpy())
        assert abs(a - b) < 1e-2 * max(abs(b), 1.0)
    pf, pp = full.parameters(), plain.parameters()
    for k in pf:
        assert np.abs(pf[k] - pp[k]).max() < 2e-2 * (np.abs(pp[k]).max() + 1e-3), k
    for g in (plain, cheap, full):
        g.close()


def test_bert_style_classifier_trains_natively(tmp_path):
    """A second model family through the native compiler: three embedding tables, post-LN encoder layers with the attention
    written out (matmul, scale, additive padding mask broadcast over heads and queries, softmax, matmul), tanh pooler over the
    first token, classification loss. Exercises scalar-minus-tensor, the general broadcast, permuted views and a row slice."""
    import math

    class Layer(nn.Module):
        def __init__(self, d, h):
            super().__init__()
            self.q, self.k, self.v, self.o = nn.Linear(d, d), nn.Linear(d, d), nn.Linear(d, d), nn.Linear(d, d)
            self.ln1, self.ln2, self.fc1, self.fc2, self.h = nn.LayerNorm(d), nn.LayerNorm(d), nn.Linear(d, 4 * d), nn.Linear(4 * d, d), h

        def forward(self, x, bias):
            B, S, D = x.shape
            heads = lambda t: t.view(B, S, self.h, D // self.h).transpose(1, 2)
            q, k, v = heads(self.q(x)), heads(self.k(x)), heads(self.v(x))
            scores = torch.matmul(q, k.transpose(-1, -2)) / math.sqrt(D // self.h) + bias
            a = torch.matmul(torch.softmax(scores, -1), v).transpose(1, 2).reshape(B, S, D)
            x = self.ln1(x + self.o(a))
            return self.ln2(x + self.fc2(F.gelu(self.fc1(x))))

    class Bert(nn.Module):
        def __init__(self, layers=2, d=64, h=2, vocab=96, seq=16, classes=4):
            super().__init__()
            self.tok, self.pos, self.typ, self.ln = nn.Embedding(vocab, d), nn.Embedding(seq, d), nn.Embedding(2, d), nn.LayerNorm(d)
            self.layers = nn.ModuleList([Layer(d, h) for _ in range(layers)])
            self.pool, self.cls = nn.Linear(d, d), nn.Linear(d, classes)

        def forward(self, ids, types, mask, labels):
            x = self.ln(self.tok(ids) + self.pos(torch.arange(ids.shape[1])) + self.typ(types))
            bias = (1.0 - mask[:, None, None, :]) * -1e4
            for layer in self.layers:
                x = layer(x, bias)
            return F.cross_entropy(self.cls(torch.tanh(self.pool(x[:, 0]))), labels)

    torch.manual_seed(21)
    m = _bf16_weights(Bert())
    ids, types, labels = torch.randint(0, 96, (4, 16)), torch.randint(0, 2, (4, 16)), torch.randint(0, 4, (4,))
    mask = (torch.rand(4, 16) > 0.2).float()
    mask[:, 0] = 1
    loss, grads = _grads_by_unit_sgd(m, (ids, types, mask, labels), str(tmp_path))
    ref = m(ids, types, mask, labels)
    ref.backward()
    assert abs(loss - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    scale = max(float(p.grad.abs().max()) for p in m.parameters())
    for name, p in m.named_parameters():
        r = p.grad.numpy().reshape(-1)
        # key biases shift every score of a row alike: their true gradient is zero, what is left is rounding
        tol = 3e-2 * (np.abs(r).max() + 1e-6) if ".k.bias" not in name else 1e-3 * scale
        assert np.abs(grads[name] - r).max() <= tol, name
    g = E.TrainingGraph(str(tmp_path), device=-1, optimizer="adamw", lr=3e-3)
    losses = [g.step(ids.numpy(), types.numpy(), mask.numpy(), labels.numpy()) for _ in range(8)]
    assert losses[-1] < 0.5 * losses[0]
    g.close()


def test_the_compiled_step_is_deterministic_and_can_be_dumped(tmp_path, monkeypatch):
    """Two loads of one directory give the same operator list, the same plan statistics and, on the host runtime, the same
    bits; ONEFLOW_API_DUMP_IR writes the list the plan compiler sees."""
    torch.manual_seed(22)
    m = _bf16_weights(TiedLM(d=64, heads=1, vocab=96, seq=16))
    ids, tgt = torch.randint(0, 96, (2, 16)), torch.randint(0, 96, (2, 16))
    d = E.export_graph(m, (ids, tgt), str(tmp_path / "g"), fuse=False, train_mode=True)
    monkeypatch.setenv("ONEFLOW_API_DUMP_IR", str(tmp_path / "ir.txt"))
    a = E.TrainingGraph(d, device=-1, optimizer="adamw", lr=1e-2, clip_grad_norm=1.0, recompute_cheap_activations=True, seed=4)
    monkeypatch.delenv("ONEFLOW_API_DUMP_IR")
    b = E.TrainingGraph(d, device=-1, optimizer="adamw", lr=1e-2, clip_grad_norm=1.0, recompute_cheap_activations=True, seed=4, n_streams=1)
    assert a.dump() == b.dump() == open(str(tmp_path / "ir.txt")).read()
    sa, sb = a.stats(), b.stats()
    assert sa["ops"] == sb["ops"] and sa["activation_bytes"] == sb["activation_bytes"] and (sa["streams_used"], sb["streams_used"]) == (2, 1)
    # one stream or two, the numbers are the same: the dependency edges order everything that shares data or memory
    assert [a.step(ids.numpy(), tgt.numpy()) for _ in range(4)] == [b.step(ids.numpy(), tgt.numpy()) for _ in range(4)]
    pa, pb = a.parameters(), b.parameters()
    assert all(np.array_equal(pa[k], pb[k]) for k in pa)
    a.close()
    b.close()


def test_vit_style_classifier_trains_natively(tmp_path):
    """A third model family: patch projection, a class token broadcast over the batch and concatenated in front, a learned
    position table added with a leading broadcast axis, bidirectional attention, classification from the class token. The
    class token's gradient is a sum over the batch axis of a strided view of the concatenation's gradient."""

    class Block(nn.Module):
        def __init__(self, d, heads):
            super().__init__()
            self.ln1, self.qkv, self.proj = nn.LayerNorm(d), nn.Linear(d, 3 * d), nn.Linear(d, d)
            self.ln2, self.fc1, self.fc2, self.heads = nn.LayerNorm(d), nn.Linear(d, 4 * d), nn.Linear(4 * d, d), heads

        def forward(self, x):
            B, S, _ = x.shape
            q, k, v = self.qkv(self.ln1(x)).view(B, S, 3, self.heads, -1).unbind(2)
            a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
            x = x + self.proj(a.transpose(1, 2).reshape(B, S, -1))
            return x + self.fc2(F.gelu(self.fc1(self.ln2(x))))

    class ViT(nn.Module):
        def __init__(self, d=64, patches=15, patch_dim=48, classes=8):
            super().__init__()
            self.embed = nn.Linear(patch_dim, d)
            self.cls = nn.Parameter(torch.randn(1, 1, d) * 0.1)
            self.pos = nn.Parameter(torch.randn(1, patches + 1, d) * 0.1)
            self.blocks = nn.ModuleList([Block(d, 1) for _ in range(2)])
            self.ln, self.head = nn.LayerNorm(d), nn.Linear(d, classes)

        def forward(self, patches, labels):
            x = self.embed(patches)
            x = torch.cat([self.cls.expand(x.shape[0], -1, -1), x], dim=1) + self.pos
            for block in self.blocks:
                x = block(x)
            return F.cross_entropy(self.head(self.ln(x)[:, 0]), labels)

    torch.manual_seed(23)
    m = _bf16_weights(ViT())
    patches, labels = torch.randn(4, 15, 48).bfloat16().float(), torch.randint(0, 8, (4,))
    loss, grads = _grads_by_unit_sgd(m, (patches, labels), str(tmp_path))
    ref = m(patches, labels)
    ref.backward()
    assert abs(loss - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    assert float(m.embed.weight.grad.abs().max()) > 0 and float(m.cls.grad.abs().max()) > 0
    _check_grads(m, grads)
    g = E.TrainingGraph(str(tmp_path), device=-1, optimizer="adamw", lr=3e-3)
    losses = [g.step(patches.numpy(), labels.numpy()) for _ in range(8)]
    assert losses[-1] < 0.5 * losses[0]
    g.close()


def test_external_gradient_reduction_reproduces_the_large_batch_step(tmp_path):
    """Two graphs stand for two data-parallel ranks: each runs forward and backward on its half of the batch, the gradients
    are averaged outside the graphs, each applies the update. Both end where one graph with the whole batch ends."""
    torch.manual_seed(24)
    m = _bf16_weights(Mlp())
    x, y = torch.randn(24, 32).bfloat16().float(), torch.randint(0, 16, (24,))
    d_full = E.export_graph(m, (x, y), str(tmp_path / "full"), fuse=False)
    d_half = E.export_graph(m, (x[:12], y[:12]), str(tmp_path / "half"), fuse=False)
    kw = dict(device=-1, optimizer="adamw", lr=1e-2, clip_grad_norm=0.5)
    full = E.TrainingGraph(d_full, **kw)
    ranks = [E.TrainingGraph(d_half, external_gradient_reduction=True, **kw) for _ in range(2)]
    with pytest.raises(RuntimeError, match="no gradients"):
        ranks[0].apply_update()
    with pytest.raises(RuntimeError, match="external_gradient_reduction"):
        full.gradients()
    for _ in range(3):
        lf = full.step(x.numpy(), y.numpy())
        losses = [ranks[0].step(x[:12].numpy(), y[:12].numpy()), ranks[1].step(x[12:].numpy(), y[12:].numpy())]
        assert abs(0.5 * sum(losses) - lf) < 2e-2 * max(abs(lf), 0.1)
        before = ranks[0].parameters()
        grads = [r.gradients() for r in ranks]
        mean = {k: 0.5 * (grads[0][k] + grads[1][k]) for k in grads[0]}
        for r in ranks:
            r.set_gradients(mean)
            r.apply_update()
        assert any(not np.array_equal(before[k], v) for k, v in ranks[0].parameters().items())
    assert ranks[0].steps == 3
    p0, p1, pf = ranks[0].parameters(), ranks[1].parameters(), full.parameters()
    for k in pf:
        assert np.array_equal(p0[k], p1[k])
        assert np.abs(p0[k] - pf[k]).max() < 1e-2, k
    for g in ranks + [full]:
        g.close()


def test_native_data_parallel_on_two_cpu_ranks():
    """Two processes (gloo): per-rank compiled plans, gradients averaged by one collective, identical weights on both ranks and
    the same result as one plan over the whole batch (tests/flow_worker.py: native_data_parallel)."""
    from test_flow_api import launch
    launch("native_dp", 2)


def test_mean_pooling_over_the_sequence_exports_and_differentiates(tmp_path):
    """x.mean(dim=1) lowers to a zero fill, one column sum per batch index into an fp32 buffer and a scaling cast; backward
    repeats the gradient over the reduced axis with a zero-stride copy."""
    class Pooled(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb, self.fc, self.head = nn.Embedding(50, 32), nn.Linear(32, 32), nn.Linear(32, 8)

        def forward(self, ids, labels):
            h = torch.tanh(self.fc(self.emb(ids)))          # [B, S, 32]
            return F.cross_entropy(self.head(h.mean(dim=1) + h.sum(1) * 0.125), labels)

    torch.manual_seed(25)
    m = _bf16_weights(Pooled())
    ids, labels = torch.randint(0, 50, (6, 9)), torch.randint(0, 8, (6,))
    loss, grads = _grads_by_unit_sgd(m, (ids, labels), str(tmp_path))
    ref = m(ids, labels)
    ref.backward()
    assert abs(loss - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    _check_grads(m, grads)
    text = open(os.path.join(str(tmp_path), "graph.txt")).read()
    assert text.count("op column_sum") == 12 and text.count("op cast") == 2
    # the same directory as an inference graph
    out = E.InferenceGraph(str(tmp_path), device=-1).run(ids.numpy(), labels.numpy())[0][0]
    assert abs(out - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))


def test_weight_decay_on_matrices_only_matches_torch_parameter_groups(tmp_path):
    torch.manual_seed(26)
    m = _bf16_weights(Mlp())
    x, y = torch.randn(24, 32).bfloat16().float(), torch.randint(0, 16, (24,))
    d = E.export_graph(m, (x, y), str(tmp_path), fuse=False)
    g = E.TrainingGraph(d, device=-1, optimizer="adamw", lr=1e-2, weight_decay=0.5, decay_matrices_only=True, clip_grad_norm=10.0)
    text = g.dump()
    assert text.count("op adamw_update") == 2 and "decay=0" in text and "decay=1" in text
    opt = torch.optim.AdamW([{"params": [p for p in m.parameters() if p.dim() >= 2], "weight_decay": 0.5},
                             {"params": [p for p in m.parameters() if p.dim() < 2], "weight_decay": 0.0}], lr=1e-2)
    for _ in range(5):
        ref = m(x, y)
        opt.zero_grad()
        ref.backward()
        opt.step()
        assert abs(g.step(x.numpy(), y.numpy()) - float(ref.detach())) < 3e-2 * max(abs(float(ref.detach())), 0.1)
    ps = g.parameters()
    for name, p in m.named_parameters():
        assert np.abs(ps[name] - p.detach().numpy().reshape(-1)).max() < 2.5e-2, name
    # the strong decay shows on the matrices and must not show on the vectors: compare with a run that decays everything
    h = E.TrainingGraph(d, device=-1, optimizer="adamw", lr=1e-2, weight_decay=0.5)
    for _ in range(5):
        h.step(x.numpy(), y.numpy())
    ph = h.parameters()
    assert np.abs(ph["ln.weight"]).mean() < np.abs(ps["ln.weight"]).mean() - 0.01
    g.close()
    h.close()


def test_compile_training_and_parameters_back_into_the_module(tmp_path):
    torch.manual_seed(27)
    m = _bf16_weights(Mlp())
    x, y = torch.randn(24, 32).bfloat16().float(), torch.randint(0, 16, (24,))
    before = float(m(x, y).detach())
    g = E.compile_training(m, (x, y), str(tmp_path), device=-1, optimizer="adamw", lr=1e-2)
    for _ in range(10):
        g.step(x.numpy(), y.numpy())
    want = g.evaluate(x.numpy(), y.numpy())
    g.copy_parameters_to(m)
    m.eval()
    after = float(m(x, y).detach())
    assert after < 0.7 * before and abs(after - want) < 3e-2 * max(want, 0.05)      # the module now computes what the graph trained
    g.close()


def test_multihead_attention_module_trains_natively(tmp_path):
    class Enc(nn.Module):
        def __init__(self):
            super().__init__()
            self.ln, self.mha, self.out = nn.LayerNorm(64), nn.MultiheadAttention(64, 1, batch_first=True), nn.Linear(64, 8)

        def forward(self, x, y):
            h = self.ln(x)
            a, _ = self.mha(h, h, h, need_weights=False)
            return F.cross_entropy(self.out(x + a)[:, 0], y)

    torch.manual_seed(28)
    m = _bf16_weights(Enc())
    x, y = torch.randn(4, 16, 64).bfloat16().float(), torch.randint(0, 8, (4,))
    loss, grads = _grads_by_unit_sgd(m, (x, y), str(tmp_path))
    ref = m(x, y)
    ref.backward()
    assert abs(loss - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    assert "mha.in_proj_weight" in grads and "mha.out_proj.weight" in grads
    scale = max(float(p.grad.abs().max()) for p in m.parameters())
    for name, p in m.named_parameters():
        r = p.grad.numpy().reshape(-1)
        # the key third of the packed bias shifts all scores of a row alike: zero true gradient, rounding is what is left
        tol = 3e-2 * (np.abs(r).max() + 1e-6) if name != "mha.in_proj_bias" else 3e-2 * (np.abs(r).max() + 1e-6) + 1e-3 * scale
        assert np.abs(grads[name] - r).max() <= tol, name


@pytest.mark.parametrize("norm_first", [True, False])
def test_torch_transformer_encoder_exports_and_trains_natively(tmp_path, norm_first):
    """nn.TransformerEncoder / nn.TransformerEncoderLayer (whose forward cannot be traced) are written out by the exporter:
    packed projection, fused attention, feed-forward, pre- or post-norm; gradients against autograd."""
    class Tagger(nn.Module):
        def __init__(self):
            super().__init__()
            layer = nn.TransformerEncoderLayer(64, 1, 128, dropout=0.0, activation="gelu", batch_first=True, norm_first=norm_first)
            self.emb, self.enc, self.head = nn.Embedding(50, 64), nn.TransformerEncoder(layer, 2, norm=nn.LayerNorm(64), enable_nested_tensor=False), nn.Linear(64, 8)

        def forward(self, ids, labels):
            return F.cross_entropy(self.head(self.enc(self.emb(ids))).view(-1, 8), labels.view(-1))

    torch.manual_seed(29)
    m = _bf16_weights(Tagger())
    ids, labels = torch.randint(0, 50, (3, 16)), torch.randint(0, 8, (3, 16))
    loss, grads = _grads_by_unit_sgd(m, (ids, labels), str(tmp_path))
    ref = m(ids, labels)
    ref.backward()
    assert abs(loss - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    scale = max(float(p.grad.abs().max()) for p in m.parameters())
    for name, p in m.named_parameters():
        r = p.grad.numpy().reshape(-1)
        extra = 1e-3 * scale if name.endswith("in_proj_bias") else 0.0       # the key third has zero true gradient
        assert np.abs(grads[name] - r).max() <= 3e-2 * (np.abs(r).max() + 1e-6) + extra, name
    text = open(os.path.join(str(tmp_path), "graph.txt")).read()
    assert text.count("op attention") == 2 and text.count("op layer_norm") == 5


def test_encoder_decoder_with_cross_attention_trains_natively(tmp_path):
    """A sequence-to-sequence model from torch's own building blocks: encoder over the source, decoder with causal
    self-attention and cross-attention over the encoder's output (query from one sequence, keys / values from another of a
    different length: two GEMMs reading row slices of the packed projection weight), tied nothing, token-level loss."""
    class Seq2Seq(nn.Module):
        def __init__(self):
            super().__init__()
            # gelu: with relu a pre-activation near zero falls on different sides in bf16 and in the fp32 reference, and the
            # gradient of that unit is all or nothing
            enc = nn.TransformerEncoderLayer(64, 1, 128, dropout=0.0, activation="gelu", batch_first=True, norm_first=True)
            dec = nn.TransformerDecoderLayer(64, 1, 128, dropout=0.0, activation="gelu", batch_first=True, norm_first=True)
            self.src, self.tgt = nn.Embedding(40, 64), nn.Embedding(40, 64)
            self.encoder = nn.TransformerEncoder(enc, 1, enable_nested_tensor=False)
            self.decoder = nn.TransformerDecoder(dec, 1, norm=nn.LayerNorm(64))
            self.head = nn.Linear(64, 40)

        def forward(self, src, tgt_in, tgt_out):
            memory = self.encoder(self.src(src))
            mask = nn.Transformer.generate_square_subsequent_mask(tgt_in.shape[1])
            h = self.decoder(self.tgt(tgt_in), memory, tgt_mask=mask, tgt_is_causal=True)
            return F.cross_entropy(self.head(h).view(-1, 40), tgt_out.view(-1))

    torch.manual_seed(30)
    m = _bf16_weights(Seq2Seq())
    src, tgt_in, tgt_out = torch.randint(0, 40, (2, 24)), torch.randint(0, 40, (2, 16)), torch.randint(0, 40, (2, 16))
    loss, grads = _grads_by_unit_sgd(m, (src, tgt_in, tgt_out), str(tmp_path))
    ref = m(src, tgt_in, tgt_out)
    ref.backward()
    assert abs(loss - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    scale = max(float(p.grad.abs().max()) for p in m.parameters())
    for name, p in m.named_parameters():
        r = p.grad.numpy().reshape(-1)
        # the encoder's gradients arrive through the cross-attention as bf16 activation gradients: small against the decoder's,
        # so their rounding is measured against the largest gradient of the model as well
        assert np.abs(grads[name] - r).max() <= 3e-2 * (np.abs(r).max() + 1e-6) + 1e-3 * scale, name
    text = open(os.path.join(str(tmp_path), "graph.txt")).read()
    assert text.count("op attention") == 3


def test_modern_decoder_block_with_rope_swiglu_and_grouped_query_attention_trains_natively(tmp_path):
    """Rotary position embedding (slices, negation, concatenation, broadcast tables), a gated SiLU feed-forward (chunk views),
    grouped-query attention (two query heads per key / value head) and bias-free projections: all on operators the IR already
    has, gradients against autograd."""
    def rope(t, cos, sin):            # t [B, heads, S, D]
        h = t.shape[-1] // 2
        rot = torch.cat([-t[..., h:], t[..., :h]], dim=-1)
        return t * cos + rot * sin
    class Block(nn.Module):
        def __init__(s, d=64, heads=2, kv_heads=1, seq=16):
            super().__init__()
            s.h, s.hk, s.dh = heads, kv_heads, d // heads
            s.ln1, s.ln2 = nn.LayerNorm(d), nn.LayerNorm(d)
            s.wq, s.wkv, s.wo = nn.Linear(d, d, bias=False), nn.Linear(d, 2 * kv_heads * s.dh, bias=False), nn.Linear(d, d, bias=False)
            s.gate_up, s.down = nn.Linear(d, 2 * 128, bias=False), nn.Linear(128, d, bias=False)
            pos = torch.arange(seq)[:, None] * (1.0 / 10000 ** (torch.arange(0, s.dh, 2) / s.dh))[None, :]
            s.register_buffer("cos", torch.cat([pos.cos(), pos.cos()], -1))
            s.register_buffer("sin", torch.cat([pos.sin(), pos.sin()], -1))
        def forward(s, x):
            B, S, D = x.shape
            h = s.ln1(x)
            q = s.wq(h).view(B, S, s.h, s.dh).transpose(1, 2)
            k, v = s.wkv(h).view(B, S, 2, s.hk, s.dh).unbind(2)
            k, v = k.transpose(1, 2), v.transpose(1, 2)
            q, k = rope(q, s.cos, s.sin), rope(k, s.cos, s.sin)
            a = F.scaled_dot_product_attention(q, k, v, is_causal=True, enable_gqa=True)
            x = x + s.wo(a.transpose(1, 2).reshape(B, S, D))
            g, u = s.gate_up(s.ln2(x)).chunk(2, dim=-1)
            return x + s.down(F.silu(g) * u)
    class LM(nn.Module):
        def __init__(s):
            super().__init__()
            s.emb, s.blocks, s.ln, s.head = nn.Embedding(96, 64), nn.ModuleList([Block(), Block()]), nn.LayerNorm(64), nn.Linear(64, 96, bias=False)
        def forward(s, ids, tgt):
            x = s.emb(ids)
            for b in s.blocks:
                x = b(x)
            return F.cross_entropy(s.head(s.ln(x)).view(-1, 96), tgt.view(-1))

    torch.manual_seed(31)
    m = _bf16_weights(LM())
    ids, tgt = torch.randint(0, 96, (2, 16)), torch.randint(0, 96, (2, 16))
    loss, grads = _grads_by_unit_sgd(m, (ids, tgt), str(tmp_path))
    ref = m(ids, tgt)
    ref.backward()
    assert abs(loss - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    _check_grads(m, grads)
    text = open(os.path.join(str(tmp_path), "graph.txt")).read()
    assert text.count("op attention") == 2 and "fn=6" in text           # fused attention with grouped heads; silu


def test_rms_norm_exports_onto_the_layer_norm_kernels_and_trains(tmp_path):
    """RMSNorm(x) = first half of LayerNorm([x, -x]) with unit scale and zero shift, times the learned scale."""
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.emb, self.n1, self.fc, self.n2, self.head = nn.Embedding(50, 64), nn.RMSNorm(64, eps=1e-6), nn.Linear(64, 64), nn.RMSNorm(64), nn.Linear(64, 8)

        def forward(self, ids, labels):
            h = self.emb(ids)
            h = h + F.silu(self.fc(self.n1(h)))
            return F.cross_entropy(self.head(F.rms_norm(self.n2(h), (64,)))[:, 0], labels)

    torch.manual_seed(32)
    m = _bf16_weights(Net())
    with torch.no_grad():
        m.n1.weight.mul_(torch.linspace(0.5, 1.5, 64))
    ids, labels = torch.randint(0, 50, (4, 12)), torch.randint(0, 8, (4,))
    loss, grads = _grads_by_unit_sgd(m, (ids, labels), str(tmp_path))
    ref = m(ids, labels)
    ref.backward()
    assert abs(loss - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    assert "n1.weight" in grads and "n2.weight" in grads
    _check_grads(m, grads)


def test_log_softmax_followed_by_nll_loss_becomes_one_cross_entropy_operator(tmp_path):
    class Classic(nn.Module):
        def __init__(self):
            super().__init__()
            self.fc1, self.fc2 = nn.Linear(32, 64), nn.Linear(64, 16)

        def forward(self, x, y):
            return F.nll_loss(F.log_softmax(self.fc2(torch.relu(self.fc1(x))), dim=1), y)

    torch.manual_seed(33)
    m = _bf16_weights(Classic())
    x, y = torch.randn(24, 32).bfloat16().float(), torch.randint(0, 16, (24,))
    d = E.export_graph(m, (x, y), str(tmp_path), fuse=False)
    text = open(os.path.join(d, "graph.txt")).read()
    assert text.count("op cross_entropy") == 1 and "log_softmax" not in text
    g = E.TrainingGraph(d, device=-1, optimizer="sgd", lr=0.1)
    opt = torch.optim.SGD(m.parameters(), lr=0.1)
    for _ in range(5):
        ref = m(x, y)
        opt.zero_grad()
        ref.backward()
        opt.step()
        assert abs(g.step(x.numpy(), y.numpy()) - float(ref.detach())) < 3e-2 * max(abs(float(ref.detach())), 0.1)
    g.close()

    class Leaks(nn.Module):
        def forward(self, x, y):
            lp = F.log_softmax(x, dim=1)
            return F.nll_loss(lp, y) + lp.sum() * 0.0

    with pytest.raises(Exception, match="only as the input of nll_loss"):
        E.export_graph(Leaks(), (torch.randn(4, 8), torch.randint(0, 8, (4,))), str(tmp_path / "leak"))


def test_classic_image_classifier_with_flatten_powers_and_nll_loss(tmp_path):
    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.body = nn.Sequential(nn.Flatten(), nn.Linear(64, 32), nn.ReLU(), nn.Identity(), nn.Linear(32, 16))

        def forward(self, img, y):
            z = self.body(img)
            return F.nll_loss(F.log_softmax(z ** 2 * 0.5 + z.pow(3) * 0.01, dim=1), y)

    torch.manual_seed(34)
    m = _bf16_weights(Net())
    img, y = torch.randn(8, 1, 8, 8).bfloat16().float(), torch.randint(0, 16, (8,))
    loss, grads = _grads_by_unit_sgd(m, (img, y), str(tmp_path))
    ref = m(img, y)
    ref.backward()
    assert abs(loss - float(ref.detach())) < 2e-2 * abs(float(ref.detach()))
    scale = max(float(p.grad.abs().max()) for p in m.parameters())
    for name, p in m.named_parameters():          # relu: units whose pre-activation is near zero may fall on the other side in bf16
        r = p.grad.numpy().reshape(-1)
        assert np.abs(grads[name] - r).max() <= 5e-2 * (np.abs(r).max() + 1e-6) + 5e-3 * scale, name
    with pytest.raises(Exception, match="exponent"):
        E.export_graph(type("P", (nn.Module,), {"forward": lambda self, x: x ** 1.5})(), (torch.rand(2, 8),), str(tmp_path / "p"))
