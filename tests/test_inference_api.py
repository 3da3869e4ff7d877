"""C++ inference API: export a network, load it through the C ABI of libofb_api.so (graph compiler + executor), compare with
PyTorch. The host implementation of the operators (device -1) runs everywhere; the GPU tests run the sm_100a kernels."""
import os

import numpy as np
import pytest
import torch
import torch.nn as nn
import torch.nn.functional as F

from oneflow_b200.utils import export as E


def _bf16_weights(m):
    for p in m.parameters():
        p.data = p.data.bfloat16().float()
    return m


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.GELU(), torch.nn.LayerNorm(256),
                               torch.nn.Sequential(torch.nn.Linear(256, 128), torch.nn.ReLU()), torch.nn.Dropout(0.1),
                               torch.nn.Linear(128, 16, bias=False))


class Block(nn.Module):
    """Embedding + one pre-LN transformer layer + output projection, written the usual PyTorch way."""

    def __init__(self, d=64, heads=4, vocab=96, seq=16):
        super().__init__()
        self.emb, self.pos = nn.Embedding(vocab, d), nn.Embedding(seq, d)
        self.ln1, self.qkv, self.proj = nn.LayerNorm(d), nn.Linear(d, 3 * d), nn.Linear(d, d)
        self.ln2, self.fc1, self.fc2 = nn.LayerNorm(d), nn.Linear(d, 4 * d), nn.Linear(4 * d, d)
        self.head = nn.Linear(d, vocab, bias=False)
        self.heads = heads

    def forward(self, ids):
        B, S = ids.shape
        x = self.emb(ids) + self.pos(torch.arange(S))
        q, k, v = self.qkv(self.ln1(x)).view(B, S, 3, self.heads, -1).unbind(2)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
        x = x + self.proj(a.transpose(1, 2).reshape(B, S, -1))
        x = x + self.fc2(F.gelu(self.fc1(self.ln2(x))))
        return self.head(x)


class TwoBranches(nn.Module):
    """Two independent towers (they can run on different streams), joined by a concatenation; an unfused attention built from
    matmul and softmax; an in-place activation."""

    def __init__(self):
        super().__init__()
        self.a1, self.a2 = nn.Linear(32, 64), nn.Linear(64, 32)
        self.b1, self.b2 = nn.Linear(32, 128), nn.Linear(128, 32)
        self.act = nn.ReLU(inplace=True)
        self.out = nn.Linear(64, 8)

    def forward(self, x, y):
        a = self.a2(torch.tanh(self.a1(x)))                      # [B, T, 32]
        b = self.b2(self.act(self.b1(y))) * 0.5                  # [B, T, 32]
        scores = torch.matmul(a, b.transpose(-1, -2)) / 4.0      # [B, T, T]
        mixed = torch.matmul(torch.softmax(scores, -1), b)       # [B, T, 32]
        z = torch.cat([a + mixed, b], dim=-1)                    # [B, T, 64]
        return self.out(z), scores


def _run_host(module, inputs, tmp_path, **kw):
    d = E.export_graph(module, inputs, str(tmp_path))
    g = E.InferenceGraph(d, device=-1, **kw)
    outs = g.run(*[t.numpy() for t in inputs])
    return g, outs


def test_export_writes_graph_description(tmp_path):
    d = E.export_inference_graph(_model(), str(tmp_path))
    lines = open(os.path.join(d, "graph.txt")).read().splitlines()
    assert lines[0] == "oneflow_b200 inference graph v1"
    assert lines[1].startswith("linear 64 256") and lines[1].endswith("gelu")
    assert lines[2].startswith("layer_norm 256")
    assert lines[3].startswith("linear 256 128") and lines[3].endswith("relu")
    assert lines[4].split()[:3] == ["linear", "128", "16"] and lines[4].split()[4] == "-"
    assert os.path.getsize(os.path.join(d, "p0.weight.bin")) == 64 * 256 * 2


def test_layer_list_graph_on_the_host_runtime(tmp_path):
    """The layer-list form has no batch size: the plan is compiled for the rows of the first call and again when they change."""
    model = _bf16_weights(_model().eval())
    d = E.export_inference_graph(model, str(tmp_path))
    g = E.InferenceGraph(d, device=-1)
    for rows in (5, 12, 5):
        x = torch.randn(rows, 64).bfloat16().float()
        y = g.forward(x.numpy())
        torch.testing.assert_close(torch.from_numpy(y), model(x).detach(), atol=3e-2, rtol=3e-2)
    g.close()


def test_transformer_block_graph_on_the_host_runtime(tmp_path):
    torch.manual_seed(1)
    m = _bf16_weights(Block().eval())
    ids = torch.randint(0, 96, (2, 16))
    g, outs = _run_host(m, (ids,), tmp_path)
    ref = m(ids).detach().numpy().reshape(-1)
    assert np.abs(outs[0] - ref).max() < 0.05 * np.abs(ref).max()
    text = open(os.path.join(str(tmp_path), "graph.txt")).read()
    # the attention reads q, k, v in place from the packed projection; GELU and both residual additions ride in GEMM epilogues
    assert "op attention" in text and "q_stride=192 kv_stride=192" in text and "op copy" not in text
    assert "act=gelu" in text and text.count("op binary") == 1 and text.count("op unary") == 0
    st = g.stats()
    assert st["ops"] == 11 and st["streams_used"] == 2          # the two embedding lookups are independent
    assert st["arena_bytes"] < st["activation_bytes"]           # buffers with disjoint lifetimes share memory
    # other ids, same plan
    ids2 = torch.randint(0, 96, (2, 16))
    out2 = g.run(ids2.numpy())[0]
    assert np.abs(out2 - m(ids2).detach().numpy().reshape(-1)).max() < 0.05 * np.abs(ref).max()
    g.close()


@pytest.mark.parametrize("n_streams", [1, 3])
def test_branches_concat_and_unfused_attention_on_the_host_runtime(tmp_path, n_streams):
    torch.manual_seed(2)
    m = _bf16_weights(TwoBranches().eval())
    x, y = torch.randn(3, 8, 32).bfloat16().float(), torch.randn(3, 8, 32).bfloat16().float()
    g, outs = _run_host(m, (x, y), tmp_path, n_streams=n_streams)
    ref_out, ref_scores = m(x.clone(), y.clone())
    assert np.abs(outs[0] - ref_out.detach().numpy().reshape(-1)).max() < 3e-2
    assert np.abs(outs[1] - ref_scores.detach().numpy().reshape(-1)).max() < 3e-2
    text = open(os.path.join(str(tmp_path), "graph.txt")).read()
    assert "tb=1" in text                                       # b^T is read in place as a K-major operand, no transpose copy
    assert g.stats()["streams_used"] == min(n_streams, 2)
    # many calls through one plan: the scheduler's dependency state carries over correctly
    for _ in range(3):
        again = g.run(x.numpy(), y.numpy())
        assert np.array_equal(again[0], outs[0]) and np.array_equal(again[1], outs[1])
    g.close()


def test_graph_errors_are_reported(tmp_path):
    class Bad(nn.Module):
        def forward(self, x):
            return torch.cumsum(x, -1)
    with pytest.raises(ValueError, match="cannot export operator cumsum"):
        E.export_graph(Bad(), (torch.randn(2, 8),), str(tmp_path / "bad"))
    d = tmp_path / "broken"
    d.mkdir()
    (d / "graph.txt").write_text("oneflow_b200 graph v2\ntensor 0 bf16 input 2 4 8\ntensor 1 bf16 act 2 4 8\n"
                                 "op linear in=0,1,-1,-1 out=1 act=none\ninput 0\noutput 1\n")
    with pytest.raises(RuntimeError, match="linear"):
        E.InferenceGraph(str(d), device=-1)
    (d / "graph.txt").write_text("oneflow_b200 graph v2\ntensor 0 bf16 input 2 4 8\ntensor 1 bf16 act 2 4 8\n"
                                 "op unary in=1 out=1 fn=3\ninput 0\noutput 1\n")
    with pytest.raises(RuntimeError, match="before it is written"):
        E.InferenceGraph(str(d), device=-1)
    m = _bf16_weights(Block().eval())
    g, _ = _run_host(m, (torch.randint(0, 96, (2, 16)),), tmp_path / "ok")
    with pytest.raises(ValueError, match="elements"):
        g.run(np.zeros((3, 16), dtype=np.int64))
    g.close()


@pytest.mark.gpu
def test_cpp_inference_matches_pytorch(tmp_path):
    model = _model().eval()
    d = E.export_inference_graph(model, str(tmp_path))
    g = E.InferenceGraph(d)
    assert (g.in_features, g.out_features) == (64, 16)
    x = torch.randn(37, 64)
    y = g.forward(x.numpy())
    ref_model = _bf16_weights(_model().eval())
    ref = ref_model(x.bfloat16().float()).detach()
    torch.testing.assert_close(torch.from_numpy(y), ref, atol=5e-2, rtol=5e-2)
    g.close()


@pytest.mark.gpu
def test_transformer_block_graph_on_the_gpu_runtime(tmp_path):
    """The same exported graph on the sm_100a kernels (tcgen05 GEMMs with fused epilogues, fused attention reading the packed
    projection, LayerNorm, gather) over two CUDA streams, against PyTorch fp32 and against the host runtime."""
    torch.manual_seed(1)
    m = _bf16_weights(Block(d=128, heads=2, vocab=256, seq=128).eval())
    ids = torch.randint(0, 256, (2, 128))
    d = E.export_graph(m, (ids,), str(tmp_path))
    g = E.InferenceGraph(d, device=0)
    out = g.run(ids.numpy())[0]
    ref = m(ids).detach().numpy().reshape(-1)
    assert np.abs(out - ref).max() < 0.05 * np.abs(ref).max()
    host = E.InferenceGraph(d, device=-1).run(ids.numpy())[0]
    assert np.abs(out - host).max() < 0.05 * np.abs(ref).max()
    for _ in range(3):
        assert np.array_equal(g.run(ids.numpy())[0], out)
    assert g.stats()["graph_replays"] == 3     # every run after the first is one CUDA-graph launch
    g.close()


@pytest.mark.gpu
def test_branches_graph_on_the_gpu_runtime(tmp_path):
    torch.manual_seed(2)
    m = _bf16_weights(TwoBranches().eval())
    x, y = torch.randn(4, 64, 32).bfloat16().float(), torch.randn(4, 64, 32).bfloat16().float()
    d = E.export_graph(m, (x, y), str(tmp_path))
    g = E.InferenceGraph(d, device=0, n_streams=2)
    outs = g.run(x.numpy(), y.numpy())
    ref_out, ref_scores = m(x.clone(), y.clone())
    assert np.abs(outs[0] - ref_out.detach().numpy().reshape(-1)).max() < 5e-2
    assert np.abs(outs[1] - ref_scores.detach().numpy().reshape(-1)).max() < 5e-2
    assert g.stats()["streams_used"] == 2
    # replays of the recorded two-stream graph read the inputs of their own call, not those of the recording
    for seed in (5, 6):
        torch.manual_seed(seed)
        x2, y2 = torch.randn(4, 64, 32).bfloat16().float(), torch.randn(4, 64, 32).bfloat16().float()
        outs2 = g.run(x2.numpy(), y2.numpy())
        r_out, r_scores = m(x2.clone(), y2.clone())
        assert np.abs(outs2[0] - r_out.detach().numpy().reshape(-1)).max() < 5e-2
        assert np.abs(outs2[1] - r_scores.detach().numpy().reshape(-1)).max() < 5e-2
    assert g.stats()["graph_replays"] == 2
    g.close()


class Glu(nn.Module):
    """Views that need strided copies (chunk halves, a slice of an input, a row select, a transposed output), a tied weight
    used by an embedding lookup and by a linear layer, softmax output."""

    def __init__(self):
        super().__init__()
        self.emb, self.fc, self.ln = nn.Embedding(50, 32), nn.Linear(32, 64), nn.LayerNorm(32)

    def forward(self, ids, y):
        x = self.emb(ids)
        a, b = self.fc(x).chunk(2, dim=-1)
        g = self.ln(a * torch.sigmoid(b) + y[:, 1:, :])
        logits = F.linear(g[:, -1], self.emb.weight)
        return torch.softmax(logits, -1), g.transpose(1, 2).contiguous()


def test_views_tied_weights_and_two_outputs_on_the_host_runtime(tmp_path):
    torch.manual_seed(4)
    m = _bf16_weights(Glu().eval())
    ids, y = torch.randint(0, 50, (3, 7)), torch.randn(3, 8, 32).bfloat16().float()
    g, outs = _run_host(m, (ids, y), tmp_path)
    r1, r2 = m(ids, y)
    assert np.abs(outs[0] - r1.detach().numpy().reshape(-1)).max() < 3e-2
    assert np.abs(outs[1] - r2.detach().numpy().reshape(-1)).max() < 3e-2
    text = open(os.path.join(str(tmp_path), "graph.txt")).read()
    assert text.count("file=") == 5           # embedding table (once, although two operators read it), fc.weight / bias, ln.weight / bias
    assert text.count("op copy") == 5 and text.count("op embedding") == 1
    g.close()


def test_cpp_program_links_the_api_and_runs_a_graph(tmp_path):
    """A C++ program (csrc/api/examples/run_graph.cpp) compiled against oneflow_api.h and libofb_api.so loads an exported
    transformer block and reproduces what the Python binding computes: the API is usable from C++ as documented."""
    import shutil
    import subprocess
    if shutil.which("g++") is None:
        pytest.skip("no C++ compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    api = os.path.join(root, "oneflow_b200", "csrc", "api")
    lib = os.path.join(root, "oneflow_b200", "lib")
    exe = str(tmp_path / "run_graph")
    r = subprocess.run(["g++", "-std=c++17", "-O1", os.path.join(api, "examples", "run_graph.cpp"), "-I", api, "-L", lib, "-lofb_api",
                        "-lofb_kernels", "-lofb_core", f"-Wl,-rpath,{lib}", "-o", exe], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    torch.manual_seed(1)
    m = _bf16_weights(Block().eval())
    ids = torch.randint(0, 96, (2, 16))
    d = E.export_graph(m, (ids,), str(tmp_path / "g"))
    ids.numpy().astype(np.int64).tofile(str(tmp_path / "ids.bin"))
    r = subprocess.run([exe, d, "-1", str(tmp_path / "ids.bin")], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr[-2000:]
    out = np.array([float(v) for v in r.stdout.strip().split()], dtype=np.float32)
    py = E.InferenceGraph(d, device=-1).run(ids.numpy())[0]
    assert out.shape == py.shape and np.allclose(out, py, rtol=1e-5, atol=1e-5)
    assert "ops 11" in r.stderr


def test_compile_from_torch_runs_a_module_through_cached_native_plans(tmp_path):
    """oneflow.framework.infer_compiler: the wrapper exports per input signature, caches the loaded graphs, lets attribute
    access through to the wrapped module, and saves / loads the exported directories."""
    from oneflow.framework.infer_compiler import DeployableModule, compile_from_torch
    torch.manual_seed(1)
    m = _bf16_weights(Block().eval())
    dm = compile_from_torch(m, options={"size": 2})
    assert isinstance(dm, DeployableModule) and compile_from_torch(dm) is dm
    ids = torch.randint(0, 96, (2, 16))
    out = dm(ids)
    ref = m(ids).detach()
    assert out.shape == ref.shape and float((out - ref).abs().max()) < 0.05 * float(ref.abs().max())
    assert dm.heads == m.heads and set(dm.state_dict()) == set(m.state_dict())          # attributes and weights of the module
    first = dm.get_graph()
    assert torch.equal(dm(ids), out) and dm.get_graph() is first                         # same signature: the cached plan
    ids3 = torch.randint(0, 96, (3, 16))
    assert dm(ids3).shape == (3, 16, 96) and dm.get_graph() is not first                 # another batch size: another plan
    saved = dm.save_graph(str(tmp_path / "saved"))
    fresh = compile_from_torch(m).load_graph(os.path.join(saved, "graph0"), (ids,), run_warmup=True)
    assert torch.equal(fresh(ids), out)
    eager = compile_from_torch(m, use_graph=False)
    assert torch.equal(eager(ids), m(ids))


def test_torch_compile_backend_on_the_native_runtime():
    from oneflow.framework.infer_compiler import oneflow_backend
    torch.manual_seed(2)
    mlp = _bf16_weights(nn.Sequential(nn.Linear(32, 64), nn.GELU(), nn.LayerNorm(64), nn.Linear(64, 16)).eval())
    x = torch.randn(8, 32).bfloat16().float()
    compiled = torch.compile(mlp, backend=oneflow_backend)
    with torch.no_grad():
        y = compiled(x)
        assert float((y - mlp(x)).abs().max()) < 3e-2

        class Odd(nn.Module):                       # an operator the exporter does not know: that graph runs eagerly
            def forward(self, t):
                return torch.sin(t) * 2

        odd = torch.compile(Odd(), backend=oneflow_backend)
        assert torch.allclose(odd(x), torch.sin(x) * 2)


def test_multihead_attention_module_exports_as_fused_attention(tmp_path):
    class Enc(nn.Module):
        def __init__(self):
            super().__init__()
            self.ln, self.mha, self.out = nn.LayerNorm(64), nn.MultiheadAttention(64, 1, batch_first=True), nn.Linear(64, 8)

        def forward(self, x):
            h = self.ln(x)
            a, _ = self.mha(h, h, h, need_weights=False)
            return self.out(x + a)

    torch.manual_seed(3)
    m = _bf16_weights(Enc().eval())
    x = torch.randn(2, 16, 64).bfloat16().float()
    g, outs = _run_host(m, (x,), tmp_path)
    ref = m(x).detach().numpy().reshape(-1)
    assert np.abs(outs[0] - ref).max() < 3e-2 * max(np.abs(ref).max(), 1.0)
    text = open(os.path.join(str(tmp_path), "graph.txt")).read()
    assert text.count("op attention") == 1 and "q_stride=192" in text          # q, k, v read in place from the packed projection
    g.close()

    class Weights(nn.Module):
        def __init__(self):
            super().__init__()
            self.mha = nn.MultiheadAttention(64, 1, batch_first=True)

        def forward(self, x):
            return self.mha(x, x, x)[0]

    with pytest.raises(Exception, match="need_weights=False"):
        E.export_graph(Weights().eval(), (x,), str(tmp_path / "w"))


def test_torch_transformer_model_exports(tmp_path):
    """nn.Transformer (encoder-decoder) as one leaf: both stacks are written out by the exporter."""
    class Translator(nn.Module):
        def __init__(self):
            super().__init__()
            self.core = nn.Transformer(d_model=64, nhead=1, num_encoder_layers=1, num_decoder_layers=2, dim_feedforward=128, dropout=0.0,
                                       activation="gelu", batch_first=True, norm_first=True)
            self.src, self.tgt, self.head = nn.Embedding(40, 64), nn.Embedding(40, 64), nn.Linear(64, 40)

        def forward(self, src, tgt):
            mask = nn.Transformer.generate_square_subsequent_mask(tgt.shape[1])
            return self.head(self.core(self.src(src), self.tgt(tgt), tgt_mask=mask, tgt_is_causal=True))

    torch.manual_seed(4)
    m = _bf16_weights(Translator().eval())
    src, tgt = torch.randint(0, 40, (2, 24)), torch.randint(0, 40, (2, 16))
    g, outs = _run_host(m, (src, tgt), tmp_path)
    ref = m(src, tgt).detach().numpy().reshape(-1)
    assert np.abs(outs[0] - ref).max() < 4e-2 * max(np.abs(ref).max(), 1.0)
    assert open(os.path.join(str(tmp_path), "graph.txt")).read().count("op attention") == 1 + 2 * 2
    g.close()


def test_sqrt_and_clamp_at_zero_export_as_compositions(tmp_path):
    class M(nn.Module):
        def forward(self, x):
            return torch.sqrt(x * x + 1.0) + x.clamp(min=0) + torch.clamp(x, 0)

    x = torch.randn(4, 16).bfloat16().float()
    g, outs = _run_host(M(), (x,), tmp_path)
    ref = M()(x).numpy().reshape(-1)
    assert np.abs(outs[0] - ref).max() < 2e-2 * np.abs(ref).max()
    text = open(os.path.join(str(tmp_path), "graph.txt")).read()
    assert "fn=9" in text and text.count("fn=3") == 2            # rsqrt; relu twice
    g.close()


def test_decode_step_with_key_value_cache_matches_the_full_forward(tmp_path):
    """Serving with a cache needs nothing special from the runtime: the decode step is a module of its own whose inputs and
    outputs include the cache tensors (one query position attends the cached keys plus its own: Sq = 1, Sk = S)."""
    class Attn(nn.Module):
        def __init__(self, d=64, vocab=96, seq=16):
            super().__init__()
            self.emb, self.pos, self.ln = nn.Embedding(vocab, d), nn.Embedding(seq, d), nn.LayerNorm(d)
            self.q, self.kv, self.o, self.head = nn.Linear(d, d), nn.Linear(d, 2 * d), nn.Linear(d, d), nn.Linear(d, vocab)

        def full(self, ids):                                          # [B, S] -> logits of the last position, and the cache
            B, S = ids.shape
            x = self.emb(ids) + self.pos(torch.arange(S))
            h = self.ln(x)
            k, v = self.kv(h).view(B, S, 2, 1, -1).unbind(2)
            a = F.scaled_dot_product_attention(self.q(h).view(B, S, 1, -1).transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
            x = x + self.o(a.transpose(1, 2).reshape(B, S, -1))
            return self.head(x[:, -1]), k.contiguous(), v.contiguous()

    class Prefill(nn.Module):
        def __init__(self, net):
            super().__init__()
            self.net = net

        def forward(self, ids):
            return self.net.full(ids)

    class Decode(nn.Module):
        def __init__(self, net, position):
            super().__init__()
            self.net, self.position = net, position

        def forward(self, token, k_cache, v_cache):                  # token [B, 1]; caches [B, S, 1, D]
            net, B = self.net, token.shape[0]
            x = net.emb(token) + net.pos(torch.full((1,), self.position))
            h = net.ln(x)
            k_new, v_new = net.kv(h).view(B, 1, 2, 1, -1).unbind(2)
            k, v = torch.cat([k_cache, k_new], dim=1), torch.cat([v_cache, v_new], dim=1)
            a = F.scaled_dot_product_attention(net.q(h).view(B, 1, 1, -1).transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
            x = x + net.o(a.transpose(1, 2).reshape(B, 1, -1))
            return net.head(x[:, -1]), k, v

    torch.manual_seed(5)
    net = _bf16_weights(Attn().eval())
    ids = torch.randint(0, 96, (2, 12))
    want = net.full(ids)[0].detach().numpy().reshape(-1)
    pre = E.InferenceGraph(E.export_graph(Prefill(net), (ids[:, :11],), str(tmp_path / "prefill")), device=-1)
    _, k_cache, v_cache = pre.run(ids[:, :11].numpy())
    k0, v0 = torch.from_numpy(k_cache).view(2, 11, 1, 64), torch.from_numpy(v_cache).view(2, 11, 1, 64)
    dec = E.InferenceGraph(E.export_graph(Decode(net, 11), (ids[:, 11:], k0, v0), str(tmp_path / "decode")), device=-1)
    logits, k1, v1 = dec.run(ids[:, 11:].numpy(), k0.numpy(), v0.numpy())
    assert np.abs(logits - want).max() < 3e-2 * np.abs(want).max()
    assert k1.size == 2 * 12 * 64 and np.array_equal(k1.reshape(2, 12, 64)[:, :11], k_cache.reshape(2, 11, 64))
    pre.close()
    dec.close()
