"""C++ inference API: export a network, load it through the C ABI of libofb_api.so, compare with PyTorch."""
import os

import pytest
import torch

from oneflow_b200.utils import export as E


def _model():
    torch.manual_seed(0)
    return torch.nn.Sequential(torch.nn.Linear(64, 256), torch.nn.GELU(), torch.nn.LayerNorm(256),
                               torch.nn.Sequential(torch.nn.Linear(256, 128), torch.nn.ReLU()), torch.nn.Dropout(0.1),
                               torch.nn.Linear(128, 16, bias=False))


def test_export_writes_graph_description(tmp_path):
    d = E.export_inference_graph(_model(), str(tmp_path))
    lines = open(os.path.join(d, "graph.txt")).read().splitlines()
    assert lines[0] == "oneflow_b200 inference graph v1"
    assert lines[1].startswith("linear 64 256") and lines[1].endswith("gelu")
    assert lines[2].startswith("layer_norm 256")
    assert lines[3].startswith("linear 256 128") and lines[3].endswith("relu")
    assert lines[4].split()[:3] == ["linear", "128", "16"] and lines[4].split()[4] == "-"
    assert os.path.getsize(os.path.join(d, "p0.weight.bin")) == 64 * 256 * 2


@pytest.mark.gpu
def test_cpp_inference_matches_pytorch(tmp_path):
    model = _model().eval()
    d = E.export_inference_graph(model, str(tmp_path))
    g = E.InferenceGraph(d)
    assert (g.in_features, g.out_features) == (64, 16)
    x = torch.randn(37, 64)
    y = g.forward(x.numpy())
    ref_model = _model().eval()
    for p in ref_model.parameters():
        p.data = p.data.bfloat16().float()
    ref = ref_model(x.bfloat16().float()).detach()
    torch.testing.assert_close(torch.from_numpy(y), ref, atol=5e-2, rtol=5e-2)
    g.close()
