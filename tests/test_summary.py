import torch

from oneflow_b200.utils import summary as S


def test_crc32c_known_vectors():
    assert S.crc32c(b"") == 0
    assert S.crc32c(b"123456789") == 0xE3069283
    assert S.crc32c(bytes(32)) == 0x8A9136AA


def test_event_file_round_trip(tmp_path):
    with S.SummaryWriter(str(tmp_path)) as w:
        for step in range(5):
            w.add_scalar("loss", 1.0 / (step + 1), step)
        w.add_histogram("weights", torch.randn(1000), 5)
        w.add_text("note", "hello", 6)
        path = w.path
    events = list(S.read_events(path))
    scalars = [(s, t, v) for s, t, v in events if t == "loss"]
    assert [s for s, _, _ in scalars] == [0, 1, 2, 3, 4]
    assert abs(scalars[2][2] - 1.0 / 3) < 1e-6
    assert ("weights" in [t for _, t, _ in events]) and ("note" in [t for _, t, _ in events])
