"""``flow.Generator``: one seed, one random stream per device.

The reference's generator (python/oneflow/framework/generator.py, oneflow/core/framework/random_generator.h)
may be built for ``"auto"``: it then serves whichever device the consuming op runs on. ``torch.Generator`` is
bound to one device, so this class keeps a ``torch.Generator`` per device, all seeded alike, and hands the
right one out through :func:`resolve`. Ops that take ``generator=`` call ``resolve(generator, device)`` first.
"""
import torch

__all__ = ["Generator", "default_generator", "resolve", "get_rng_state", "set_rng_state"]


def _parse(device):
    s = str(device)
    if s == "auto":
        return None
    kind, _, idx = s.partition(":")
    if kind not in ("cpu", "cuda") or (idx and not idx.isdigit()):
        raise RuntimeError(f"Expected one of cpu, cuda, auto device type at start of device string: {s}")
    if kind == "cpu":
        return torch.device("cpu")              # the host has one stream whatever the index says
    if idx and (not torch.cuda.is_available() or int(idx) >= torch.cuda.device_count()):
        from oneflow._oneflow_internal import exception
        raise exception.RuntimeError(f"CUDA device index {idx} is out of range")
    return torch.device("cuda", int(idx)) if idx else torch.device("cuda")


class Generator:
    """``flow.Generator(device="auto")`` with ``manual_seed`` / ``seed`` / ``initial_seed`` / ``get_state`` /
    ``set_state``. ``device`` fixes the device of an explicit generator; an ``"auto"`` one follows its consumer."""

    def __init__(self, device="auto", *, _default=False):
        self._device = _parse(device)
        self._default = _default
        self._seed = torch.default_generator.initial_seed()
        self._gens = {}

    @property
    def device(self):
        if self._device is not None:
            return self._device
        return torch.device("cuda" if torch.cuda.is_available() else "cpu")

    def for_device(self, device=None):
        """The ``torch.Generator`` that draws on ``device`` (this generator's own device when None)."""
        dev = torch.device(device) if device is not None else self.device
        if self._device is not None and dev.type != self._device.type:
            dev = self._device
        if dev.type == "cuda" and dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        if self._default:
            return torch.default_generator if dev.type == "cpu" else torch.cuda.default_generators[dev.index]
        g = self._gens.get(dev)
        if g is None:
            g = self._gens[dev] = torch.Generator(device=dev)
            g.manual_seed(self._seed)
        return g

    def _all(self):
        if self._default:
            gens = [torch.default_generator]
            if torch.cuda.is_available() and torch.cuda.is_initialized():
                gens += list(torch.cuda.default_generators)
            return gens
        return list(self._gens.values())

    def manual_seed(self, seed):
        self._seed = int(seed)
        if self._default:
            torch.manual_seed(self._seed)
        for g in self._all():
            g.manual_seed(self._seed)
        return self

    def seed(self):
        self.manual_seed(torch.Generator().seed() & ((1 << 63) - 1))
        return self._seed

    def initial_seed(self):
        return self.for_device("cpu").initial_seed() if self._default else self._seed

    def get_state(self):
        """The state of this generator's own device; an ``"auto"`` generator answers with its host stream."""
        return self.for_device(self._device or "cpu").get_state()

    def set_state(self, state):
        self.for_device(self._device or "cpu").set_state(state.cpu() if isinstance(state, torch.Tensor) else state)
        return self

    def __repr__(self):
        return f"oneflow.Generator(device='{self._device or 'auto'}', seed={self.initial_seed()})"


default_generator = Generator("auto", _default=True)


def resolve(generator, device=None):
    """``generator`` as a ``torch.Generator`` for ``device``; None and plain torch generators pass through."""
    if isinstance(generator, Generator):
        return generator.for_device(device)
    return generator


def get_rng_state():
    return torch.get_rng_state()


def set_rng_state(state):
    torch.set_rng_state(state.cpu() if isinstance(state, torch.Tensor) else state)
