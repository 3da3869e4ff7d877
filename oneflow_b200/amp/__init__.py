"""``flow.amp``: autocast and the loss-scale policies nn.Graph consumes
(reference: python/oneflow/amp/grad_scaler.py:17-60, dynamic_loss_scale_schedule_kernel.cu)."""
import torch

autocast = torch.autocast


class GradScaler:
    """Dynamic loss scaling: the scale doubles (growth_factor) after ``growth_interval`` clean steps and
    shrinks (backoff_factor) when a non-finite gradient is found; that step's update is skipped."""
    dynamic = True

    def __init__(self, init_scale=2.0 ** 30, growth_factor=2.0, backoff_factor=0.5, growth_interval=2000):
        if growth_factor <= 1.0 or not 0.0 < backoff_factor < 1.0:
            raise ValueError("growth_factor must be > 1 and backoff_factor in (0, 1)")
        self._scale, self.growth_factor, self.backoff_factor, self.growth_interval = float(init_scale), growth_factor, backoff_factor, growth_interval
        self._good_steps = 0

    def get_scale(self):
        return self._scale

    def update(self, found_inf):
        if found_inf:
            self._scale *= self.backoff_factor
            self._good_steps = 0
        else:
            self._good_steps += 1
            if self._good_steps >= self.growth_interval:
                self._scale *= self.growth_factor
                self._good_steps = 0

    def state_dict(self):
        return {"scale": self._scale, "good_steps": self._good_steps}

    def load_state_dict(self, sd):
        self._scale, self._good_steps = float(sd["scale"]), int(sd["good_steps"])


class StaticGradScaler:
    dynamic = False

    def __init__(self, scale_factor):
        if scale_factor <= 0:
            raise ValueError("StaticGradScaler's scale_factor must be > 0")
        self._scale = float(scale_factor)

    def get_scale(self):
        return self._scale

    def update(self, found_inf):
        pass

    def state_dict(self):
        return {"scale": self._scale}

    def load_state_dict(self, sd):
        self._scale = float(sd["scale"])
