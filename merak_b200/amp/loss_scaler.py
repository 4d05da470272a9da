"""Loss scaling for fp16 training."""
from __future__ import annotations


class DynamicLossScaler:
    """fp16 loss scaling with hysteresis (Merak/core/zero/utils.py:232-384)."""

    def __init__(self, init_scale=2.0 ** 16, scale_factor=2.0, scale_window=1000, min_scale=1.0, hysteresis=2,
                 static: bool = False):
        self.cur_scale = float(init_scale)
        self.scale_factor, self.scale_window, self.min_scale = scale_factor, scale_window, min_scale
        self.delayed_shift, self.cur_hysteresis = hysteresis, hysteresis
        self.last_overflow_iter, self.cur_iter = -1, 0
        self.static = static

    def update_scale(self, overflow: bool):
        if self.static:
            return
        if overflow:
            if self.delayed_shift == 1 or self.cur_hysteresis == 1:
                self.cur_scale = max(self.cur_scale / self.scale_factor, self.min_scale)
            else:
                self.cur_hysteresis -= 1
            self.last_overflow_iter = self.cur_iter
        else:
            if (self.cur_iter - self.last_overflow_iter) % self.scale_window == 0:
                self.cur_hysteresis = self.delayed_shift
                self.cur_scale *= self.scale_factor
        self.cur_iter += 1

    def state_dict(self):
        return dict(self.__dict__)

    def load_state_dict(self, sd):
        self.__dict__.update(sd)
