"""Polynomial-decay learning rate with linear warm-up (the schedule of the reference's
examples/bert_pretraining/schedulers.py)."""


class PolyWarmUpScheduler:
    def __init__(self, optimizer, warmup: float, total_steps: int, degree: float = 0.5):
        self.optimizer, self.warmup, self.total, self.degree = optimizer, warmup, max(1, total_steps), degree
        self.base = [g["lr"] for g in optimizer.param_groups]
        self.last_step = 0
        self._apply()

    def _factor(self):
        progress = self.last_step / self.total
        if progress < self.warmup:
            return progress / self.warmup
        return max(0.0, 1.0 - progress) ** self.degree

    def _apply(self):
        for g, b in zip(self.optimizer.param_groups, self.base):
            g["lr"] = b * self._factor()

    def step(self):
        self.last_step += 1
        self._apply()

    def get_last_lr(self):
        return [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self):
        return {"last_step": self.last_step, "base": self.base}

    def load_state_dict(self, sd):
        self.last_step, self.base = sd["last_step"], sd["base"]
        self._apply()
