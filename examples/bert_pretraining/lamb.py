"""LAMB optimizer (layer-wise adaptive moments for large-batch BERT pre-training), plain PyTorch.
Plays the role of the apex FusedLAMB the reference's example wires in through the trainer hook
(examples/bert_pretraining/run_bert.py:104-117)."""
import torch


class Lamb(torch.optim.Optimizer):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-6, weight_decay=0.01, max_grad_norm=1.0):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.max_grad_norm = max_grad_norm

    @torch.no_grad()
    def step(self, closure=None):
        grads = [p.grad for g in self.param_groups for p in g["params"] if p.grad is not None]
        if not grads:
            return None
        gnorm = torch.sqrt(sum((g.float() ** 2).sum() for g in grads))
        clip = torch.clamp(gnorm / self.max_grad_norm, min=1.0) if self.max_grad_norm > 0 else 1.0
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float() / clip
                st = self.state[p]
                if not st:
                    st["step"], st["m"], st["v"] = 0, torch.zeros_like(g), torch.zeros_like(g)
                st["step"] += 1
                st["m"].mul_(b1).add_(g, alpha=1 - b1)
                st["v"].mul_(b2).addcmul_(g, g, value=1 - b2)
                m_hat = st["m"] / (1 - b1 ** st["step"])
                v_hat = st["v"] / (1 - b2 ** st["step"])
                upd = m_hat / (v_hat.sqrt() + group["eps"]) + group["weight_decay"] * p.float()
                w_norm, u_norm = p.float().norm(), upd.norm()
                trust = torch.where((w_norm > 0) & (u_norm > 0), w_norm / u_norm, torch.ones_like(w_norm))
                p.add_((-group["lr"] * trust * upd).to(p.dtype))
        return None
