"""Expert parallelism: top-k softmax router, token dispatch to the ranks that own the experts,
per-expert SwiGLU MLPs, and the weighted combine.

The reference has no mixture-of-experts support (only inherited flags, Merak/core/pipeline/utils.py:
46-47); this module is what the DeepSeek-V2-Lite-shape workload needs.  Experts are split
contiguously over the expert-parallel group (a sub-group of the data-parallel group, see
``ProcessTopology``); expert parameters carry ``expert_parallel = True`` so the engine keeps them out
of the data-parallel gradient reduction over that group.

Data path of one layer (T tokens, k experts per token, E experts, n ranks):

1. router: fp32 logits, softmax, top-k                          -> weights [T,k], expert ids [T,k]
2. permute: the T*k (token, expert) pairs sorted by expert      -> rows ordered by destination rank
3. dispatch: all-to-all of the per-expert counts, then of the rows
4. experts: rows regrouped expert-major; one gate_up GEMM + SwiGLU + down GEMM per local expert
5. combine: inverse regroup, all-to-all back, scale by the router weight, scatter-add per token

On CUDA the row exchange uses the peer-store kernels of ``csrc/moe_dispatch.cu`` when the group is
peer-mapped (``comm_mode='fused'``); otherwise ``torch.distributed.all_to_all_single`` (gloo on CPU).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..ops.elementwise import swiglu
from ..ops.linear import linear as k_linear
from . import mpu


class _AllToAllRows(torch.autograd.Function):
    """Rows of ``x`` split by ``in_splits`` go to the ranks of ``group``; ``out_splits`` rows arrive."""

    @staticmethod
    def forward(ctx, x, in_splits: List[int], out_splits: List[int], group):
        ctx.group, ctx.in_splits, ctx.out_splits = group, in_splits, out_splits
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, dy):
        dx = dy.new_empty((sum(ctx.in_splits),) + tuple(dy.shape[1:]))
        dist.all_to_all_single(dx, dy.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return dx, None, None, None


def exchange_rows(x: torch.Tensor, in_splits: List[int], out_splits: List[int], group) -> torch.Tensor:
    if group is None or dist.get_world_size(group) == 1:
        return x
    return _AllToAllRows.apply(x, in_splits, out_splits, group)


# ---- peer-store exchange ---------------------------------------------------------------------------
FUSED_ENABLED = True      # cleared when ``comm_mode`` is not "fused"


class EPComm:
    """Peer-mapped receive buffers of one expert-parallel group for the push all-to-all kernel
    (``csrc/moe_dispatch.cu``).  Two buffers rotate: a rank can only start call k after every rank
    has finished call k-1, i.e. after everybody has consumed what call k-2 delivered."""

    def __init__(self, symm):
        self.symm, self.n, self.rank = symm, symm.n, symm.rank
        self.bufs = [None, None]
        self.cap_bytes = 0
        self.calls = 0
        self.budget_ms = 20000

    def _ensure(self, worst_bytes: int):
        """``worst_bytes``: size of the largest possible delivery (every row of every rank arriving
        here); the same on all ranks, so growing needs no negotiation."""
        if worst_bytes > self.cap_bytes:
            torch.cuda.synchronize(self.symm.device)
            dist.barrier(group=self.symm.group)
            self.cap_bytes = max(worst_bytes, 1 << 20)
            self.bufs = [self.symm.alloc(self.cap_bytes, torch.uint8) for _ in range(2)]

    def push(self, x: torch.Tensor, send_begin: List[int], dst_row: List[int], rows_out: int,
             worst_rows: int) -> torch.Tensor:
        import ctypes
        from ..ops import _lib
        H = x.shape[1]
        self._ensure(worst_rows * H * x.element_size())
        buf = self.bufs[self.calls % 2]
        self.calls += 1
        n = self.n
        sb = (ctypes.c_longlong * (n + 1))(*send_begin)
        dr = (ctypes.c_longlong * n)(*dst_row)
        x = x.contiguous()
        _lib.check(_lib.kernels().mrk_moe_alltoall_push(buf.table, self.symm.ctrl.table, n, self.rank, x.data_ptr(), sb,
                                                        dr, H, x.element_size(), self.calls, 1, self.budget_ms,
                                                        _lib.stream_ptr()), "mrk_moe_alltoall_push")
        nbytes = rows_out * H * x.element_size()
        return buf.tensor[:nbytes].view(x.dtype).view(rows_out, H).clone()


_EP_COMMS = {}


def get_ep_comm(group, device) -> Optional[EPComm]:
    """Collective on first use: the EPComm of ``group`` or None (CPU, peer mapping unavailable)."""
    key = id(group)
    if key not in _EP_COMMS:
        sg = None
        if FUSED_ENABLED and device.type == "cuda":
            from .symm import SymmGroup
            sg = SymmGroup.create(group, device)
        _EP_COMMS[key] = EPComm(sg) if sg is not None else None
    return _EP_COMMS[key]


class _PushRows(torch.autograd.Function):
    """All-to-all of rows by peer stores.  ``C[s][d]`` = rows rank s sends to rank d (host matrix);
    ``forward_dir`` True sends this rank's blocks C[rank][:], False returns blocks C[:][rank]."""

    @staticmethod
    def forward(ctx, x, C, comm: EPComm, forward_dir: bool):
        ctx.C, ctx.comm, ctx.forward_dir = C, comm, forward_dir
        return _push(x, C, comm, forward_dir)

    @staticmethod
    def backward(ctx, dy):
        return _push(dy, ctx.C, ctx.comm, not ctx.forward_dir), None, None, None


def _push(x, C, comm: EPComm, forward_dir: bool):
    n, me = comm.n, comm.rank
    if forward_dir:
        sizes = [C[me][d] for d in range(n)]                                   # my block for each destination
        dst_row = [sum(C[s][d] for s in range(me)) for d in range(n)]            # after lower-ranked sources
        rows_out = sum(C[s][me] for s in range(n))
    else:
        sizes = [C[s][me] for s in range(n)]                                   # give each source its rows back
        dst_row = [sum(C[s][d] for d in range(me)) for s in range(n)]            # its block for me, in its order
        rows_out = sum(C[me][d] for d in range(n))
    begin = [0]
    for v in sizes:
        begin.append(begin[-1] + v)
    return comm.push(x, begin, dst_row, rows_out, worst_rows=sum(sum(r) for r in C))


class TopKRouter(nn.Module):
    """Softmax-then-top-k gate (DeepSeek-V2: ``norm_topk_prob`` off, ``routed_scaling_factor``)."""

    def __init__(self, hidden_size: int, num_experts: int, top_k: int, scaling: float = 1.0,
                 norm_topk_prob: bool = False):
        super().__init__()
        self.top_k, self.num_experts, self.scaling, self.norm_topk_prob = top_k, num_experts, scaling, norm_topk_prob
        self.weight = nn.Parameter(torch.empty(num_experts, hidden_size))
        nn.init.normal_(self.weight, std=0.006)

    def forward(self, x2: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        logits = F.linear(x2.float(), self.weight.float())
        probs = torch.softmax(logits, dim=-1)
        w, idx = torch.topk(probs, self.top_k, dim=-1)
        if self.norm_topk_prob:
            w = w / (w.sum(-1, keepdim=True) + 1e-20)
        return w * self.scaling, idx, probs


def load_balance_loss(probs: torch.Tensor, idx: torch.Tensor, num_experts: int) -> torch.Tensor:
    """Switch-style auxiliary loss: E * sum_e(fraction of routed pairs to e * mean router prob of e)."""
    T, k = idx.shape
    frac = torch.zeros(num_experts, dtype=probs.dtype, device=probs.device)
    frac.scatter_add_(0, idx.reshape(-1), torch.ones(T * k, dtype=probs.dtype, device=probs.device))
    frac = frac / (T * k)
    return num_experts * (frac * probs.mean(0)).sum()


class ExpertMLPs(nn.Module):
    """The local experts' SwiGLU MLPs as stacked weights: ``gate_up_proj [E_local, 2F, H]`` (gate rows
    first, as the fused Llama projection) and ``down_proj [E_local, H, F]``."""

    def __init__(self, num_local: int, hidden_size: int, ffn: int, std: float = 0.006, first_global: int = 0,
                 seed: Optional[int] = None):
        super().__init__()
        self.num_local, self.hidden_size, self.ffn = num_local, hidden_size, ffn
        gen = None
        if seed is not None:       # expert e draws the same weights whatever the expert-parallel degree
            gen = torch.Generator()
        gu = torch.empty(num_local, 2 * ffn, hidden_size)
        dn = torch.empty(num_local, hidden_size, ffn)
        for e in range(num_local):
            if gen is not None:
                gen.manual_seed(seed * 100003 + first_global + e)
            gu[e].normal_(0.0, std, generator=gen)
            dn[e].normal_(0.0, std, generator=gen)
        self.gate_up_proj = nn.Parameter(gu)
        self.down_proj = nn.Parameter(dn)
        for p in (self.gate_up_proj, self.down_proj):
            p.expert_parallel = True

    def forward(self, rows: torch.Tensor, counts: List[int]) -> torch.Tensor:
        """``rows`` are expert-major: the first counts[0] rows belong to local expert 0, and so on."""
        outs, off = [], 0
        mg_gu = getattr(self.gate_up_proj, "main_grad", None)
        mg_dn = getattr(self.down_proj, "main_grad", None)
        for e, c in enumerate(counts):
            if c == 0:
                continue
            xe = rows[off:off + c]
            w_gu, w_dn = self.gate_up_proj[e], self.down_proj[e]
            if mg_gu is not None:        # wgrad GEMMs accumulate straight into the expert's slice
                w_gu.main_grad, w_dn.main_grad = mg_gu[e], mg_dn[e]
            h = swiglu(k_linear(xe, w_gu))
            outs.append(k_linear(h, w_dn))
            off += c
        if not outs:
            return rows.new_zeros((0, self.hidden_size)) + 0.0 * (self.gate_up_proj.sum() + self.down_proj.sum())
        return torch.cat(outs, dim=0)


class MoELayer(nn.Module):
    """Routed experts (expert parallel) plus optional always-on shared experts."""

    def __init__(self, hidden_size: int, moe_ffn: int, num_experts: int, top_k: int, num_shared: int = 0,
                 scaling: float = 1.0, norm_topk_prob: bool = False, aux_loss_alpha: float = 0.0, std: float = 0.006,
                 seed: Optional[int] = 1234):
        super().__init__()
        ep, rank = mpu.get_expert_parallel_world_size(), mpu.get_expert_parallel_rank()
        if num_experts % ep != 0:
            raise ValueError("%d experts do not divide over expert-parallel degree %d" % (num_experts, ep))
        self.ep, self.ep_rank = ep, rank
        self.num_experts, self.num_local, self.top_k = num_experts, num_experts // ep, top_k
        self.aux_loss_alpha = aux_loss_alpha
        self.gate = TopKRouter(hidden_size, num_experts, top_k, scaling, norm_topk_prob)
        self.experts = ExpertMLPs(self.num_local, hidden_size, moe_ffn, std, first_global=rank * self.num_local,
                                  seed=seed)
        self.shared_experts = None
        if num_shared > 0:
            from ..ops.modules import Linear
            self.shared_experts = nn.ModuleDict({
                "gate_up_proj": Linear(hidden_size, 2 * moe_ffn * num_shared, bias=False),
                "down_proj": Linear(moe_ffn * num_shared, hidden_size, bias=False)})
            for m in self.shared_experts.values():
                nn.init.normal_(m.weight, std=std)
        self.aux_loss: Optional[torch.Tensor] = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        H = shape[-1]
        x2 = x.reshape(-1, H)
        T, k, E, n = x2.shape[0], self.top_k, self.num_experts, self.ep
        w, idx, probs = self.gate(x2)
        self.aux_loss = load_balance_loss(probs, idx, E) * self.aux_loss_alpha if self.aux_loss_alpha > 0 else None

        # (token, expert) pairs sorted by expert: rows for rank r are contiguous and expert-ordered
        flat_e = idx.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        token_of = torch.div(order, k, rounding_mode="floor")
        send = x2.index_select(0, token_of)
        counts = torch.bincount(flat_e, minlength=E)

        group = mpu.get_expert_parallel_group() if n > 1 else None
        if n > 1:
            all_counts = torch.empty(n * E, dtype=counts.dtype, device=counts.device)
            dist.all_gather_into_tensor(all_counts, counts, group=group)       # every rank's per-expert counts
            all_counts = all_counts.view(n, n, self.num_local)                 # [source, destination, local expert]
            rc = all_counts[:, self.ep_rank, :]                                 # rows arriving here, per source
            C = all_counts.sum(2).tolist()                                      # rows source -> destination
            in_splits, out_splits = C[self.ep_rank], [C[s_][self.ep_rank] for s_ in range(n)]
            comm = get_ep_comm(group, x.device) if x.is_cuda else None
            if comm is not None:
                recv = _PushRows.apply(send, C, comm, True)
            else:
                recv = exchange_rows(send, in_splits, out_splits, group)
            # received rows are [source][local expert]; regroup expert-major
            src_expert = torch.arange(self.num_local, device=x.device).repeat(n)
            row_expert = torch.repeat_interleave(src_expert, rc.reshape(-1))
            regroup = torch.argsort(row_expert, stable=True)
            rows = recv.index_select(0, regroup)
            per_expert = rc.sum(0).tolist()
        else:
            rows, per_expert = send, counts.tolist()

        y = self.experts(rows, per_expert)

        if n > 1:
            inv = torch.empty_like(regroup)
            inv[regroup] = torch.arange(regroup.numel(), device=x.device)
            if comm is not None:
                back = _PushRows.apply(y.index_select(0, inv), C, comm, False)
            else:
                back = exchange_rows(y.index_select(0, inv), out_splits, in_splits, group)
        else:
            back = y
        pair_w = w.reshape(-1).index_select(0, order).to(back.dtype).unsqueeze(1)
        out = torch.zeros_like(x2).index_add_(0, token_of, back * pair_w)
        if self.shared_experts is not None:
            h = swiglu(self.shared_experts["gate_up_proj"](x2))
            out = out + self.shared_experts["down_proj"](h)
        return out.view(shape)
