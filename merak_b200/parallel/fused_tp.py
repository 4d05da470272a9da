"""Tensor-parallel linears whose collective is fused into the GEMM kernel.

* ``row_linear_fused``    ``Y = sum_ranks(X_r W_r^T)``: the GEMM writes its bf16 partial product into a
  peer-mapped buffer; the rank that owns a sequence segment pulls that segment's rows of every
  rank's partial over NVLink (coalesced 16-byte loads), sums them in fp32 and adds the bias
  (reduce-scatter); without sequence parallelism a second kernel pulls the other ranks' reduced
  rows (all-reduce).
* ``column_linear_fused`` ``Y = gather(X) W^T`` under Megatron sequence parallelism: a few CTAs of
  the GEMM grid stream the peers' sequence shards into the local gathered matrix (bulk async
  copies) while the other CTAs already multiply this rank's own rows.

The backward passes use the mirror-image kernel (column: dgrad GEMM -> reduce-scatter / all-reduce;
row: all-gather -> dgrad GEMM) and the weight gradients reuse the gathered operand.

These replace the ``torch.distributed`` collectives around the matmuls of the reference's
``ColumnParallelLinear`` / ``RowParallelLinear`` (Merak/core/mpu/layers.py:168-369,
Merak/core/mpu/mappings.py:30-120).
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as G
from ..ops.linear import _as2d, _bias_grad, _weight_grad
from .symm import SymmGroup

REDUCE_CTAS = 8      # CTAs of a fused GEMM -> reduce-scatter that only pull and sum (resident from the start)
# GEMM -> reduce-scatter as ONE launch (sub-tile flags, reduce phase inside the GEMM kernel) or as the
# GEMM followed by the pull-and-sum kernel.  Measured on two B200s the two-launch form is still the
# faster one (0.319 ms against 0.353 ms at 8192 x 4096 x 5504; NCCL + matmul: 0.451 ms), so it is the
# default; MERAK_TP_ONE_LAUNCH=1 selects the one-launch kernel.
ONE_LAUNCH = os.environ.get("MERAK_TP_ONE_LAUNCH", "0") == "1"
GATHER_CTAS = 16     # upper bound on the CTAs of a fused all-gather GEMM that only move data
ENABLED = True      # cleared by the engine when ``comm_mode`` is not "fused"
_FLAG_B_MN = 16


class TPComm:
    """Symmetric buffers and call counters of one tensor-parallel group.  Every rank makes the same
    sequence of calls, so counters (barrier epochs, buffer rotation) stay in lockstep."""

    def __init__(self, symm: SymmGroup):
        self.symm = symm
        self.n, self.rank = symm.n, symm.rank
        self.device = symm.device
        self.part = [None, None]            # bf16 partial products of this rank (rotating), pulled by the owners
        self.part_elems = 0
        self.red = [None, None]             # bf16 reduced rows of this rank (rotating), pulled for an all-reduce
        self.red_elems = 0
        self.stage = [None, None]           # bf16 staging of this rank's all-gather input (rotating)
        self.stage_elems = 0
        self.rs_calls = 0
        self.ag_calls = 0
        self.tile_flags = None              # per-sub-tile epochs of the one-launch GEMM -> reduce-scatter
        self.tile_flag_units = 0
        self.fused_rs_calls = 0
        self.force_one_launch = False
        self.rs_queue = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.seg_flags = torch.zeros(1 << 14, dtype=torch.int32, device=self.device)
        self._flag_segs = 0
        self._flag_calls = 0
        self.budget_ms = 20000

    def _quiesce(self):
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.symm.group)

    def _ensure_part(self, elems: int, red_elems: int):
        if elems > self.part_elems:
            self._quiesce()
            self.part_elems = max(elems, int(self.part_elems * 1.5))
            self.part = [self.symm.alloc(self.part_elems * 2, torch.bfloat16) for _ in range(2)]
        if red_elems > self.red_elems:
            self._quiesce()
            self.red_elems = max(red_elems, int(self.red_elems * 1.5))
            self.red = [self.symm.alloc(self.red_elems * 2, torch.bfloat16) for _ in range(2)]

    def _ensure_stage(self, elems: int):
        if elems > self.stage_elems:
            self._quiesce()
            self.stage_elems = max(elems, int(self.stage_elems * 1.5))
            self.stage = [self.symm.alloc(self.stage_elems * 2, torch.bfloat16) for _ in range(2)]

    # -- GEMM -> reduce-scatter (or all-reduce) ----------------------------------------------------
    @staticmethod
    def one_launch_ok(M: int, N: int, seg_rows: int) -> bool:
        """Shapes the one-launch kernel tiles: 128-row sub-tiles that do not straddle sequence
        segments, 64-column TMA store boxes."""
        return M % 128 == 0 and seg_rows % 128 == 0 and N % 64 == 0 and M > 128 and N > 128

    def _ensure_tile_flags(self, units: int):
        """The flag array only ever sees growing epochs, so one allocation serves every shape up to
        its size; a larger shape re-allocates (collective, every rank takes the same path)."""
        if units > self.tile_flag_units:
            self._quiesce()
            self.tile_flag_units = max(units, 1 << 14)
            self.tile_flags = self.symm.alloc(4 * self.n * self.tile_flag_units, torch.int32)
            self.fused_rs_calls = 0

    def gemm_reduce(self, x2: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], seg_rows: int,
                    all_rows: bool, b_mn: bool = False) -> torch.Tensor:
        """x2 [M, Kl] (this rank's slice of the contraction), w [N, Kl] (or [Kl, N] with ``b_mn``).
        Returns rows of ``sum over ranks of x2 w^T (+ bias)``: all M rows when ``all_rows`` else this
        rank's.  The GEMM writes its partial product into a peer-mapped buffer; the owners of the rows
        pull and sum them (fp32) in the kernel that follows.  Buffers rotate over two calls: a rank
        re-uses one only after it has passed the barrier of the call in between, which every rank
        reaches after it has finished reading."""
        lib = _lib.kernels()
        M, K = x2.shape
        N = w.shape[1] if b_mn else w.shape[0]
        rows_local = M // self.n
        self._ensure_part(M * N, rows_local * N if all_rows else 0)
        k = self.rs_calls
        self.rs_calls += 1
        part = self.part[k % 2]
        st = _lib.stream_ptr()
        if all_rows:
            red = self.red[k % 2]
            dst_ptr = red.local_ptr
        else:
            out = torch.empty(rows_local, N, dtype=torch.bfloat16, device=x2.device)
            dst_ptr = out.data_ptr()
        if (ONE_LAUNCH or self.force_one_launch) and self.one_launch_ok(M, N, seg_rows) and x2.stride(1) == 1 and \
                w.stride(1) == 1:
            # one launch: sub-tile flags instead of a barrier, the sum starts while peers still multiply
            units = int(lib.mrk_gemm_bf16_rs_units(M, N))
            self._ensure_tile_flags(units)
            self.fused_rs_calls += 1
            _lib.check(lib.mrk_gemm_bf16_rs(
                x2.data_ptr(), w.data_ptr(), part.table, self.tile_flags.table, dst_ptr,
                bias.data_ptr() if bias is not None else None, M, N, K, x2.stride(0), w.stride(0),
                _FLAG_B_MN if b_mn else 0, self.n, self.rank, seg_rows, self.fused_rs_calls, 3, REDUCE_CTAS,
                self.rs_queue.data_ptr(), self.budget_ms, st), "mrk_gemm_bf16_rs")
        else:
            G.gemm(x2, w, b_mn=b_mn, out=part.tensor[:M * N].view(M, N))
            _lib.check(lib.mrk_tp_reduce_pull(part.table, self.symm.ctrl.table, self.n, self.rank, dst_ptr, rows_local,
                                              N, seg_rows, bias.data_ptr() if bias is not None else None, k + 1, 1,
                                              self.budget_ms, st), "mrk_tp_reduce_pull")
        if not all_rows:
            return out
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x2.device)
        _lib.check(lib.mrk_tp_gather_rows(red.table, self.symm.ctrl.table, self.n, self.rank, out.data_ptr(), M, N,
                                          seg_rows, k + 1, 1, self.budget_ms, st), "mrk_tp_gather_rows")
        return out

    # -- all-gather -> GEMM ---------------------------------------------------------------------------
    def _gather_ctas(self, M: int, N: int, K: int) -> int:
        """CTAs taken from the GEMM grid to stream the peers' shards: enough for the remote bytes to
        arrive while the tiles that do not need them are computed (one SM sustains about 35 GB/s of
        global -> shared -> global bulk copies), no more."""
        gemm_s = 2.0 * M * N * K / 1.3e15
        window = gemm_s * (self.n - 1) / self.n
        remote = 2.0 * M * K * (self.n - 1) / self.n
        need = int(remote / max(window, 1e-6) / 35e9) + 1
        return max(2, min(GATHER_CTAS, (need + 1) // 2 * 2))       # even: the pair kernel gathers with whole clusters

    def gather_gemm(self, x_local: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], seg_rows: int,
                    b_mn: bool = False, act: int = G.ACT_NONE, want_preact: bool = False):
        """x_local [M/n, K] (this rank's sequence shard).  Returns (y [M, N], gathered [M, K], preact)."""
        lib = _lib.kernels()
        Ml, K = x_local.shape
        M = Ml * self.n
        N = w.shape[1] if b_mn else w.shape[0]
        self._ensure_stage(Ml * K)
        k = self.ag_calls
        self.ag_calls += 1
        stage = self.stage[k % 2]
        stage.tensor[:Ml * K].view(Ml, K).copy_(x_local)
        num_seg = M // seg_rows
        if num_seg != self._flag_segs:
            assert num_seg <= self.seg_flags.numel()
            self.seg_flags.zero_()
            self._flag_segs, self._flag_calls = num_seg, 0
        gather_ctas = self._gather_ctas(M, N, K)
        self._flag_calls += gather_ctas          # every gather CTA bumps every segment counter once
        gathered = torch.empty(M, K, dtype=torch.bfloat16, device=x_local.device)
        y = torch.empty(M, N, dtype=torch.bfloat16, device=x_local.device)
        pre = torch.empty(M, N, dtype=torch.bfloat16, device=x_local.device) if want_preact else None
        _lib.check(lib.mrk_gemm_bf16_ag(
            gathered.data_ptr(), stage.table, w.data_ptr(), y.data_ptr(), M, N, K, w.stride(0), N,
            bias.data_ptr() if bias is not None else None, pre.data_ptr() if pre is not None else None, N, act,
            _FLAG_B_MN if b_mn else 0, 1.0, self.symm.ctrl.table, self.seg_flags.data_ptr(),
            self._flag_calls, gather_ctas, self.n, self.rank, seg_rows, k + 1, self.budget_ms,
            _lib.stream_ptr()), "mrk_gemm_bf16_ag")
        return y, gathered, pre


_COMMS: Dict[int, Optional[TPComm]] = {}


def get_comm(group, device: torch.device) -> Optional[TPComm]:
    """Collective on first use: the TPComm of ``group`` or None when peer mapping is unavailable."""
    key = id(group)
    if key not in _COMMS:
        sg = SymmGroup.create(group, device) if device.type == "cuda" and dist.get_world_size(group) <= 8 else None
        _COMMS[key] = TPComm(sg) if sg is not None else None
    return _COMMS[key]


def reset():
    _COMMS.clear()


class _RowLinearFused(torch.autograd.Function):
    """Row-parallel linear: forward GEMM -> reduce-scatter (sequence parallel) or all-reduce."""

    @staticmethod
    def forward(ctx, x, weight, bias, comm: TPComm, sequence_parallel: bool):
        N, Kl = weight.shape
        x2 = _as2d(x, Kl)
        B, L = x.shape[0], x.shape[1]
        seg = L // comm.n
        out = comm.gemm_reduce(x2, weight, bias, seg, all_rows=not sequence_parallel)
        ctx.save_for_backward(x2, weight, bias)
        ctx.comm, ctx.sp, ctx.in_shape, ctx.seg = comm, sequence_parallel, x.shape, seg
        return out.view(B, seg if sequence_parallel else L, N)

    @staticmethod
    def backward(ctx, dy):
        x2, weight, bias = ctx.saved_tensors
        comm: TPComm = ctx.comm
        N, Kl = weight.shape
        dy2 = _as2d(dy, N)
        if ctx.sp:
            # dY is sharded along the sequence: all-gather it inside the dgrad GEMM
            dx2, dy_full, _ = comm.gather_gemm(dy2, weight, None, ctx.seg, b_mn=True)
        else:
            dy_full = dy2
            dx2, _ = G.gemm(dy2, weight, b_mn=True)
        dw = _weight_grad(dy_full, x2, weight) if weight.requires_grad else None
        # the bias is added once (by rank 0) to the summed output: its gradient is the column sum of
        # this rank's rows of dY; the engine sums sequence-parallel parameters over the group
        db = _bias_grad(dy2 if ctx.sp else dy_full, bias)
        return dx2.view(ctx.in_shape), dw, db, None, None


class _ColumnLinearFused(torch.autograd.Function):
    """Column-parallel linear: forward all-gather -> GEMM under sequence parallelism (plain GEMM
    otherwise); backward dgrad GEMM -> reduce-scatter / all-reduce."""

    @staticmethod
    def forward(ctx, x, weight, bias, comm: TPComm, sequence_parallel: bool):
        Nl, K = weight.shape
        x2 = _as2d(x, K)
        B = x.shape[0]
        if sequence_parallel:
            seg = x.shape[1]
            y, x_full, _ = comm.gather_gemm(x2, weight, bias, seg)
            L = seg * comm.n
        else:
            L = x.shape[1]
            seg = L // comm.n
            x_full = x2
            y, _ = G.gemm(x2, weight, bias=bias)
        ctx.save_for_backward(x_full, weight, bias)
        ctx.comm, ctx.sp, ctx.seg, ctx.in_shape = comm, sequence_parallel, seg, x.shape
        return y.view(B, L, Nl)

    @staticmethod
    def backward(ctx, dy):
        x_full, weight, bias = ctx.saved_tensors
        comm: TPComm = ctx.comm
        Nl, K = weight.shape
        dy2 = _as2d(dy, Nl)
        dx2 = comm.gemm_reduce(dy2, weight, None, ctx.seg, all_rows=not ctx.sp, b_mn=True)
        dw = _weight_grad(dy2, x_full, weight) if weight.requires_grad else None
        db = _bias_grad(dy2, bias)
        return dx2.view(ctx.in_shape), dw, db, None, None


def usable(x: torch.Tensor, weight: torch.Tensor, n: int, sequence_parallel: bool, seq_dim: int,
           input_sharded: bool) -> bool:
    """Shapes the fused kernels accept: bf16 CUDA, batch-first 3-D activations, sequence shards that
    are whole row blocks of the GEMM."""
    if not (x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and x.dim() == 3
            and seq_dim == 1):
        return False
    L = x.shape[1] * (n if (sequence_parallel and input_sharded) else 1)
    if L % n != 0:
        return False
    return weight.shape[0] % 32 == 0 and weight.shape[1] % 32 == 0


def row_linear_fused(x, weight, bias, comm: TPComm, sequence_parallel: bool):
    return _RowLinearFused.apply(x, weight, bias, comm, sequence_parallel)


def column_linear_fused(x, weight, bias, comm: TPComm, sequence_parallel: bool):
    return _ColumnLinearFused.apply(x, weight, bias, comm, sequence_parallel)
