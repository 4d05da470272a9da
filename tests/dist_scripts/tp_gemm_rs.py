"""GEMM -> reduce-scatter over a tensor-parallel group of real GPUs: the one-launch kernel against
(a) an fp32 reference built with ``torch.distributed`` and (b), with ``--bench``, the two-kernel
path and NCCL (``torch.matmul`` + ``reduce_scatter_tensor``), timed with CUDA events (max over
ranks).  Launched through torch.distributed.run, one rank per GPU."""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
os.environ.setdefault("MERAK_QUIET", "1")

import torch
import torch.distributed as dist


def timed(fn, iters, group):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier(group=group)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="1x1024x512x256")       # BxLxNxK(local) ; separated by commas
    ap.add_argument("--ag_shapes", default="")                  # all-gather -> GEMM: BxLxN(local)xK
    ap.add_argument("--bench", type=int, default=0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", required=True)
    o = ap.parse_args()
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl")
    from merak_b200.ops import _lib
    from merak_b200.parallel import fused_tp
    group = dist.group.WORLD
    n, rank = dist.get_world_size(), dist.get_rank()
    comm = fused_tp.get_comm(group, torch.device("cuda", local))
    assert comm is not None, "peer mapping unavailable"
    comm.force_one_launch = True
    results = []
    for spec in o.shapes.split(","):
        B, L, N, K = (int(v) for v in spec.split("x"))
        M, seg = B * L, L // n
        torch.manual_seed(1234 + rank)
        x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16) * 0.3
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.3
        torch.manual_seed(99)
        bias = torch.randn(N, device="cuda", dtype=torch.bfloat16)
        assert comm.one_launch_ok(M, N, seg)
        before = comm.fused_rs_calls
        got = comm.gemm_reduce(x, w, bias, seg, all_rows=False)
        assert comm.fused_rs_calls == before + 1, "the one-launch kernel did not run"
        full = x.float() @ w.float().t()
        dist.all_reduce(full, group=group)
        full = (full + bias.float()).view(B, n, seg, N)[:, rank].reshape(M // n, N)
        err = float((got.float() - full).abs().max())
        tol = 3e-2 * float(full.abs().max()) + 0.3
        rec = {"shape": spec, "max_err": err, "tol": tol, "ok": err <= tol}
        if o.bench:
            rec["fused_ms"] = timed(lambda: comm.gemm_reduce(x, w, bias, seg, all_rows=False), o.iters, group)
            comm.force_one_launch = False
            rec["two_kernel_ms"] = timed(lambda: comm.gemm_reduce(x, w, bias, seg, all_rows=False), o.iters, group)
            comm.force_one_launch = True
            out = torch.empty(M // n, N, device="cuda", dtype=torch.bfloat16)
            x3 = x.view(B, n, seg, K)

            def nccl():
                y = torch.matmul(x, w.t()).view(B, n, seg, N).transpose(0, 1).contiguous().view(M, N)
                dist.reduce_scatter_tensor(out.view(-1), y.view(-1), group=group)
                out.add_(bias)
            rec["nccl_ms"] = timed(nccl, o.iters, group)
            rec["gemm_only_ms"] = timed(lambda: torch.matmul(x, w.t()), o.iters, group)
            flops = 2.0 * M * N * K
            bytes_link = 2.0 * M * N * (n - 1) / n
            rec["roofline_ms"] = max(flops / 1601.6e12, bytes_link / 770e9) * 1e3
            rec["fraction_of_roofline"] = rec["roofline_ms"] / rec["fused_ms"]
        results.append(rec)
    for spec in [t for t in o.ag_shapes.split(",") if t]:
        B, L, N, K = (int(v) for v in spec.split("x"))
        M, seg = B * L, L // n
        torch.manual_seed(4321 + rank)
        xl = (torch.randn(B, seg, K, device="cuda", dtype=torch.bfloat16) * 0.3).view(B * seg, K)
        w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16) * 0.3
        y, gathered, _ = comm.gather_gemm(xl, w, None, seg)
        parts = [torch.empty_like(xl) for _ in range(n)]
        dist.all_gather(parts, xl, group=group)
        full = torch.stack([t.view(B, seg, K) for t in parts], 1).reshape(M, K)
        ref = full.float() @ w.float().t()
        err = float((y.float() - ref).abs().max())
        tol = 3e-2 * float(ref.abs().max()) + 0.3
        rec = {"shape": "ag " + spec, "max_err": err, "tol": tol, "ok": err <= tol and torch.equal(gathered, full)}
        if o.bench:
            rec["fused_ms"] = timed(lambda: comm.gather_gemm(xl, w, None, seg), o.iters, group)
            buf = torch.empty(n * xl.numel(), device="cuda", dtype=torch.bfloat16)

            def nccl_ag():
                dist.all_gather_into_tensor(buf, xl.view(-1), group=group)
                g = buf.view(n, B, seg, K).transpose(0, 1).reshape(M, K)
                return torch.matmul(g, w.t())
            rec["nccl_ms"] = timed(nccl_ag, o.iters, group)
            rec["gemm_only_ms"] = timed(lambda: torch.matmul(full, w.t()), o.iters, group)
            rec["roofline_ms"] = max(2.0 * M * N * K / 1601.6e12, 2.0 * M * K * (n - 1) / n / 770e9) * 1e3
            rec["fraction_of_roofline"] = rec["roofline_ms"] / rec["fused_ms"]
        results.append(rec)
    torch.cuda.synchronize()
    status = _lib.status()
    if rank == 0:
        with open(o.out, "w") as f:
            json.dump({"n": n, "results": results, "status": status}, f, indent=1)
        print(json.dumps({"n": n, "results": results, "status": status}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
