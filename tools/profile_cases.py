"""Small stand-alone cases of the hot kernels, sized for a profiler capture: inputs larger than the
126 MB L2 so DRAM figures mean something, a few hundred MB on the device, a handful of launches.

    python tools/profile_cases.py <case> [--iters N]

Cases: gemm, gemm_gelu, gemm_k1024, gemm_table, wgrad, attn_fwd, attn_bwd, norm, adamw, dp_step, ag_gemm, tp_reduce,
cross_entropy, rope, swiglu, embedding, colsum, moe_push.
Each prints the CUDA-event time per launch and the achieved TFLOP/s or GB/s.  The multi-rank
kernels run with all ranks' buffers on this one GPU and the cross-rank barriers pre-satisfied, so
they measure the kernels' data path, not NVLink.
"""
from __future__ import annotations

import argparse
import ctypes

import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from merak_b200.ops import _lib          # noqa: E402
from merak_b200.ops import gemm as G     # noqa: E402


def _time(fn, iters):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def _table(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*ptrs)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("case")
    ap.add_argument("--iters", type=int, default=3)
    o = ap.parse_args()
    dev = torch.device("cuda")
    torch.manual_seed(0)
    bf = torch.bfloat16
    lib = _lib.kernels()
    it = o.iters
    if o.case in ("gemm", "gemm_gelu", "gemm_k1024"):
        M, N, K = (16384, 4096, 4096) if o.case != "gemm_k1024" else (16384, 3072, 1024)
        a = torch.randn(M, K, device=dev, dtype=bf)
        b = torch.randn(N, K, device=dev, dtype=bf) * 0.02
        bias = torch.randn(N, device=dev, dtype=bf)
        act = G.ACT_GELU_ERF if o.case == "gemm_gelu" else G.ACT_NONE
        ms = _time(lambda: G.gemm(a, b, bias=bias, act=act, want_preact=o.case == "gemm_gelu"), it)
        print("%s %dx%dx%d: %.3f ms  %.1f TFLOP/s" % (o.case, M, N, K, ms, 2.0 * M * N * K / ms / 1e9))
    elif o.case == "gemm_table":
        # forward / data-gradient / weight-gradient GEMMs of the model configurations, against torch.matmul
        # (cuBLAS) on the same box: median of 20 launches each, L2 flushed between launches
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

        def med(fn, n=20):
            for _ in range(5):
                fn()
            ts = []
            for _ in range(n):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                fn()
                e1.record()
                torch.cuda.synchronize()
                ts.append(e0.elapsed_time(e1))
            return sorted(ts)[n // 2]

        T = 16384                      # tokens per micro-batch
        shapes = [("BERT-large qkv", T, 3072, 1024), ("BERT-large out/ffn2-dgrad", T, 1024, 1024),
                  ("BERT-large ffn1", T, 4096, 1024), ("BERT-large ffn2", T, 1024, 4096),
                  ("GPT-2 1.5B tp2 qkv", T, 2400, 1600), ("GPT-2 1.5B tp2 ffn1", T, 3200, 1600),
                  ("GPT-2 1.5B tp2 proj", T, 1600, 800), ("GPT-2 1.5B tp2 ffn2", T, 1600, 3200),
                  ("Llama-7B tp4 qkv", T, 3072, 4096), ("Llama-7B tp4 gate/up", T, 2752, 4096),
                  ("Llama-7B tp4 o", T, 4096, 1024), ("Llama-7B tp4 down", T, 4096, 2752),
                  ("square", 8192, 8192, 8192)]
        print("| GEMM | M x N x K | fprop ours / cuBLAS (ms) | ratio | wgrad ours / cuBLAS (ms) | ratio |")
        print("|---|---|---|---|---|---|")
        for name, M, N, K in shapes:
            a = torch.randn(M, K, device=dev, dtype=bf)
            w = torch.randn(N, K, device=dev, dtype=bf) * 0.02
            dy = torch.randn(M, N, device=dev, dtype=bf)
            dw = torch.zeros(N, K, device=dev)
            t_f = med(lambda: G.gemm(a, w))
            c_f = med(lambda: torch.matmul(a, w.t()))
            t_w = med(lambda: G.gemm(dy, a, a_mn=True, b_mn=True, out=dw, accumulate=True))
            c_w = med(lambda: torch.matmul(dy.t(), a))           # bf16 output, no accumulation: a lower bound
            print("| %s | %d x %d x %d | %.4f / %.4f | %.2f | %.4f / %.4f | %.2f |"
                  % (name, M, N, K, t_f, c_f, t_f / c_f, t_w, c_w, t_w / c_w), flush=True)
    elif o.case == "wgrad":
        M, N, K = 16384, 4096, 1024           # dW[N,K] += dY[M,N]^T X[M,K]
        dy = torch.randn(M, N, device=dev, dtype=bf)
        x = torch.randn(M, K, device=dev, dtype=bf)
        dw = torch.zeros(N, K, device=dev)
        ms = _time(lambda: G.gemm(dy, x, a_mn=True, b_mn=True, out=dw, accumulate=True), it)
        print("wgrad %dx%dx%d: %.3f ms  %.1f TFLOP/s" % (N, K, M, ms, 2.0 * M * N * K / ms / 1e9))
    elif o.case in ("attn_fwd", "attn_bwd"):
        from merak_b200.ops.attention import flash_attention
        B, H, L, D = 32, 16, 512, 64
        q, k, v = (torch.randn(B, L, H, D, device=dev, dtype=bf, requires_grad=True) for _ in range(3))
        fl = 4.0 * B * H * L * L * D
        if o.case == "attn_fwd":
            with torch.no_grad():
                ms = _time(lambda: flash_attention(q, k, v, causal=False), it)
            print("attn_fwd B%d H%d L%d D%d: %.3f ms  %.1f TFLOP/s" % (B, H, L, D, ms, fl / ms / 1e9))
        else:
            out = flash_attention(q, k, v, causal=False)
            do = torch.randn_like(out)
            ms = _time(lambda: torch.autograd.grad(out, (q, k, v), do, retain_graph=True), it)
            print("attn_bwd B%d H%d L%d D%d: %.3f ms  %.1f TFLOP/s" % (B, H, L, D, ms, 2.5 * fl / ms / 1e9))
    elif o.case == "norm":
        from merak_b200.ops.norm import fused_norm
        M, H = 65536, 1024
        x = torch.randn(M, H, device=dev, dtype=bf, requires_grad=True)
        res = torch.randn(M, H, device=dev, dtype=bf)
        g = torch.ones(H, device=dev, dtype=bf, requires_grad=True)
        b = torch.zeros(H, device=dev, dtype=bf, requires_grad=True)
        with torch.no_grad():
            ms = _time(lambda: fused_norm(x, g, b, residual=res), it)
        print("norm_fwd %dx%d (+residual): %.3f ms  %.0f GB/s" % (M, H, ms, 4 * M * H * 2 / ms / 1e6))
        y, z = fused_norm(x, g, b, residual=res)
        dy = torch.randn_like(y)
        ms = _time(lambda: torch.autograd.grad(y, (x, g, b), dy, retain_graph=True), it)
        print("norm_bwd %dx%d: %.3f ms  %.0f GB/s" % (M, H, ms, 3 * M * H * 2 / ms / 1e6))
    elif o.case in ("adamw", "dp_step"):
        n = 1 << 26                                   # 64M parameters: 256 MB of fp32 gradients
        grad = torch.randn(n, device=dev) * 0.01
        model = torch.zeros(n, dtype=bf, device=dev)
        master, m, v = torch.randn(n, device=dev), torch.zeros(n, device=dev), torch.zeros(n, device=dev)
        ctrl = torch.zeros(lib.mrk_symm_ctrl_bytes(), dtype=torch.uint8, device=dev)
        hp = torch.tensor([1e-4, 0.9, 0.999, 1e-8, 0.01, 0.1, 0.001], device=dev)
        norm, skip = torch.zeros(1, device=dev), torch.zeros(1, dtype=torch.int32, device=dev)
        gt, mt, ct = _table([grad.data_ptr()]), _table([model.data_ptr()]), _table([ctrl.data_ptr()])

        def step():
            st = _lib.stream_ptr()
            _lib.check(lib.mrk_dp_reduce_scatter(gt, ct, 1, 0, 0, n, None, 1, 0, 100, st), "rs")
            _lib.check(lib.mrk_dp_adamw_allgather(mt, ct, 1, 0, 0, n, grad.data_ptr(), master.data_ptr(),
                                                  m.data_ptr(), v.data_ptr(), None, hp.data_ptr(), 1.0, 1.0, None,
                                                  norm.data_ptr(), skip.data_ptr(), 1, 0, 1, 100, st), "ag")
        ms = _time(step, it)
        # reduce-scatter pass: read 4n, write 4n; update pass: read 16n, write 12n + 2n
        print("dp_step (1 rank) %d params: %.3f ms  %.0f GB/s" % (n, ms, 38.0 * n / ms / 1e6))
    elif o.case in ("ag_gemm", "tp_reduce"):
        n, B, seg, K, N = 2, 2, 2048, 4096, 4096
        M = B * seg * n
        ctrls = [torch.zeros(lib.mrk_symm_ctrl_bytes(), dtype=torch.uint8, device=dev) for _ in range(n)]
        ct = _table([c.data_ptr() for c in ctrls])
        if o.case == "ag_gemm":
            shards = [torch.randn(M // n, K, device=dev, dtype=bf) for _ in range(n)]
            w = torch.randn(N, K, device=dev, dtype=bf) * 0.02
            stt = _table([s.data_ptr() for s in shards])
            for c in ctrls:
                c.view(torch.int32)[4 * 16: 5 * 16] = 1 << 30      # entry barrier already satisfied
            flags = torch.zeros(M // seg, dtype=torch.int32, device=dev)
            gathered = torch.empty(M, K, dtype=bf, device=dev)
            y = torch.empty(M, N, dtype=bf, device=dev)
            calls = [0]
            Gc = 4

            def run():
                calls[0] += 1
                _lib.check(lib.mrk_gemm_bf16_ag(gathered.data_ptr(), stt, w.data_ptr(), y.data_ptr(), M, N, K, K, N,
                                                None, None, 0, 0, 0, 1.0, ct, flags.data_ptr(), Gc * calls[0], Gc, n,
                                                0, seg, 1, 200, _lib.stream_ptr()), "ag")
            ms = _time(run, it)
            print("ag_gemm (2 ranks on one GPU) %dx%dx%d: %.3f ms  %.1f TFLOP/s" % (M, N, K, ms, 2.0 * M * N * K / ms / 1e9))
        else:
            parts = [torch.randn(M, N, device=dev, dtype=bf) for _ in range(n)]
            pt = _table([p.data_ptr() for p in parts])
            out = torch.empty(M // n, N, dtype=bf, device=dev)
            ms = _time(lambda: _lib.check(lib.mrk_tp_reduce_pull(pt, ct, n, 0, out.data_ptr(), M // n, N, seg, None, 1,
                                                                 0, 50, _lib.stream_ptr()), "pull"), it)
            print("tp_reduce_pull %dx%d from %d ranks: %.3f ms  %.0f GB/s" % (M // n, N, n, ms, (n + 1) * (M // n) * N * 2 / ms / 1e6))
    elif o.case == "cross_entropy":
        from merak_b200.ops.cross_entropy import softmax_cross_entropy
        M, V = 8192, 30522
        logits = (torch.randn(M, V, device=dev, dtype=bf) * 2).requires_grad_(True)
        labels = torch.randint(0, V, (M,), device=dev)
        labels[::7] = -100

        def run():
            loss = softmax_cross_entropy(logits, labels)
            torch.autograd.grad(loss, logits)
        ms = _time(run, it)
        # forward reads the logits once, backward reads them again and writes the gradient
        print("cross_entropy fwd+bwd %dx%d: %.3f ms  %.0f GB/s" % (M, V, ms, 3.0 * M * V * 2 / ms / 1e6))
    elif o.case == "rope":
        from merak_b200.ops.elementwise import apply_rope, rope_tables
        B, L, H, D = 8, 4096, 32, 128
        x = torch.randn(B, L, H, D, device=dev, dtype=bf)
        cos, sin = rope_tables(L, D, 10000.0, dev)
        with torch.no_grad():
            ms = _time(lambda: apply_rope(x, cos, sin), it)
        print("rope B%d L%d H%d D%d: %.3f ms  %.0f GB/s" % (B, L, H, D, ms, 2.0 * x.numel() * 2 / ms / 1e6))
    elif o.case == "swiglu":
        from merak_b200.ops.elementwise import swiglu
        M, F = 16384, 11008
        gu = torch.randn(M, 2 * F, device=dev, dtype=bf, requires_grad=True)
        with torch.no_grad():
            ms = _time(lambda: swiglu(gu), it)
        print("swiglu fwd %dx%d: %.3f ms  %.0f GB/s" % (M, F, ms, 3.0 * M * F * 2 / ms / 1e6))
        y = swiglu(gu)
        dy = torch.randn_like(y)
        ms = _time(lambda: torch.autograd.grad(y, gu, dy, retain_graph=True), it)
        print("swiglu bwd %dx%d: %.3f ms  %.0f GB/s" % (M, F, ms, 5.0 * M * F * 2 / ms / 1e6))
    elif o.case == "embedding":
        from merak_b200.ops.elementwise import embedding_sum
        T, H, V = 65536, 1024, 30522
        table = torch.randn(V, H, device=dev, dtype=bf, requires_grad=True)
        ids = torch.randint(0, V, (64, T // 64), device=dev)
        with torch.no_grad():
            ms = _time(lambda: embedding_sum([ids], [table]), it)
        print("embedding fwd %d tokens x %d: %.3f ms  %.0f GB/s" % (T, H, ms, 2.0 * T * H * 2 / ms / 1e6))
        out = embedding_sum([ids], [table])
        dy = torch.randn_like(out)
        ms = _time(lambda: torch.autograd.grad(out, table, dy, retain_graph=True), it)
        print("embedding bwd %d tokens x %d: %.3f ms" % (T, H, ms))
    elif o.case == "colsum":
        from merak_b200.ops.elementwise import colsum
        M, N = 16384, 4096
        x = torch.randn(M, N, device=dev, dtype=bf)
        out = torch.zeros(N, device=dev)
        ms = _time(lambda: colsum(x, out), it)
        print("colsum %dx%d: %.3f ms  %.0f GB/s" % (M, N, ms, M * N * 2 / ms / 1e6))
    elif o.case == "moe_push":
        n, H = 2, 2048
        rows = 24576                                  # 4096 tokens x top-6 per rank
        sends = [torch.randn(rows, H, device=dev, dtype=bf) for _ in range(n)]
        recvs = [torch.empty(rows, H, device=dev, dtype=bf) for _ in range(n)]
        ctrls = [torch.zeros(lib.mrk_symm_ctrl_bytes(), dtype=torch.uint8, device=dev) for _ in range(n)]
        rt, ct = _table([r.data_ptr() for r in recvs]), _table([c.data_ptr() for c in ctrls])
        half = rows // 2
        sb = (ctypes.c_longlong * (n + 1))(0, half, rows)
        dr = (ctypes.c_longlong * n)(0, 0)             # rank 0's blocks go first in every destination
        ms = _time(lambda: _lib.check(lib.mrk_moe_alltoall_push(rt, ct, n, 0, sends[0].data_ptr(), sb, dr, H, 2, 1, 0,
                                                                50, _lib.stream_ptr()), "push"), it)
        print("moe_alltoall_push %d rows x %d (one rank, both destinations on this GPU): %.3f ms  %.0f GB/s" % (
            rows, H, ms, 2.0 * rows * H * 2 / ms / 1e6))
    else:
        raise SystemExit("unknown case " + o.case)
    torch.cuda.synchronize()
    assert _lib.status() == 0, "device status word %d" % _lib.status()


if __name__ == "__main__":
    main()
