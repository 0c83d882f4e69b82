"""Times one kernel at one shape with CUDA events (the reference has the same kind of tool per kernel,
kernels/bench/gemv_bench.cu, attn_bench.cu): median / min of `reps` launches after warm-up, achieved GB/s of the
bytes the kernel has to read and TFLOP/s of its arithmetic.

    python -m infer_b200.cli.kernel_bench linear --M 8 --N 1536 --K 8960 [--kernel auto|skinny|tc|plain] [--epi none|residual|swiglu]
    python -m infer_b200.cli.kernel_bench attention --batch 8 --context 2048 --q-len 1 [--heads 12 --kv-heads 2 --head-dim 128]
    python -m infer_b200.cli.kernel_bench rmsnorm --M 8 --K 1536
    python -m infer_b200.cli.kernel_bench layer --M 8 --hidden 1536 --intermediate 8960 --qkv 2048 [--phases 1..4]

Inputs rotate over enough copies to exceed the 126 MB L2, as in the model where every layer brings its own weights;
the launches (one per copy) are captured in a CUDA graph and the replay is timed, so the number is what the kernel
costs inside a captured step, without the host's launch latency.
"""
from __future__ import annotations

import argparse
import json
import math
import sys


def _time(fn, n_variants, reps, warmup=3):
    """Captures one launch per variant into a CUDA graph and replays it: the time per launch then holds what a
    kernel costs inside a captured decode step (its duration and the gap to the next node), not the host's launch
    latency. Returns (median, min) microseconds per launch over `reps` replays."""
    import torch
    for i in range(max(warmup, 1)):
        for v in range(n_variants):
            fn(v)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for v in range(n_variants):
            fn(v)
    graph.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        e1.synchronize()
        times.append(e0.elapsed_time(e1) * 1e3 / n_variants)
    times.sort()
    return times[len(times) // 2], times[0]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("what", choices=["linear", "attention", "rmsnorm", "layer"])
    ap.add_argument("--M", type=int, default=8)
    ap.add_argument("--N", type=int, default=1536)
    ap.add_argument("--K", type=int, default=1536)
    ap.add_argument("--kernel", default="auto", choices=["auto", "skinny", "tc", "plain"])
    ap.add_argument("--epi", default="none", choices=["none", "residual", "swiglu"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--q-len", type=int, default=1)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--kv-heads", type=int, default=2)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--bn", type=int, default=0, help="tc: the tile code instead of the planner's (many tokens; 768 with --splits 2, 4 or 8: K slices as a cluster)")
    ap.add_argument("--cluster", type=int, default=0)
    ap.add_argument("--fused", action="store_true", help="attention: the decode kernel that also rotates and stores k/v")
    ap.add_argument("--norm", action="store_true", help="skinny kernel with the fused RMSNorm prologue")
    ap.add_argument("--hidden", type=int, default=1536)
    ap.add_argument("--intermediate", type=int, default=8960)
    ap.add_argument("--qkv", type=int, default=2048)
    ap.add_argument("--phases", type=int, default=4, help="layer: only the first n products")
    ap.add_argument("--reps", type=int, default=50)
    args = ap.parse_args(argv)
    import torch
    from infer_b200 import fast_ops, ops
    dev = "cuda:0"
    L2 = 256 << 20
    out = {"what": args.what}
    if args.what == "linear":
        M, N, K = args.M, args.N, args.K
        copies = max(4, min(64, L2 // (N * K * 2) + 1))
        ws = [(torch.randn(N, K, device=dev) * 0.05).bfloat16() for _ in range(copies)]
        x = torch.randn(M, K, device=dev).bfloat16()
        hx, nw = torch.randn(M, K, device=dev), torch.ones(K, device=dev)
        n_out = N // 2 if args.epi == "swiglu" else N
        res = torch.randn(M, n_out, device=dev) if args.epi == "residual" else None
        swiglu = args.epi == "swiglu"
        odt = torch.float32 if res is not None else torch.bfloat16

        plan = fast_ops.gemm_plan(M, N, K, fast_ops.device_state(dev).sm_count)
        if plan is not None and args.splits:
            tiles = -(-(N if plan[0] else M) // 128) * -(-(M if plan[0] else N) // plan[1])
            plan = (plan[0], plan[1], args.splits, args.splits * tiles * 128 * plan[1], tiles)

        if plan is not None and args.bn:
            plan = (0, args.bn, (args.splits or 2) if args.bn == 768 else 1, 0, 0)

        def run(i):
            r = res
            if args.kernel == "skinny":
                if args.norm:
                    return fast_ops.linear_skinny(hx, ws[i], None, r, odt, r, swiglu, args.cluster, nw, 1e-6)
                return fast_ops.linear_skinny(x, ws[i], None, r, odt, r, swiglu, args.cluster)
            if args.kernel == "tc":
                return fast_ops.gemm_tc(x, ws[i], None, r, odt, r, swiglu=swiglu, plan=plan)
            if args.kernel == "plain":
                return ops.linear_plain(x, ws[i], None, r, odt, r)
            return fast_ops.linear(x, ws[i], None, r, odt, r, swiglu)
        if run(0) is None:
            print(json.dumps({"error": "the kernel refuses this shape"}))
            return 1
        med, mn = _time(run, copies, args.reps)
        nbytes = N * K * 2 + M * K * 2 + M * n_out * (4 if res is not None else 2) * (2 if res is not None else 1)
        out.update(M=M, N=N, K=K, kernel=args.kernel, epi=args.epi, us_median=round(med, 2), us_min=round(mn, 2),
                   gbs=round(nbytes / med / 1e3, 1), tflops=round(2 * M * N * K / med / 1e6, 2), plan=plan)
    elif args.what == "attention":
        B, ctx, q_len, nh, nkv, hd = args.batch, args.context, args.q_len, args.heads, args.kv_heads, args.head_dim
        pages_per = -(-(ctx + q_len) // 16)
        n_layers = max(4, min(32, L2 // (B * pages_per * 16 * nkv * hd * 4) + 1))
        n_pages = B * pages_per
        ks = [torch.randn(n_pages, nkv, 16, hd, device=dev).bfloat16() for _ in range(n_layers)]
        vs = [torch.randn(n_pages, nkv, 16, hd, device=dev).bfloat16() for _ in range(n_layers)]
        table = torch.arange(n_pages, dtype=torch.int32, device=dev).view(B, pages_per).contiguous()
        q = torch.randn(B * q_len, nh * hd, device=dev).bfloat16()
        seg_start = torch.arange(0, (B + 1) * q_len, q_len, dtype=torch.int32, device=dev)
        pos0 = torch.full((B,), ctx, dtype=torch.int32, device=dev)

        qkv = torch.randn(B * q_len, (nh + 2 * nkv) * hd, device=dev).bfloat16()
        cos, sin = torch.rand(ctx + q_len + 1, hd // 2, device=dev), torch.rand(ctx + q_len + 1, hd // 2, device=dev)

        def run(i):
            if args.fused:
                return fast_ops.attention_decode_fused(qkv, cos, sin, ks[i], vs[i], table, seg_start, pos0, nh, nkv, hd, None,
                                                       1 / math.sqrt(hd), ctx + 1, True, args.splits or None)
            return fast_ops.attention_fast(q, ks[i], vs[i], table, seg_start, pos0, nh, nkv, hd, None, 1 / math.sqrt(hd),
                                           q_len == 1, q_len, ctx + q_len, B if q_len == 1 else 0, args.splits or None)
        med, mn = _time(run, n_layers, args.reps)
        nbytes = B * (ctx + q_len) * nkv * hd * 2 * 2
        flops = 4 * B * nh * hd * (q_len * ctx + q_len * (q_len + 1) / 2)
        out.update(batch=B, context=ctx, q_len=q_len, us_median=round(med, 2), us_min=round(mn, 2),
                   gbs=round(nbytes / med / 1e3, 1), tflops=round(flops / med / 1e6, 2))
    elif args.what == "layer":
        # what a decode layer does between two attention kernels: o product + residual, norm + gate/up + SwiGLU,
        # down + residual, the next layer's norm + q/k/v product with bias (the norm inside the product where the
        # streaming kernel takes it, as in the model)
        from infer_b200.parts.base import DeferredNorm
        M, H, I, Q = args.M, args.hidden, args.intermediate, args.qkv
        F = fast_ops
        per_layer = (H * H + 3 * H * I + Q * H) * 2
        copies = max(3, min(16, L2 // per_layer + 1))
        mk = lambda n, k: (torch.randn(n, k, device=dev) * 0.03).bfloat16()
        layers = [dict(wo=mk(H, H), wgu=mk(2 * I, H), wd=mk(H, I), wqkv=mk(Q, H)) for _ in range(copies)]
        g, bias = torch.ones(H, device=dev), torch.zeros(Q, device=dev)
        ctx = torch.randn(M, H, device=dev).bfloat16()
        h = torch.randn(M, H, device=dev)
        qkv = torch.empty(M, Q, dtype=torch.bfloat16, device=dev)

        class _Norm:
            weight, eps = g, 1e-6
            @staticmethod
            def forward(x):
                return ops.rmsnorm(x, g, 1e-6, torch.bfloat16)

        def run(i):
            L = layers[i]
            F.linear(ctx, L["wo"], None, h, torch.float32, h)
            if args.phases > 1:
                a = F.gate_up_swiglu(DeferredNorm(_Norm, h), L["wgu"])
            if args.phases > 2:
                F.linear(a, L["wd"], None, h, torch.float32, h)
            if args.phases > 3:
                F.linear(DeferredNorm(_Norm, h), L["wqkv"], bias, None, torch.bfloat16, qkv)
        med, mn = _time(run, copies, args.reps)
        nbytes = [H * H, H * H + 2 * I * H, H * H + 3 * I * H, per_layer // 2][args.phases - 1] * 2
        out.update(M=M, hidden=H, intermediate=I, qkv=Q, phases=args.phases,
                   us_median=round(med, 2), us_min=round(mn, 2), gbs=round(nbytes / med / 1e3, 1))
    else:
        M, K = args.M, args.K
        x = torch.randn(M, K, device=dev)
        w = torch.ones(K, device=dev)
        med, mn = _time(lambda i: ops.rmsnorm(x, w, 1e-6, torch.bfloat16), 16, args.reps)
        out.update(M=M, K=K, us_median=round(med, 2), us_min=round(mn, 2))
    st = fast_ops.device_state(dev).status.item()
    if st:
        out["status"] = st
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
