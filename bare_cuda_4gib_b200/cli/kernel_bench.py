"""`llm-kernel-bench`: one kernel of the engine alone, timed with CUDA events, beside its roofline.

    bin/llm-kernel-bench gemm --rows 8 --out 2560 --in 2048 [--swiglu] [--partials]
    bin/llm-kernel-bench gemv --tokens 8 --out 5632 --in 2048 --form swiglu --norm
    bin/llm-kernel-bench attention --batch 8 --q-len 1 --context 2048 --heads 32 --kv-heads 4 --head-dim 64
    bin/llm-kernel-bench norm --rows 2048 --hidden 2048 --partials 1
    bin/llm-kernel-bench rope --rows 2048 --heads 32 --kv-heads 4 --head-dim 64

It plays the part of the per-kernel table of cuongvng/bare-cuda-4gib's `llm-bench --kernels`
(bench/src/bench_main.cc:208-254): time, achieved GB/s and TFLOP/s, and their fraction of the
peaks (MEASURED_PEAKS.json beside the repository's bench.py when present, else 6.65 TB/s and
1.59 PFLOP/s).  Matrix products rotate over enough copies of the weight to exceed the L2 cache, as
consecutive layers of a model do.  The same command line is what the profiles under profiles/
were captured with.
"""

from __future__ import annotations

import argparse
import json
import math
import pathlib
import sys
import types


def _peaks():
    root = pathlib.Path(__file__).resolve().parents[2]
    hbm, tf = 6650.0, 1590.0
    try:
        d = json.loads((root / "MEASURED_PEAKS.json").read_text())
        hbm, tf = float(d.get("hbm_gbs", hbm)), float(d.get("bf16_tflops", tf))
    except (OSError, ValueError):
        pass
    return hbm, tf


GRAPH = [True]   # time a CUDA graph of `iters` launches, so that host launch cost does not hide short kernels


def _time(fn, iters, warmup):
    import torch
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if GRAPH[0]:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(iters):
                fn()
        graph.replay()
        torch.cuda.synchronize()
        start.record()
        graph.replay()
        end.record()
    else:
        start.record()
        for _ in range(iters):
            fn()
        end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters * 1e3   # microseconds


def _ctx(max_rows, max_seqs=256):
    import torch
    from ..engine.step import Workspace
    class Ctx(types.SimpleNamespace):
        @property
        def stream(self):          # the current stream, which is the capture stream inside a graph capture
            return torch.cuda.current_stream().cuda_stream
    return Ctx(ws=Workspace(torch.device("cuda"), max_rows), max_rows=max_rows, max_seqs=max_seqs, pad_seqs=0,
               extras={})


def _report(name, us, bytes_moved, flops):
    hbm, tf = _peaks()
    gbs, tflops = bytes_moved / us / 1e3, flops / us / 1e6
    print(json.dumps({"kernel": name, "us": round(us, 2), "GB/s": round(gbs, 1), "hbm_frac": round(gbs / hbm, 3),
                      "TFLOP/s": round(tflops, 1), "bf16_frac": round(tflops / tf, 3)}))


def bench_gemm(a):
    import torch
    from ..kernels import gemm
    ctx = _ctx(max(a.rows, 256))
    n = 2 * a.out if a.swiglu else a.out
    weight_bytes = n * a.inner * 2
    copies = max(1, min(64, -(-a.l2_mb * (1 << 20) * 2 // weight_bytes))) if a.rows <= 256 else 1
    weights = [(torch.randn(n, a.inner, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
    plans = [gemm.plan_for(w) for w in weights]
    act = ctx.ws.get("a", (a.rows, a.inner), torch.bfloat16)
    act.copy_(torch.randn(a.rows, a.inner, device="cuda"))
    state = {"i": 0}
    out_dtype = torch.float32 if (a.partials or a.add_norm) else torch.bfloat16
    epilogue = None
    if a.add_norm:      # the product adds into a float32 residual stream and prepares the norm that reads it next
        from ..kernels import lib as K
        norm = types.SimpleNamespace(prenormable=True, tensors={"weight": torch.ones(a.out, device="cuda", dtype=torch.bfloat16)},
                                     params={"eps": 1e-5})
        epilogue = K.AddTo(torch.zeros(a.rows, a.out, device="cuda"), norm)

    def run():
        plan = plans[state["i"] % copies]
        state["i"] += 1
        gemm.run(ctx, plan, act, a.rows, out_dtype, "out", a.partials, a.swiglu, epilogue)

    us = _time(run, a.iters, a.warmup)
    gemm.check_errors()
    out_bytes = a.rows * a.out * (4 if a.partials else 2)
    if a.add_norm:
        out_bytes = a.rows * a.out * (4 + 4 + 2)      # residual read and written, prepared input written
    _report(f"gemm rows={a.rows} out={a.out} in={a.inner} swiglu={a.swiglu} add_norm={a.add_norm} copies={copies}", us,
            weight_bytes + a.rows * a.inner * 2 + out_bytes, 2.0 * a.rows * n * a.inner)


def bench_gemv(a):
    """The few-token fused product: --form plain | add | swiglu | rope (out = (heads + 2 kv heads) * head dim),
    --norm takes the input from a float32 residual stream through RMSNorm."""
    import torch
    from ..kernels import gemv
    from ..kernels import lib as K
    ctx = _ctx(max(a.tokens, 16))
    ctx.dtype = torch.bfloat16
    n = 2 * a.out if a.form == "swiglu" else a.out
    weight_bytes = n * a.inner * 2
    copies = max(1, min(64, -(-a.l2_mb * (1 << 20) * 2 // weight_bytes)))
    weights = [(torch.randn(n, a.inner, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
    residual = torch.randn(a.tokens, a.inner, device="cuda")
    norm_w = torch.ones(a.inner, device="cuda", dtype=torch.bfloat16)
    x_plain = torch.randn(a.tokens, a.inner, device="cuda").to(torch.bfloat16)
    target = torch.zeros(a.tokens, a.out, device="cuda")
    epilogue = None
    if a.form == "add":
        epilogue = K.AddTo(target)
    elif a.form == "rope":
        d, kvh = a.head_dim, a.kv_heads
        heads = a.out // d - 2 * kvh
        page, blocks = 64, 4
        elems = 2 * kvh * page * d
        storage = torch.zeros(a.tokens * blocks, elems, device="cuda", dtype=torch.bfloat16)
        table = torch.arange(a.tokens * blocks, dtype=torch.int32, device="cuda").view(a.tokens, blocks)
        view = K.CacheView(storage.data_ptr(), storage.data_ptr() + elems, table, elems, blocks, page, kvh, d, torch.bfloat16)
        pos = torch.full((a.tokens,), 100, dtype=torch.int32, device="cuda")
        seq = torch.arange(a.tokens, dtype=torch.int32, device="cuda")
        inv = (1.0 / (10000.0 ** (torch.arange(d // 2, dtype=torch.float32) * 2.0 / d))).cuda()
        q_out = torch.empty(a.tokens, heads * d, device="cuda", dtype=torch.bfloat16)
        epilogue = K.RotateAndCache(q_out, view, pos, seq, inv, heads, True)
    prenormed = None
    if a.prenormed:      # the input as the product before it would have left it (see kernels.lib.Prenormed)
        items = -(-a.inner // 16)
        prenormed = K.Prenormed(None, (residual * norm_w.float()).to(torch.bfloat16),
                                (residual.square().sum(-1) / items).repeat(items, 1).contiguous().float().new_zeros(items, 32), items)
        prenormed.sq[:, : a.tokens] = (residual.square().sum(-1) / items)[None, :]
    state = {"i": 0}

    def run():
        w = weights[state["i"] % copies]
        state["i"] += 1
        x = K.LazyNorm(ctx, residual, norm_w, 1e-5, a.tokens, None, "normed", prenormed) if a.norm else x_plain
        gemv.run(ctx, w, x, a.tokens, torch.bfloat16 if a.form == "swiglu" else torch.float32, "out",
                 a.form == "swiglu", epilogue)

    us = _time(run, a.iters, a.warmup)
    _report(f"gemv tokens={a.tokens} out={a.out} in={a.inner} form={a.form} norm={a.norm} copies={copies}", us,
            weight_bytes + a.tokens * a.inner * (4 if a.norm else 2) + a.tokens * a.out * 4, 2.0 * a.tokens * n * a.inner)


def bench_attention(a):
    import torch
    from ..kernels import attention as fast
    from ..kernels.lib import CacheView
    page = a.page
    blocks = -(-a.context // page)
    n_pages = a.batch * blocks
    elems = 2 * a.kv_heads * page * a.head_dim
    storage = (torch.randn(n_pages, elems, device="cuda") * 0.5).to(torch.bfloat16)
    table = torch.arange(n_pages, dtype=torch.int32, device="cuda").view(a.batch, blocks)
    view = CacheView(storage.data_ptr(), storage.data_ptr() + elems, table, elems, blocks, page, a.kv_heads,
                     a.head_dim, torch.bfloat16, storage.data_ptr(), storage.numel())
    rows = a.batch * a.q_len
    ctx = _ctx(max(rows, 256), max(a.batch, 8))
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    ctx.seq_q_start = i32([i * a.q_len for i in range(a.batch)])
    ctx.seq_q_len, ctx.seq_kv_len = i32([a.q_len] * a.batch), i32([a.context] * a.batch)
    ctx.token_ids = i32([0])
    ctx.host_q_len, ctx.host_kv_len = [a.q_len] * a.batch, [a.context] * a.batch
    ctx.max_q_len, ctx.max_kv_len = a.q_len, a.context
    q = torch.randn(rows, a.heads * a.head_dim, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    plan = fast.plan_for(a.head_dim, a.heads, a.kv_heads)
    scale = 1.0 / math.sqrt(a.head_dim)
    from ..kernels import gemm
    fast.run(ctx, plan, q, out, view, scale, 0)
    gemm.check_errors()          # a kernel that gave up on a wait must not be timed
    us = _time(lambda: fast.run(ctx, plan, q, out, view, scale, 0), a.iters, a.warmup)
    gemm.check_errors()
    kv_bytes = a.batch * a.context * a.kv_heads * a.head_dim * 2 * 2
    pairs = a.batch * (a.q_len * (a.context - a.q_len) + a.q_len * (a.q_len + 1) / 2)
    _report(f"attention batch={a.batch} q_len={a.q_len} context={a.context} heads={a.heads}/{a.kv_heads} d={a.head_dim}",
            us, kv_bytes + 2 * q.numel() * 2, 4.0 * a.heads * a.head_dim * pairs)


def bench_norm(a):
    import torch
    from ..kernels import lib as K
    res = torch.randn(a.rows, a.hidden, device="cuda")
    delta = torch.randn(a.partials, a.rows, a.hidden, device="cuda")
    w = torch.ones(a.hidden, device="cuda", dtype=torch.bfloat16)
    out = torch.empty(a.rows, a.hidden, device="cuda", dtype=torch.bfloat16)
    us = _time(lambda: K.add_rmsnorm(res, K.Partials(delta, a.partials), w, out, 1e-5, a.rows), a.iters, a.warmup)
    _report(f"add_rmsnorm rows={a.rows} hidden={a.hidden} partials={a.partials}", us,
            a.rows * a.hidden * (8 + 4 * a.partials + 2), 0.0)


def bench_rope(a):
    import torch
    from ..kernels import lib as K
    from ..kernels.lib import CacheView
    page, d = 64, a.head_dim
    blocks = -(-(a.rows + 1) // page)
    elems = 2 * a.kv_heads * page * d
    storage = torch.zeros(blocks, elems, device="cuda", dtype=torch.bfloat16)
    table = torch.arange(blocks, dtype=torch.int32, device="cuda").view(1, blocks)
    view = CacheView(storage.data_ptr(), storage.data_ptr() + elems, table, elems, blocks, page, a.kv_heads, d, torch.bfloat16)
    width = (a.heads + 2 * a.kv_heads) * d
    qkv = torch.randn(a.rows, width, device="cuda").to(torch.bfloat16)
    q = torch.empty(a.rows, a.heads * d, device="cuda", dtype=torch.bfloat16)
    pos = torch.arange(a.rows, dtype=torch.int32, device="cuda")
    seq = torch.zeros(a.rows, dtype=torch.int32, device="cuda")
    inv = (1.0 / (10000.0 ** (torch.arange(d // 2, dtype=torch.float32) * 2.0 / d))).cuda()
    us = _time(lambda: K.rope_cache_write(K.Partials(qkv), q, view, pos, seq, inv, a.heads, True, a.rows), a.iters, a.warmup)
    _report(f"rope_cache_write rows={a.rows} heads={a.heads}/{a.kv_heads} d={d}", us, 2 * a.rows * width * 2, 0.0)


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="llm-kernel-bench", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="kernel", required=True)
    common = argparse.ArgumentParser(add_help=False)
    common.add_argument("--iters", type=int, default=50)
    common.add_argument("--warmup", type=int, default=5)
    common.add_argument("--no-graph", action="store_true", help="time direct launches instead of one CUDA graph")
    g = sub.add_parser("gemm", parents=[common])
    g.add_argument("--rows", type=int, required=True)
    g.add_argument("--out", type=int, required=True, help="output features (per half with --swiglu)")
    g.add_argument("--in", dest="inner", type=int, required=True)
    g.add_argument("--swiglu", action="store_true")
    g.add_argument("--partials", action="store_true", help="float32 output that may be split over K")
    g.add_argument("--add-norm", action="store_true",
                   help="add into a float32 residual stream and prepare the next norm (many-token steps)")
    g.add_argument("--l2-mb", type=int, default=126)
    v = sub.add_parser("gemv", parents=[common])
    v.add_argument("--tokens", type=int, default=8)
    v.add_argument("--out", type=int, required=True, help="output features (per half with --form swiglu)")
    v.add_argument("--in", dest="inner", type=int, required=True)
    v.add_argument("--form", default="plain", choices=["plain", "add", "swiglu", "rope"])
    v.add_argument("--norm", action="store_true")
    v.add_argument("--prenormed", action="store_true", help="with --norm: the input prepared by the product before")
    v.add_argument("--kv-heads", type=int, default=4)
    v.add_argument("--head-dim", type=int, default=64)
    v.add_argument("--l2-mb", type=int, default=126)
    t = sub.add_parser("attention", parents=[common])
    for name, default in (("batch", 8), ("q-len", 1), ("context", 2048), ("heads", 32), ("kv-heads", 4),
                          ("head-dim", 64), ("page", 64)):
        t.add_argument(f"--{name}", type=int, default=default)
    n = sub.add_parser("norm", parents=[common])
    n.add_argument("--rows", type=int, default=2048)
    n.add_argument("--hidden", type=int, default=2048)
    n.add_argument("--partials", type=int, default=1)
    r = sub.add_parser("rope", parents=[common])
    for name, default in (("rows", 2048), ("heads", 32), ("kv-heads", 4), ("head-dim", 64)):
        r.add_argument(f"--{name}", type=int, default=default)
    args = ap.parse_args(argv)
    GRAPH[0] = not args.no_graph
    {"gemm": bench_gemm, "gemv": bench_gemv, "attention": bench_attention, "norm": bench_norm, "rope": bench_rope}[args.kernel](args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
