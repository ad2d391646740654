"""Times one kernel of this package alone, on synthetic inputs, and prints what it achieves.

    python -m zephyr_b200.kernels.timing decode_attention --batch 8 --context 4096
    python -m zephyr_b200.kernels.timing prefill_attention --tokens 2048
    python -m zephyr_b200.kernels.timing gemm_small --rows 8 --n 6144 --k 1024 [--swiglu]
    python -m zephyr_b200.kernels.timing fused_chain --rows 8 --hidden 1024 --ffn 3072
    python -m zephyr_b200.kernels.timing sample --rows 8 --vocab 151936
    python -m zephyr_b200.kernels.timing products --tokens 2048 --hidden 1024 --ffn 3072
    python -m zephyr_b200.kernels.timing gemm_tc --tokens 2048 --n 6144 --k 1024 [--swiglu] [--library]

Each case rotates over several copies of its large operands, together larger than the L2 cache, so
that a kernel bound by memory is timed against memory and not against L2.  Time is taken with CUDA
events around a CUDA graph of ``--iters`` launches, after ``--warmup`` plain launches.  The line printed is JSON: the
kernel, its sizes, microseconds per launch, and GB/s over the bytes the kernel has to read, or
TFLOP/s over the products it has to form.  This is also the small program that a profiler is
pointed at when one kernel is to be looked at by itself.
"""
from __future__ import annotations

import argparse
import json
import math
import sys

import torch

from . import ops

L2_BYTES = 126 << 20


def _time(run, warmup: int, iters: int) -> float:
    """Microseconds per call of ``run(i)``.  The timed calls are captured in one CUDA graph, so that
    a kernel of a few microseconds is not timed against the host's launch rate."""
    for i in range(warmup):
        run(i)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with ops.capture(graph, stream=stream):
            for i in range(iters):
                run(warmup + i)
        graph.replay()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record(stream)
        graph.replay()
        end.record(stream)
        torch.cuda.synchronize()
    return begin.elapsed_time(end) / iters * 1e3


RESIDENT = False      # --resident: one copy of every operand, so that a small one stays in L2


def _copies(bytes_each: int) -> int:
    if RESIDENT:
        return 1
    return max(2, min(16, math.ceil(2 * L2_BYTES / max(bytes_each, 1))))


SEQUENTIAL_PAGES = False      # --sequential-pages: a request's pages lie behind one another in the pool


def _paged_inputs(batch: int, context: int, nkv: int, hd: int, page: int, device):
    pages_per = math.ceil(context / page)
    num_pages = batch * pages_per + 1
    cache_bytes = num_pages * 2 * nkv * page * hd * 2
    caches = [torch.randn((num_pages, 2, nkv, page, hd), device=device, dtype=torch.bfloat16)
              for _ in range(_copies(cache_bytes))]
    order = torch.arange(num_pages - 1, device=device) if SEQUENTIAL_PAGES else torch.randperm(num_pages - 1, device=device)
    table = (order[: batch * pages_per] + 1).int().view(batch, pages_per)
    return caches, table.contiguous()


def decode_attention(args) -> dict:
    device = torch.device("cuda")
    nh, nkv, hd, B, ctx = args.heads, args.kv_heads, args.head_dim, args.batch, args.context
    caches, table = _paged_inputs(B, ctx, nkv, hd, args.page_size, device)
    q = torch.randn((B, nh * hd), device=device, dtype=torch.bfloat16)
    rows = torch.arange(B, dtype=torch.int32, device=device)
    row_ctx = torch.full((B,), ctx - 1, dtype=torch.int32, device=device)
    status, out = ops.new_status(device), torch.empty_like(q)
    split = args.split or None

    def run(i):
        ops.paged_decode(q, caches[i % len(caches)], table, rows, rows, row_ctx, ctx, nh, nkv, hd, args.window,
                         1 / math.sqrt(hd), status, out=out, split_size=split)
    us = _time(run, args.warmup, args.iters)
    trace = torch.zeros((1024, 8), dtype=torch.int32, device=device)
    ops.paged_decode_trace(trace)
    for i in range(3):          # the last launch's timeline stays
        run(i)
    ops.paged_decode_trace(None)
    ops.check_status(status, "decode_attention")
    live = min(ctx, args.window) if args.window else ctx
    read = B * live * nkv * hd * 2 * 2
    return {"kernel": "paged_decode_kernel", "batch": B, "context": ctx, "heads": nh, "kv_heads": nkv, "head_dim": hd,
            "page_size": args.page_size, "window": args.window, "split_size": split or "balanced", "us": round(us, 2),
            "bytes_read": read, "gbs": round(read / us / 1e3, 1), "timeline_ns": _decode_timeline(trace)}


def _decode_timeline(trace: torch.Tensor) -> dict:
    """The last launch over all its CTAs: when the first and the last CTA reached each mark,
    nanoseconds from the earliest start; and the fewest and most items and tiles of a CTA."""
    t = trace.cpu().to(torch.int64)
    t = t[t[:, 4] != 0]
    if t.shape[0] == 0:
        return {}
    marks = ("start", "earlier_kernels_done", "first_tile_landed", "last_tile_done", "end")
    rel = (t[:, :5] - t[:, 0].min()) & 0xFFFFFFFF
    out = {m: [int(rel[:, i].min()), int(rel[:, i].max())] for i, m in enumerate(marks)}
    counted = t[t[:, 7] != 0]
    if counted.shape[0]:
        arrival = (counted[:, 7] - t[:, 0].min()) & 0xFFFFFFFF
        out["last_arrival_counted"] = [int(arrival.min()), int(arrival.max())]
    out.update(ctas=int(t.shape[0]), items=[int(t[:, 5].min()), int(t[:, 5].max())],
               tiles=[int(t[:, 6].min()), int(t[:, 6].max())])
    return out


def prefill_attention(args) -> dict:
    device = torch.device("cuda")
    nh, nkv, hd, T = args.heads, args.kv_heads, args.head_dim, args.tokens
    caches, table = _paged_inputs(1, T, nkv, hd, args.page_size, device)
    q = torch.randn((T, nh * hd), device=device, dtype=torch.bfloat16)
    tile = ops.paged_prefill_tile_tokens()
    n_tiles = math.ceil(T / tile)
    tile_row = torch.zeros(n_tiles, dtype=torch.int32, device=device)
    tile_q0 = (torch.arange(n_tiles, dtype=torch.int32, device=device) * tile).contiguous()
    zero = torch.zeros(1, dtype=torch.int32, device=device)
    q_len = torch.full((1,), T, dtype=torch.int32, device=device)
    status, out = ops.new_status(device), torch.empty_like(q)

    def run(i):
        ops.paged_prefill(q, caches[i % len(caches)], table, tile_row, tile_q0, zero, q_len, zero, nh, nkv, hd,
                          args.window, 1 / math.sqrt(hd), status, out=out)
    us = _time(run, args.warmup, args.iters)
    trace = torch.zeros((2, 64, 4), dtype=torch.int32, device=device)
    ops.paged_prefill_trace(trace)
    for i in range(2):
        run(i)
    ops.paged_prefill_trace(None)
    ops.check_status(status, "prefill_attention")
    # Two products of 2 * hd flops per (query, visible key) pair and head.
    pairs = sum(min(t + 1, args.window) if args.window else t + 1 for t in range(T))
    flops = 4 * hd * pairs * nh
    return {"kernel": "paged_prefill_kernel", "tokens": T, "heads": nh, "kv_heads": nkv, "head_dim": hd,
            "page_size": args.page_size, "window": args.window, "us": round(us, 2), "flops": flops,
            "tflops": round(flops / us / 1e6, 1), "longest_cta_ns": _prefill_timeline(trace)}


def _prefill_timeline(trace: torch.Tensor) -> list:
    """The launch's longest CTA, tile by tile: [S issued, softmax began, probabilities written,
    O += P V issued, keys asked for, values asked for], ns from the first mark.  Empty if the kernel
    that ran keeps no timeline."""
    t = trace.cpu().to(torch.int64)
    n = int((t[0, :, 3] != 0).sum())
    if n == 0:
        return []
    base = min(int(t[0, 0, 0]), int(t[1, 0, 0]))
    both = torch.cat([t[0, :n], t[1, :n, :2]], dim=1)
    return ((both - base) & 0xFFFFFFFF).tolist()


def gemm_small(args) -> dict:
    device = torch.device("cuda")
    M, N, K = args.rows, args.n, args.k
    weights = [torch.randn((N, K), device=device, dtype=torch.bfloat16) for _ in range(_copies(N * K * 2))]
    x = torch.randn((M, K), device=device, dtype=torch.bfloat16)
    out_dtype = torch.float32 if args.float_out else torch.bfloat16

    def run(i):
        ops.gemm_small(x, weights[i % len(weights)], out_dtype=out_dtype, swiglu=args.swiglu)
    us = _time(run, args.warmup, args.iters)
    read = N * K * 2
    return {"kernel": "gemm_small_kernel", "rows": M, "n": N, "k": K, "swiglu": bool(args.swiglu),
            "out": str(out_dtype).replace("torch.", ""), "us": round(us, 2), "bytes_read": read,
            "gbs": round(read / us / 1e3, 1)}


def sample(args) -> dict:
    device = torch.device("cuda")
    R, V = args.rows, args.vocab
    logits = [torch.randn((R, V), device=device, dtype=torch.float32) * args.logit_scale for _ in range(_copies(R * V * 4))]
    rows = None
    if args.temperature >= 1e-7 or args.top_logprobs >= 0:
        rows = [ops.SampleRow(temperature=args.temperature, uniform=0.1 + 0.8 * r / R, top_k=args.top_k,
                              top_p=args.top_p, min_p=args.min_p, num_logprobs=args.top_logprobs) for r in range(R)]
    status = ops.new_status(device)

    def run(i):
        ops.sample_rows(logits[i % len(logits)], rows, status)
    us = _time(run, args.warmup, args.iters)
    ops.check_status(status, "sample")
    state = ops.last_sample_job_state()
    return {"kernel": "sample kernels", "rows": R, "vocab": V, "temperature": args.temperature, "top_k": args.top_k,
            "top_p": args.top_p, "min_p": args.min_p, "top_logprobs": args.top_logprobs, "logit_scale": args.logit_scale,
            "rankings": len(state), "rankings_decided_in_the_head": sum(done for _, done in state), "us": round(us, 2)}


def _chain_timeline(trace: torch.Tensor) -> dict:
    """The last launch's stages over all CTAs: when the first and the last CTA reached each mark
    (start, input in place, products done, barrier passed), nanoseconds from the earliest start."""
    t = trace.cpu().to(torch.int64)
    t = (t - t[:, 0, 0].min()) & 0xFFFFFFFF
    marks = ("start", "input", "products", "barrier")
    return {f"stage{s}": {m: [int(t[:, s, i].min()), int(t[:, s, i].max())] for i, m in enumerate(marks)}
            for s in range(t.shape[1])}


def fused_chain(args) -> dict:
    """A layer's tail as one chain: output projection, add + norm + gate/up + silu * up, down
    projection, add + norm + the next layer's input projection."""
    device = torch.device("cuda")
    M, d, q, ffn, qkv = args.rows, args.hidden, args.heads * args.head_dim, args.ffn, (args.heads + 2 * args.kv_heads) * args.head_dim
    layer_bytes = 2 * (d * q + 2 * ffn * d + d * ffn + qkv * d)
    rnd = lambda *shape: torch.randn(shape, device=device, dtype=torch.bfloat16) * 0.05
    layers = [(rnd(d, q), rnd(2 * ffn, d), rnd(d, ffn), rnd(qkv, d)) for _ in range(_copies(layer_bytes))]
    norm = torch.ones(d, device=device, dtype=torch.bfloat16)
    attn, residual = rnd(M, q), rnd(M, d)
    buf = lambda n: torch.empty((M, n), device=device, dtype=torch.bfloat16)
    o, act, down, out, r1, r2 = buf(d), buf(ffn), buf(d), buf(qkv), buf(d), buf(d)
    status = ops.new_status(device)
    trace = torch.zeros((ops.fused_chain_grid(), 4, 4), dtype=torch.int32, device=device)

    def stages(i):
        w_o, w_gu, w_down, w_qkv = layers[i % len(layers)]
        return [ops.ChainStage(w=w_o, y=o, x=attn),
                ops.ChainStage(w=w_gu, y=act, residual_in=residual, residual_out=r1, delta=o, norm_w=norm, eps=1e-6, swiglu=True),
                ops.ChainStage(w=w_down, y=down, x=act),
                ops.ChainStage(w=w_qkv, y=out, residual_in=r1, residual_out=r2, delta=down, norm_w=norm, eps=1e-6)]

    whole = all(ops.fused_chain_stage_supported(M, st.w, st.norm_w is not None, st.swiglu) for st in stages(0))
    if whole:
        def run(i):
            ops.fused_chain(stages(i), M, status, trace=trace)
    else:
        # A stage whose input does not fit in shared memory (the down projection of a wide model) runs as
        # kernels of its own between two shorter chains, as in a model's step.
        from ..parts.fused import run_stages

        def run(i):
            run_stages(stages(i), M, status)
    us = _time(run, args.warmup, args.iters)
    ops.check_status(status, "fused_chain")
    return {"kernel": "fused_chain_kernel" if whole else "fused_chain_kernel + gemm_small_kernel", "rows": M, "hidden": d,
            "q": q, "ffn": ffn, "qkv": qkv, "us": round(us, 2), "bytes_read": layer_bytes,
            "gbs": round(layer_bytes / us / 1e3, 1), "timeline_ns": _chain_timeline(trace) if whole else {}}


def products(args) -> dict:
    """A layer's four matrix products for a prompt portion of ``--tokens`` tokens, as the engine runs
    them: the vendor library's tensor-core product for bfloat16 beyond 16 rows, and for gate/up, from
    ``ops.GEMM_TC_MIN_ROWS`` rows on, this package's tcgen05 product with the activation in its epilogue."""
    device = torch.device("cuda")
    T, d, q, ffn, qkv = args.tokens, args.hidden, args.heads * args.head_dim, args.ffn, (args.heads + 2 * args.kv_heads) * args.head_dim
    layer_bytes = 2 * (d * q + 2 * ffn * d + d * ffn + qkv * d)
    rnd = lambda *shape: torch.randn(shape, device=device, dtype=torch.bfloat16) * 0.05
    layers = [(rnd(qkv, d), rnd(d, q), rnd(2 * ffn, d), rnd(d, ffn)) for _ in range(_copies(layer_bytes))]
    x, attn, act = rnd(T, d), rnd(T, q), rnd(T, ffn)

    def run(i):
        w_qkv, w_o, w_gu, w_down = layers[i % len(layers)]
        ops.linear(x, w_qkv)
        ops.linear(attn, w_o)
        if (T >= ops.GEMM_TC_MIN_ROWS or not ops.USE_LIBRARY_PRODUCTS) and ops.gemm_tc_supported(x, w_gu, swiglu=True):
            ops.gemm_tc(x, w_gu, swiglu=True)
        else:
            ops.silu_mul(ops.linear(x, w_gu), blocked=True)
        ops.linear(act, w_down)
    us = _time(run, args.warmup, args.iters)
    flops = 2.0 * T * (qkv * d + d * q + 2 * ffn * d + d * ffn)
    return {"kernel": "a layer's prompt products (cuBLASLt; gate/up + activation on tcgen05)", "tokens": T, "hidden": d, "q": q, "ffn": ffn, "qkv": qkv,
            "us": round(us, 2), "flops": flops, "tflops": round(flops / us / 1e6, 1)}


def gemm_tc(args) -> dict:
    """One product x [tokens, k] w[n, k]^T on this package's tcgen05 kernel (``--swiglu``: with the
    activation in its epilogue; ``--library``: the vendor library's product, and the activation
    kernel after it, on the same operands)."""
    device = torch.device("cuda")
    T, N, K = args.tokens, args.n, args.k
    rnd = lambda *shape: torch.randn(shape, device=device, dtype=torch.bfloat16) * 0.05
    weights = [rnd(N, K) for _ in range(_copies(2 * N * K))]
    x = rnd(T, K)
    status = torch.zeros(4, dtype=torch.int32, device=device)

    def run(i):
        w = weights[i % len(weights)]
        if args.library:
            y = ops.linear(x, w)
            if args.swiglu:
                ops.silu_mul(y, blocked=True)
        else:
            ops.gemm_tc(x, w, swiglu=args.swiglu, block_n=args.block_n, status=status)
    us = _time(run, args.warmup, args.iters)
    flops = 2.0 * T * N * K
    return {"kernel": "library product" if args.library else "gemm_tc_kernel", "tokens": T, "n": N, "k": K,
            "swiglu": args.swiglu, "block_n": args.block_n, "us": round(us, 2), "flops": flops,
            "tflops": round(flops / us / 1e6, 1), "status": status.tolist()}


CASES = {"gemm_tc": gemm_tc, "fused_chain": fused_chain, "products": products, "decode_attention": decode_attention, "prefill_attention": prefill_attention, "gemm_small": gemm_small,
         "sample": sample}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="python -m zephyr_b200.kernels.timing", description=__doc__.split("\n")[0])
    parser.add_argument("case", choices=sorted(CASES))
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--iters", type=int, default=40)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=4096)
    parser.add_argument("--tokens", type=int, default=2048)
    parser.add_argument("--heads", type=int, default=16)
    parser.add_argument("--kv-heads", type=int, default=8)
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--page-size", type=int, default=16)
    parser.add_argument("--window", type=int, default=0)
    parser.add_argument("--split", type=int, default=0, help="fixed splits of this many positions in the decode kernel (0: balanced items)")
    parser.add_argument("--rows", type=int, default=8)
    parser.add_argument("--n", type=int, default=6144)
    parser.add_argument("--k", type=int, default=1024)
    parser.add_argument("--hidden", type=int, default=1024)
    parser.add_argument("--ffn", type=int, default=3072)
    parser.add_argument("--swiglu", action="store_true")
    parser.add_argument("--float-out", action="store_true")
    parser.add_argument("--vocab", type=int, default=151936)
    parser.add_argument("--temperature", type=float, default=0.0)
    parser.add_argument("--top-k", type=int, default=0)
    parser.add_argument("--top-p", type=float, default=0.0)
    parser.add_argument("--min-p", type=float, default=0.0)
    parser.add_argument("--top-logprobs", type=int, default=-1)
    parser.add_argument("--logit-scale", type=float, default=1.0, help="the logits are normal draws times this")
    parser.add_argument("--sequential-pages", action="store_true",
                        help="block tables that walk the pool in order instead of a random permutation")
    parser.add_argument("--legacy-prefill", action="store_true", help="prompt attention on mma.sync even where tcgen05 applies")
    parser.add_argument("--library", action="store_true", help="gemm_tc: time the vendor library's product instead")
    parser.add_argument("--own-products", action="store_true", help="products: none of them on the vendor library")
    parser.add_argument("--block-n", type=int, default=0, help="gemm_tc: width of an output tile (256, 128; 0: chosen)")
    parser.add_argument("--resident", action="store_true",
                        help="do not rotate operands: what fits in L2 is read from L2")
    args = parser.parse_args(argv)
    global RESIDENT, SEQUENTIAL_PAGES
    RESIDENT, SEQUENTIAL_PAGES = args.resident, args.sequential_pages
    ops.USE_TCGEN05_PREFILL = not args.legacy_prefill
    ops.USE_LIBRARY_PRODUCTS = not args.own_products
    if not torch.cuda.is_available():
        print("a CUDA device is needed", file=sys.stderr)
        return 2
    print(json.dumps(CASES[args.case](args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
