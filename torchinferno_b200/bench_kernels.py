"""Time single kernels of the engine in isolation and relate them to the B200's measured peaks.

    python -m torchinferno_b200.bench_kernels decode-attention --batch 8 --context 2048
    python -m torchinferno_b200.bench_kernels prefill-attention --tokens 2048
    python -m torchinferno_b200.bench_kernels gemm --rows 8
    python -m torchinferno_b200.bench_kernels elementwise --rows 2048
    python -m torchinferno_b200.bench_kernels step-timeline --layers 32 --batch 8 --context 3072
    python -m torchinferno_b200.bench_kernels latent-attention --tokens 2048 --batch 8 --context 2048
    python -m torchinferno_b200.bench_kernels linear-attention --tokens 2048 --batch 8
    python -m torchinferno_b200.bench_kernels expert-product --tokens 2048
    python -m torchinferno_b200.bench_kernels sigmoid-attention --tokens 2048 --batch 8 --context 2048 --chunk 512
    python -m torchinferno_b200.bench_kernels gated-recurrence --tokens 2048 --batch 8
    python -m torchinferno_b200.bench_kernels layer-tails --rows 2048
    python -m torchinferno_b200.bench_kernels pooled-window-attention --tokens 2048 --batch 8 --context 2048 --window 512 --pool 64
    python -m torchinferno_b200.bench_kernels state-space --tokens 2048 --batch 8

Each run prints one JSON line per case: microseconds (median of CUDA-event timings, an L2 flush
between iterations), the bytes or flops the kernel has to move or do, and the fraction of the
measured copy bandwidth or tensor throughput (``MEASURED_PEAKS.json`` at the repository root when
present).  The same commands, small, are what the ``ncu`` summaries under ``profiles/`` were taken
from.  The reference keeps such microbenchmarks as stand-alone scripts (``scripts/`` in its tree).
"""
from __future__ import annotations

import argparse
import json
import math
import statistics
from pathlib import Path

import torch

from torchinferno_b200.kernels import ops

ROOT = Path(__file__).resolve().parent.parent


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        return {"hbm_gbs": data["hbm_gbs"], "bf16_tflops": data["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class Timer:
    def __init__(self, iters: int, warmup: int = 3) -> None:
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")   # larger than the 126 MB L2

    def __call__(self, fn) -> float:
        for _ in range(self.warmup):
            fn()
        times = []
        for _ in range(self.iters):
            self.flush.zero_()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            fn()
            end.record()
            torch.cuda.synchronize()
            times.append(begin.elapsed_time(end) * 1e3)
        return statistics.median(times)


def report(name: str, us: float, *, bytes_moved: float | None = None, flops: float | None = None, **extra) -> None:
    p = peaks()
    line = {"kernel": name, "us": round(us, 2), **extra}
    if bytes_moved is not None:
        line["gbs"] = round(bytes_moved / us / 1e3, 1)
        line["hbm_frac"] = round(bytes_moved / us / 1e3 / p["hbm_gbs"], 4)
    if flops is not None:
        line["tflops"] = round(flops / us / 1e6, 1)
        line["tensor_frac"] = round(flops / us / 1e6 / p["bf16_tflops"], 4)
    line["peaks"] = p["source"]
    print(json.dumps(line), flush=True)


def paged_cache(batch: int, context: int, kv_heads: int, head_dim: int, page: int):
    """A filled pool with shuffled pages and the block table of ``batch`` requests of ``context`` tokens."""
    pages_per = -(-context // page)
    total = batch * pages_per
    pool = (torch.randn(total, 2, kv_heads, page, head_dim, device="cuda") * 0.5).to(torch.bfloat16)
    order = torch.randperm(total, device="cuda", dtype=torch.int32)
    table = order.view(batch, pages_per).contiguous()
    return pool, table


def run_decode_attention(args) -> None:
    h, k, d = args.heads, args.kv_heads, args.head_dim
    pool, table = paged_cache(args.batch, args.context, k, d, args.page_size)
    n = args.batch
    q = torch.randn(n, h * d, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    q_start, kv_start, slots = i32(list(range(n + 1))), i32([args.context - 1] * n), i32(list(range(n)))
    timer = Timer(args.iters)
    kv_bytes = n * args.context * 2 * k * d * 2
    kernels = ["cp_async"] + (["tma"] if ops.decode_attention_tma_supports(d, h // k, args.page_size) else [])
    for forced in (args.splits or [None]):
        splits, chunk = (ops.decode_num_splits(n, h, k, args.context) if forced is None else forced), 0
        scratch = torch.empty(n * h * splits * (d + 2), dtype=torch.float32, device="cuda")
        for kernel in kernels:
            fn = lambda: ops.decode_attention(q, pool, out, q_start, kv_start, slots, table, n, h, k, d, 1 / math.sqrt(d),
                                              args.context, scratch=scratch, num_splits=splits, chunk=chunk, kernel=kernel)
            report(f"decode_attention[{kernel}]+merge", timer(fn), bytes_moved=kv_bytes, batch=n, context=args.context,
                   splits=splits, heads=h, kv_heads=k, head_dim=d)
        if "tma" in kernels:      # the same from the unrotated rows of the qkv product: rotary and the cache write inside
            qkv = torch.randn(n, (h + 2 * k) * d, device="cuda").to(torch.bfloat16)
            inv_freq = (1.0 / (500000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).cuda()
            fn = lambda: ops.decode_attention_rope(qkv, pool, out, q_start, kv_start, slots, table, n, h, k, d, 1 / math.sqrt(d),
                                                   args.context, inv_freq, scratch=scratch, num_splits=splits)
            report("decode_attention[tma, rotates and stores the newest token]+merge", timer(fn), bytes_moved=kv_bytes, batch=n,
                   context=args.context, splits=splits, heads=h, kv_heads=k, head_dim=d)


def run_prefill_attention(args) -> None:
    h, k, d, t = args.heads, args.kv_heads, args.head_dim, args.tokens
    pool, table = paged_cache(args.batch, t, k, d, args.page_size)
    n = args.batch
    q = torch.randn(n * t, h * d, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    q_start, kv_start, slots = i32([i * t for i in range(n + 1)]), i32([0] * n), i32(list(range(n)))
    fn = lambda: ops.prefill_attention(q, pool, out, q_start, kv_start, slots, table, n, t, h, k, d, 1 / math.sqrt(d))
    flops = n * 4 * h * d * t * (t + 1) / 2
    timer = Timer(args.iters)
    report("prefill_attention[mma.sync]", timer(fn), flops=flops, batch=n, tokens=t, heads=h, kv_heads=k, head_dim=d,
           note="causal flops")
    if ops.prefill_attention_tcgen05_supports(d, h // k, args.page_size):
        fn5 = lambda: ops.prefill_attention_tcgen05(q, pool, out, q_start, kv_start, slots, table, n, t, h, k, d, 1 / math.sqrt(d))
        report("prefill_attention[tcgen05]", timer(fn5), flops=flops, batch=n, tokens=t, heads=h, kv_heads=k, head_dim=d,
               note="causal flops")


def run_gemm(args) -> None:
    shapes = {"qkv": (6144, 4096), "o": (4096, 4096), "gate_up": (28672, 4096), "down": (4096, 14336), "lm_head": (128256, 4096)}
    timer = Timer(args.iters)
    for name, (n, k) in shapes.items():
        if args.only and name not in args.only:
            continue
        w = (torch.randn(n, k, device="cuda") * 0.02).to(torch.bfloat16)
        x = torch.randn(args.rows, k, device="cuda").to(torch.bfloat16)
        out = torch.empty(args.rows, n, dtype=torch.bfloat16, device="cuda")
        common = dict(bytes_moved=n * k * 2, flops=2 * args.rows * n * k, rows=args.rows, n=n, k=k)
        if ops.gemm_tcgen05_swapab_supports(args.rows, n, k):
            report(f"gemm_tcgen05_swapab[{name}]", timer(lambda: ops.gemm_tcgen05_swapab(x, w, out)), **common)
            w_kn = w.t().contiguous()
            for features, splits in ((256, 1), (128, 1), (128, 2), (128, 4), (128, 5)):      # the few-rows kernel's tiles
                if args.decode_config and (features, splits) != tuple(args.decode_config):
                    continue
                if ops.gemm_decode_supports(args.rows, n, k, features, splits):
                    report(f"gemm_decode[{name}, {features} features, K over {splits}]",
                           timer(lambda: ops.gemm_decode(x, w_kn, out, features=features, splits=splits)), **common)
            if name == "gate_up":      # (the columns stand for interleaved gate / up pairs: the activation in the epilogue)
                act = torch.empty(args.rows, n // 2, dtype=torch.bfloat16, device="cuda")
                for features in (256, 128):
                    if args.decode_config and features != args.decode_config[0]:
                        continue
                    report(f"gemm_decode[{name}, {features} features, SwiGLU epilogue]",
                           timer(lambda: ops.gemm_decode(x, w_kn, act, features=features, splits=1, epilogue=ops.DG_SWIGLU)), **common)
            report(f"gemm_tcgen05_swapab_kn[{name}]", timer(lambda: ops.gemm_tcgen05_swapab(x, w_kn, out, w_kn=True)), **common)
            report(f"library_gemm_kn[{name}]", timer(lambda: torch.mm(x, w_kn, out=out)), **common)
            del w_kn
        elif ops.gemm_tcgen05_supports(args.rows, n, k):
            report(f"gemm_tcgen05[{name}]", timer(lambda: ops.gemm_tcgen05(x, w, out)), **common)
            if args.rows >= 128 and ops.gemm_tcgen05_2cta_supports(args.rows, n, k):
                report(f"gemm_tcgen05_2cta[{name}]", timer(lambda: ops.gemm_tcgen05_2cta(x, w, out)), **common)
        report(f"library_gemm[{name}]", timer(lambda: torch.mm(x, w.t(), out=out)), **common)


def run_elementwise(args) -> None:
    rows, hidden, inter = args.rows, args.hidden, args.intermediate
    timer = Timer(args.iters)
    delta = torch.randn(rows, hidden, device="cuda").to(torch.bfloat16)
    residual = torch.randn(rows, hidden, device="cuda")
    weight = torch.ones(hidden, device="cuda")
    out = torch.empty_like(delta)
    report("add_rmsnorm", timer(lambda: ops.add_rmsnorm(delta, residual, weight, 1e-5, out)),
           bytes_moved=rows * hidden * (2 + 4 + 4 + 2), rows=rows, hidden=hidden)
    gate_up = torch.randn(rows, 2 * inter, device="cuda").to(torch.bfloat16)
    act = torch.empty(rows, inter, dtype=torch.bfloat16, device="cuda")
    report("swiglu", timer(lambda: ops.swiglu(gate_up, act)), bytes_moved=rows * inter * 6, rows=rows, intermediate=inter)
    h, k, d = args.heads, args.kv_heads, args.head_dim
    qkv = torch.randn(rows, (h + 2 * k) * d, device="cuda").to(torch.bfloat16)
    q_out = torch.empty(rows, h * d, dtype=torch.bfloat16, device="cuda")
    pool, table = paged_cache(1, rows, k, d, args.page_size)
    positions = torch.arange(rows, dtype=torch.int32, device="cuda")
    slot = torch.zeros(rows, dtype=torch.int32, device="cuda")
    inv_freq = (1.0 / (500000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).cuda()
    report("rope_append", timer(lambda: ops.rope_append(qkv, q_out, pool, positions, slot, table, inv_freq, h, k, d)),
           bytes_moved=rows * ((h + 2 * k) * d * 2 + (h + 2 * k) * d * 2), rows=rows)


def run_step_timeline(args) -> None:
    """Which kernels a captured decode step (or, with --prompt, the step of one whole prompt of --context tokens)
    spends its time in: every kernel of one step with its start and duration as the driver's activity records
    (CUPTI, through torch.profiler) give them, summed by kernel, and one layer listed launch by launch (a
    negative gap: the kernel was placed before the one before it had ended, by programmatic dependent launch,
    and its duration includes the wait)."""
    import collections
    from torch.profiler import ProfilerActivity, profile
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.engine.factory import make_runner, random_model
    from torchinferno_b200.kernels import gemm
    gemm.set_backend(args.gemm_backend)
    config = {"architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": args.vocab, "hidden_size": args.hidden,
              "intermediate_size": args.intermediate, "num_hidden_layers": args.layers, "num_attention_heads": args.heads,
              "num_key_value_heads": args.kv_heads, "head_dim": args.head_dim, "max_position_embeddings": 131072,
              "rope_theta": 500000.0, "rms_norm_eps": 1e-5, "tie_word_embeddings": False}
    model = random_model(config, seed=0, dtype="bfloat16")
    n, ctx = args.batch, args.context
    prompts = torch.randint(0, args.vocab, (n, ctx), generator=torch.Generator().manual_seed(0)).tolist()
    if args.prompt:
        runner = make_runner(model, page_size=args.page_size, max_tokens=2 * (ctx + 64), max_requests=2, check_errors=False)
        turn = [0]

        def step() -> None:      # a new request's whole prompt, alone in its step
            turn[0] += 1
            runner.step([StepEntry(turn[0], prompts[0], [ctx - 1])])
            runner.end([turn[0]])
    else:
        runner = make_runner(model, page_size=args.page_size, max_tokens=n * (ctx + 64), max_requests=n, check_errors=False)
        for i, prompt in enumerate(prompts):
            runner.step([StepEntry(i, prompt, [ctx - 1])])
        step = lambda: runner.step([StepEntry(i, [5], [0]) for i in range(n)])
    for _ in range(5):
        step()
    torch.cuda.synchronize()
    if args.plain:           # (for a launch list under ncu: no second profiler in the process)
        for _ in range(args.iters):
            step()
        torch.cuda.synchronize()
        print(json.dumps({"steps": args.iters, "batch": n, "context": ctx, "layers": args.layers}))
        return
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for _ in range(3):
            step()
        torch.cuda.synchronize()
    kernels = sorted((e for e in prof.events() if e.device_type == torch.autograd.DeviceType.CUDA and e.time_range.end > e.time_range.start),
                     key=lambda e: e.time_range.start)
    last = kernels[-(len(kernels) // 3):]
    t0, t1 = last[0].time_range.start, max(e.time_range.end for e in last)
    total = collections.defaultdict(lambda: [0, 0.0])
    for e in last:
        total[e.name[:64]][0] += 1
        total[e.name[:64]][1] += e.time_range.end - e.time_range.start
    print(json.dumps({"step_us": round(t1 - t0, 1), "kernels": len(last), "step": "prompt" if args.prompt else "decode",
                      "batch": 1 if args.prompt else n, "context": ctx, "layers": args.layers, "gemm_backend": args.gemm_backend}))
    for name, (count, us) in sorted(total.items(), key=lambda kv: -kv[1][1]):
        print(f"{us:9.1f} us  x{count:4d}  avg {us / count:7.2f}  {name}")
    print("one layer, launch by launch (gap to the end of the kernel before, duration):")
    per_layer = max(1, (len(last) - 3) // max(1, args.layers))
    mid = len(last) // 2
    end = None
    for e in last[mid:mid + per_layer + 2]:
        gap = 0.0 if end is None else e.time_range.start - end
        print(f"  gap {gap:7.2f}  dur {e.time_range.end - e.time_range.start:7.2f}  {e.name[:70]}")
        end = e.time_range.end


def run_latent_attention(args) -> None:
    """The latent attention kernel on a prompt of --tokens (flops: folded scores over rank + rot and values over rank, causal)
    and on --batch single tokens at --context (bytes: the latent rows of every context once)."""
    h, c, r, page = args.heads, args.rank, args.rot, args.page_size
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
    timer = Timer(args.iters)
    for mode in ("prompt", "single tokens"):
        n_entries, ctx = (1, args.tokens) if mode == "prompt" else (args.batch, args.context)
        pages_per = -(-ctx // page)
        keys = (torch.randn(n_entries * pages_per, 1, page, c + r, device="cuda") * 0.5).to(torch.bfloat16)
        table = torch.randperm(n_entries * pages_per, device="cuda", dtype=torch.int32).view(n_entries, pages_per).contiguous()
        n = ctx if mode == "prompt" else n_entries
        folded = torch.randn(n, h, c + r, device="cuda") * 0.05
        out = torch.empty(n, h, c, device="cuda")
        if mode == "prompt":
            q_start, kv_start, slots, max_q = i32([0, n]), i32([0]), i32([0]), n
            flops, moved = 2 * h * (2 * c + r) * ctx * (ctx + 1) / 2, None
        else:
            q_start, kv_start, slots, max_q = i32(list(range(n + 1))), i32([ctx - 1] * n), i32(list(range(n))), 1
            flops, moved = None, n * ctx * (c + r) * 2
        fn = lambda: ops.latent_attention(folded, keys, out, q_start, kv_start, slots, table, n_entries, max_q, h, c, r, 0.07,
                                          max_kv_len=ctx)
        report(f"latent_attention[{mode}]", timer(fn), flops=flops, bytes_moved=moved, entries=n_entries, context=ctx, heads=h,
               rank=c, rot=r)


def run_linear_attention(args) -> None:
    """The decayed linear attention kernel on a prompt of --tokens (flops of the chunked form) and on --batch single
    tokens (bytes: every head's state read and written once)."""
    h, d, v = args.heads, args.key_dim, args.value_dim
    chunk = ops.linear_attention_chunk(d, v)
    powers = (torch.full((h, 1), 0.99, dtype=torch.float64) ** torch.arange(chunk + 1, dtype=torch.float64)[None]).float().cuda()
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    timer = Timer(args.iters)
    for mode in ("prompt", "single tokens"):
        n_entries, n = (1, args.tokens) if mode == "prompt" else (args.batch, args.batch)
        q, k = (torch.randn(n, h * d, device="cuda").to(torch.bfloat16) for _ in range(2))
        val = torch.randn(n, h * v, device="cuda").to(torch.bfloat16)
        out = torch.empty(n, h * v, device="cuda")
        state = torch.zeros(n_entries, h, d, v, device="cuda")
        q_start = i32([0, n]) if mode == "prompt" else i32(list(range(n + 1)))
        slots = i32(list(range(n_entries)))
        fn = lambda: ops.linear_attention(q, k, val, out, state, powers, q_start, slots, n_entries, h, d, v, silu=True)
        if mode == "prompt":
            flops = 2 * h * n * (chunk * (d + v) / 2 + 2 * d * v)
            report("linear_attention[prompt]", timer(fn), flops=flops, tokens=n, heads=h, key_dim=d, value_dim=v, chunk=chunk)
        else:
            report("linear_attention[single tokens]", timer(fn), bytes_moved=2 * n * h * d * v * 4, batch=n, heads=h, key_dim=d,
                   value_dim=v)


def run_expert_product(args) -> None:
    """Both products of the routed experts over --tokens * --top sorted rows, and beside them one dense product of the same
    flops through the engine's ``linear`` (the like kernel of a dense feed-forward)."""
    from torchinferno_b200.kernels.gemm import LinearWeight, linear
    t, e, top, w, ff = args.tokens, args.experts, args.top, args.hidden, args.expert_size
    x = torch.randn(t, w, device="cuda").to(torch.bfloat16)
    ids = torch.stack([torch.randperm(e, device="cuda")[:top] for _ in range(t)]).to(torch.int32).contiguous()
    offsets = torch.empty(e + 1, dtype=torch.int32, device="cuda")
    order, place = (torch.empty(t * top, dtype=torch.int32, device="cuda") for _ in range(2))
    ops.moe_group(ids, e, offsets, order, place)
    up = (torch.randn(e, ff, w, device="cuda") * 0.02).to(torch.bfloat16)
    down = (torch.randn(e, w, ff, device="cuda") * 0.02).to(torch.bfloat16)
    inner = torch.empty(t * top, ff, dtype=torch.bfloat16, device="cuda")
    outer = torch.empty(t * top, w, dtype=torch.float32, device="cuda")
    timer = Timer(args.iters)
    flops = 2 * t * top * w * ff
    report("expert_product[up, relu^2]", timer(lambda: ops.moe_expert_product(x, up, inner, offsets, order, top, x_by_pair=True, act="relu2")),
           flops=flops, tokens=t, experts=e, top=top, hidden=w, expert_size=ff)
    report("expert_product[down]", timer(lambda: ops.moe_expert_product(inner, down, outer, offsets, order, top, x_by_pair=False)),
           flops=flops, tokens=t, experts=e, top=top, hidden=w, expert_size=ff)
    gate_up = (torch.randn(e, 2 * ff, w, device="cuda") * 0.02).to(torch.bfloat16)
    scale = torch.rand(t * top, device="cuda")
    report("expert_product[gate and up, clamped gated unit, row scale]",
           timer(lambda: ops.moe_expert_product(x, gate_up, inner, offsets, order, top, x_by_pair=True, act="glu_clamp", limit=7.0,
                                                alpha=1.702, row_scale=scale)),
           flops=2 * flops, tokens=t, experts=e, top=top, hidden=w, expert_size=ff)
    report("expert_product[gate and up, silu gated unit]",
           timer(lambda: ops.moe_expert_product(x, gate_up, inner, offsets, order, top, x_by_pair=True, act="swiglu")),
           flops=2 * flops, tokens=t, experts=e, top=top, hidden=w, expert_size=ff)
    dense = LinearWeight((torch.randn(top * ff, w, device="cuda") * 0.02).to(torch.bfloat16), few_rows_tcgen05=False)
    report("linear[dense, the same flops]", timer(lambda: linear(x, dense)), flops=flops, tokens=t, hidden=w, out=top * ff)


def run_sigmoid_attention(args) -> None:
    """The attention with sigmoid weights inside chunks on a prompt of --tokens (flops: both products over the keys a query
    sees) and on --batch single tokens at --context (bytes: the keys and values of the chunk each context ends in)."""
    h, k, d, v, page, chunk = args.heads, args.kv_heads, args.head_dim, args.value_dim, args.page_size, args.chunk
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    timer = Timer(args.iters)
    for mode in ("prompt", "single tokens"):
        n_entries, ctx = (1, args.tokens) if mode == "prompt" else (args.batch, args.context)
        pages_per = -(-ctx // page)
        pool = (torch.randn(n_entries * pages_per, k * page * (d + v), device="cuda") * 0.5).to(torch.bfloat16)
        keys = pool[:, :k * page * d].unflatten(1, (k, page, d))
        values = pool[:, k * page * d:].unflatten(1, (k, page, v))
        table = torch.randperm(n_entries * pages_per, device="cuda", dtype=torch.int32).view(n_entries, pages_per).contiguous()
        n = ctx if mode == "prompt" else n_entries
        q = torch.randn(n, h * d, device="cuda").to(torch.bfloat16)
        gate = torch.randn(n, h, device="cuda").to(torch.bfloat16)
        bias = torch.zeros(h, device="cuda")
        out = torch.empty(n, h * v, dtype=torch.bfloat16, device="cuda")
        seen = lambda p: p - (p // chunk) * chunk + 1 if chunk else p + 1
        if mode == "prompt":
            q_start, kv_start, slots, max_q = i32([0, n]), i32([0]), i32([0]), n
            flops, moved = 2 * h * (d + v) * sum(seen(p) for p in range(ctx)), None
        else:
            q_start, kv_start, slots, max_q = i32(list(range(n + 1))), i32([ctx - 1] * n), i32(list(range(n))), 1
            flops, moved = None, n * seen(ctx - 1) * k * (d + v) * 2
        for simt in (False, True):
            fn = lambda: ops.sigmoid_attention(q, keys, values, out, q_start, kv_start, slots, table, n_entries, max_q, h, k,
                                               scale=0.1, chunk=chunk, head_bias=bias, gate=gate, force_simt=simt)
            report(f"sigmoid_attention[{'cuda cores' if simt else 'mma.sync'}, {mode}]", timer(fn), flops=flops, bytes_moved=moved,
                   entries=n_entries, context=ctx, heads=h, kv_heads=k, head_dim=d, value_dim=v, chunk=chunk)


def run_gated_recurrence(args) -> None:
    """The element-wise gated recurrence on a prompt of --tokens and on --batch single tokens (bytes: the three projections
    read, the rows written, the state read and written)."""
    w = args.width
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    timer = Timer(args.iters)
    for mode in ("prompt", "single tokens"):
        n_entries, n = (1, args.tokens) if mode == "prompt" else (args.batch, args.batch)
        proj = torch.randn(n, 3 * w, device="cuda").to(torch.bfloat16)
        out = torch.empty(n, w, dtype=torch.bfloat16, device="cuda")
        state = torch.zeros(n_entries, w, device="cuda")
        bias = torch.zeros(w, device="cuda")
        q_start = i32([0, n]) if mode == "prompt" else i32(list(range(n + 1)))
        slots = i32(list(range(n_entries)))
        max_q = n if mode == "prompt" else 1
        fn = lambda: ops.gated_recurrence(proj, 0, w, 2 * w, bias, bias, state, q_start, slots, out, n_entries, max_q)
        report(f"gated_recurrence[{mode}]", timer(fn), bytes_moved=n * w * 8 + n_entries * w * 8, tokens=n, width=w)


def run_layer_tails(args) -> None:
    """The launches around a sublayer of a block with norms on both sides: the layer norm of the residual, and the tail
    (norm of the sublayer's output, sum, depth average over --depth earlier outputs, the next norm), beside the RMS
    norm with its fused sum (bytes: what each has to read and write)."""
    rows, w, depth = args.rows, args.hidden, args.depth
    timer = Timer(args.iters)
    history = torch.randn(depth + 1, rows, w, device="cuda")
    y = torch.randn(rows, w, device="cuda").to(torch.bfloat16)
    out = torch.empty(rows, w, dtype=torch.bfloat16, device="cuda")
    wt, b, coef = torch.ones(w, device="cuda"), torch.zeros(w, device="cuda"), torch.ones(depth, device="cuda")
    report("layernorm", timer(lambda: ops.layernorm(history[0], wt, b, 1e-6, out)), bytes_moved=rows * w * 6, rows=rows, hidden=w)
    report("layernorm_tail[norm, sum, norm]", timer(lambda: ops.layernorm_tail(history[0], 1e-6, y=y, y_norm=(wt, b), out=out, out_norm=(wt, b))),
           bytes_moved=rows * w * 12, rows=rows, hidden=w)
    report("layernorm_tail[norm, sum, depth average]",
           timer(lambda: ops.layernorm_tail(history[depth - 1], 1e-6, y=y, y_norm=(wt, b), history=history, coef=coef, count=depth)),
           bytes_moved=rows * w * (2 + 8 + 4 * depth), rows=rows, hidden=w, depth=depth)
    delta = torch.randn(rows, w, device="cuda").to(torch.bfloat16)
    report("add_rmsnorm", timer(lambda: ops.add_rmsnorm(delta, history[0], wt, 1e-6, out)), bytes_moved=rows * w * 12, rows=rows, hidden=w)


def run_pooled_window_attention(args) -> None:
    """The attention over a window plus pooled blocks on a prompt of --tokens (flops: both products over the tokens and
    blocks a query sees) and on --batch single tokens at --context (bytes: the keys and values of the window and of the
    blocks each query sees), with sink, temperature, rotated values and the output gate."""
    h, k, d, v, page, window, pool = args.heads, args.kv_heads, args.head_dim, args.value_dim, args.page_size, args.window, args.pool
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    timer = Timer(args.iters)

    def pages(n_entries, entries_per):
        per = -(-entries_per // page)
        pool_ = (torch.randn(n_entries * per, k * page * (d + v), device="cuda") * 0.5).to(torch.bfloat16)
        table = torch.randperm(n_entries * per, device="cuda", dtype=torch.int32).view(n_entries, per).contiguous()
        return pool_[:, :k * page * d].unflatten(1, (k, page, d)), pool_[:, k * page * d:].unflatten(1, (k, page, v)), table

    seen = lambda p: min(p + 1, window) + max(0, p - window + 1) // pool
    for mode in ("prompt", "single tokens"):
        n_entries, ctx = (1, args.tokens) if mode == "prompt" else (args.batch, args.context)
        keys, values, table = pages(n_entries, ctx)
        bkeys, bvalues, btable = pages(n_entries, ctx // pool + 1)
        n = ctx if mode == "prompt" else n_entries
        q = torch.randn(n, h * d, device="cuda").to(torch.bfloat16)
        gate = torch.randn(n, h * v, device="cuda").to(torch.bfloat16)
        temp, sink = torch.ones(h, device="cuda"), torch.zeros(h, device="cuda")
        vfreq = (10000.0 ** (-torch.arange(v // 2, dtype=torch.float64) * 2 / v)).float().cuda()
        out = torch.empty(n, h * v, dtype=torch.bfloat16, device="cuda")
        if mode == "prompt":
            q_start, kv_start, slots, max_q = i32([0, n]), i32([0]), i32([0]), n
            flops, moved = 2 * h * (d + v) * sum(seen(p) for p in range(ctx)), None
        else:
            q_start, kv_start, slots, max_q = i32(list(range(n + 1))), i32([ctx - 1] * n), i32(list(range(n))), 1
            flops, moved = None, n * seen(ctx - 1) * k * (d + v) * 2
        fn = lambda: ops.pooled_window_attention(q, out, q_start, kv_start, slots, keys, values, table, bkeys, bvalues, btable, n_entries,
                                                 max_q, h, k, window=window, pool=pool, scale=0.09, temp=temp, sink=sink,
                                                 value_freq=vfreq, gate=gate)
        report(f"pooled_window_attention[{mode}]", timer(fn), flops=flops, bytes_moved=moved, entries=n_entries, context=ctx, heads=h,
               kv_heads=k, head_dim=d, value_dim=v, window=window, pool=pool)
    # the launch ahead of it: biases, the two rotations, the store into the pages; then the means of completed blocks
    n = args.tokens
    keys, values, table = pages(1, n)
    bkeys, bvalues, btable = pages(1, n // pool + 1)
    proj = torch.randn(n, (h + k) * d + k * v + h * v, device="cuda").to(torch.bfloat16)
    q = torch.empty(n, h * d, dtype=torch.bfloat16, device="cuda")
    freq = (10000.0 ** (-torch.arange(d // 4, dtype=torch.float64) * 4 / d)).float().cuda()
    vfreq = (10000.0 ** (-torch.arange(v // 2, dtype=torch.float64) * 2 / v)).float().cuda()
    positions, token_slot = i32(list(range(n))), i32([0] * n)
    bias = [torch.zeros(w, device="cuda") for w in (h * d, k * d, k * v)]
    fn = lambda: ops.rotary_kv_append(proj, 0, h * d, (h + k) * d, q, keys, values, positions, token_slot, table, freq, vfreq, h, k, d, v,
                                      rot_dim=d // 2, amplitude=1.07, q_bias=bias[0], k_bias=bias[1], v_bias=bias[2])
    report("rotary_kv_append[prompt]", timer(fn), bytes_moved=n * ((h + k) * d + k * v) * 4, tokens=n)
    fn = lambda: ops.pool_blocks(keys, values, table, bkeys, bvalues, btable, positions, token_slot, pool)
    report("pool_blocks[prompt]", timer(fn), bytes_moved=n * k * (d + v) * 2 + (n // pool) * k * (d + v) * 2, tokens=n, pool=pool)


def run_biased_attention(args) -> None:
    """The causal attention with a learned bias per head and distance on a prompt of --tokens (flops: both products over
    the keys a query sees) and on --batch single tokens at --context (bytes: the keys and values of every context once);
    then the launch ahead of it (norm of q and k with a weight, the query's temperature, the store into the pages)."""
    h, k, d, v, page = args.heads, args.kv_heads, args.head_dim, args.value_dim, args.page_size
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    timer = Timer(args.iters)

    def pages(n_entries, entries_per):
        per = -(-entries_per // page)
        pool_ = (torch.randn(n_entries * per, k * page * (d + v), device="cuda") * 0.5).to(torch.bfloat16)
        table = torch.randperm(n_entries * per, device="cuda", dtype=torch.int32).view(n_entries, per).contiguous()
        return pool_[:, :k * page * d].unflatten(1, (k, page, d)), pool_[:, k * page * d:].unflatten(1, (k, page, v)), table

    rel = torch.randn(h, args.bias_max + 1, device="cuda")
    for mode in ("prompt", "single tokens"):
        n_entries, ctx = (1, args.tokens) if mode == "prompt" else (args.batch, args.context)
        keys, values, table = pages(n_entries, ctx)
        n = ctx if mode == "prompt" else n_entries
        q = torch.randn(n, h * d, device="cuda").to(torch.bfloat16)
        out = torch.empty(n, h * v, dtype=torch.bfloat16, device="cuda")
        if mode == "prompt":
            q_start, kv_start, slots, max_q = i32([0, n]), i32([0]), i32([0]), n
            flops, moved = 2 * h * (d + v) * ctx * (ctx + 1) / 2, None
        else:
            q_start, kv_start, slots, max_q = i32(list(range(n + 1))), i32([ctx - 1] * n), i32(list(range(n))), 1
            flops, moved = None, n * ctx * k * (d + v) * 2
        for name, bias in (("biased_attention", rel), ("the same without the bias", None)):
            fn = lambda: ops.pooled_window_attention(q, out, q_start, kv_start, slots, keys, values, table, None, None, None, n_entries,
                                                     max_q, h, k, window=1 << 30, pool=0, scale=0.09, rel_bias=bias, max_kv_len=ctx)
            report(f"{name}[{mode}]", timer(fn), flops=flops, bytes_moved=moved, entries=n_entries, context=ctx, heads=h, kv_heads=k,
                   head_dim=d, value_dim=v, bias_max=args.bias_max)
    n = args.tokens
    keys, values, table = pages(1, n)
    proj = torch.randn(n, (h + k) * d + k * v, device="cuda").to(torch.bfloat16)
    q = torch.empty(n, h * d, dtype=torch.bfloat16, device="cuda")
    positions, token_slot = i32(list(range(n))), i32([0] * n)
    qw, kw = torch.ones(d, device="cuda"), torch.ones(d, device="cuda")
    fn = lambda: ops.qk_norm_append(proj, 0, h * d, (h + k) * d, q, keys, values, positions, token_slot, table, None, h, k, d, v,
                                    rot_dim=0, eps=1e-6, q_weight=qw, k_weight=kw, temp_coef=0.1, temp_every=512)
    report("qk_norm_append[prompt, weights and temperature]", timer(fn), bytes_moved=n * ((h + k) * d + k * v) * 4, tokens=n)


def run_hyper_streams(args) -> None:
    """A residual in --streams streams: the write of a sublayer's output and the read for the next with the tanh norm in one
    launch (bytes: every stream read and written in fp32, the output rows read, the normed rows written), the read alone,
    and beside them the residual sum with an RMS norm of a single residual."""
    rows, w, s = args.rows, args.hidden, args.streams
    timer = Timer(args.iters)
    streams = torch.randn(s, rows, w, device="cuda")
    y = torch.randn(rows, w, device="cuda").to(torch.bfloat16)
    out = torch.empty(rows, w, dtype=torch.bfloat16, device="cuda")
    mix = (torch.eye(s, device="cuda") + 0.01).contiguous()
    coef, wt, b = torch.ones(s, device="cuda") / s, torch.ones(w, device="cuda"), torch.zeros(w, device="cuda")
    report("hyper_step[write, read, tanh norm]",
           timer(lambda: ops.hyper_step(streams, y=y, mix=mix, out_weights=coef, in_weights=coef, out=out, tanh_norm=(0.5, wt, b))),
           bytes_moved=rows * w * (8 * s + 4), rows=rows, hidden=w, streams=s)
    report("hyper_step[read, tanh norm]", timer(lambda: ops.hyper_step(streams, in_weights=coef, out=out, tanh_norm=(0.5, wt, b))),
           bytes_moved=rows * w * (4 * s + 2), rows=rows, hidden=w, streams=s)
    few = min(rows, 8)
    report("hyper_step[write, read, tanh norm, few rows]",
           timer(lambda: ops.hyper_step(streams[:, :few], y=y[:few], mix=mix, out_weights=coef, in_weights=coef, out=out[:few],
                                        tanh_norm=(0.5, wt, b))), bytes_moved=few * w * (8 * s + 4), rows=few, hidden=w, streams=s)
    report("add_rmsnorm", timer(lambda: ops.add_rmsnorm(y, streams[0], wt, 1e-6, out)), bytes_moved=rows * w * 12, rows=rows, hidden=w)


def run_state_space(args) -> None:
    """The state-space mixer's kernels on a prompt of --tokens and on --batch single tokens: the short convolution, the
    scan (bytes: the rows [x | B | C] and the step sizes read, the 32-bit sums written, the state read and written) and
    the gate with the norm in parts."""
    heads, p_, n_state, groups, taps = args.heads, args.head_dim, args.state, args.groups, args.taps
    inner, channels = heads * p_, heads * p_ + 2 * groups * n_state
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device="cuda")
    timer = Timer(args.iters)
    for mode in ("prompt", "single tokens"):
        n_entries, n = (1, args.tokens) if mode == "prompt" else (args.batch, args.batch)
        proj = (torch.randn(n, 2 * inner + 2 * groups * n_state + heads, device="cuda") * 0.5).to(torch.bfloat16)
        xbc = torch.empty(n, channels, dtype=torch.bfloat16, device="cuda")
        state = torch.zeros(n_entries, heads * n_state * p_ + (taps - 1) * channels, device="cuda")
        q_start = i32([0, n]) if mode == "prompt" else i32(list(range(n + 1)))
        slots, max_q = i32(list(range(n_entries))), (n if mode == "prompt" else 1)
        cw, cb = torch.randn(channels, taps, device="cuda") * 0.5, torch.zeros(channels, device="cuda")
        vec = [torch.zeros(heads, device="cuda") for _ in range(3)]
        y = torch.empty(n, inner, device="cuda")
        rows = torch.empty(n, inner, dtype=torch.bfloat16, device="cuda")
        weight = torch.ones(inner, device="cuda")
        fn = lambda: ops.short_conv(proj, inner, cw, cb, state, heads * n_state * p_, q_start, slots, xbc, n_entries, max_q, silu=True)
        report(f"short_conv[{mode}]", timer(fn), bytes_moved=n * channels * 4 + n_entries * (taps - 1) * channels * 8, tokens=n, channels=channels)
        fn = lambda: ops.ssd_scan(xbc, proj, inner + channels, vec[0], vec[1], vec[2], state, q_start, slots, y, n_entries, heads=heads,
                                  groups=groups, state_dim=n_state, head_dim=p_, max_q_len=max_q)
        report(f"ssd_scan[{mode}]", timer(fn), bytes_moved=n * (channels * 2 + heads * 2 + inner * 4) + n_entries * heads * n_state * p_ * 8,
               flops=None, tokens=n, heads=heads, head_dim=p_, state=n_state, scan_gflop=round(n * heads * p_ * n_state * 6 / 1e9, 2))
        fn = lambda: ops.gated_group_norm(y, proj, 0, weight, 1e-6, rows, args.norm_groups)
        report(f"gated_group_norm[{mode}]", timer(fn), bytes_moved=n * inner * 8, tokens=n, width=inner)


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="python -m torchinferno_b200.bench_kernels", description=__doc__.splitlines()[0])
    parser.add_argument("--ordinary-launches", action="store_true",
                        help="launch the kernels without programmatic dependent launch (a profiler that lists kernels "
                             "by name does not see dependent launches)")
    sub = parser.add_subparsers(dest="command", required=True)

    def common(p):
        p.add_argument("--heads", type=int, default=32)
        p.add_argument("--kv-heads", type=int, default=8)
        p.add_argument("--head-dim", type=int, default=128)
        p.add_argument("--page-size", type=int, default=16)
        p.add_argument("--iters", type=int, default=20)

    p = sub.add_parser("decode-attention")
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--splits", type=int, nargs="*", default=None, help="try these numbers of context splits")
    common(p)
    p.set_defaults(func=run_decode_attention)
    p = sub.add_parser("prefill-attention")
    p.add_argument("--batch", type=int, default=1)
    p.add_argument("--tokens", type=int, default=2048)
    common(p)
    p.set_defaults(func=run_prefill_attention)
    p = sub.add_parser("gemm")
    p.add_argument("--rows", type=int, default=8)
    p.add_argument("--only", nargs="*", default=None)
    p.add_argument("--iters", type=int, default=20)
    p.add_argument("--decode-config", type=int, nargs=2, default=None, metavar=("FEATURES", "SPLITS"),
                   help="of the few-rows kernel's configurations only this one")
    p.set_defaults(func=run_gemm)
    p = sub.add_parser("elementwise")
    p.add_argument("--rows", type=int, default=2048)
    p.add_argument("--hidden", type=int, default=4096)
    p.add_argument("--intermediate", type=int, default=14336)
    common(p)
    p.set_defaults(func=run_elementwise)
    p = sub.add_parser("step-timeline")
    p.add_argument("--layers", type=int, default=32)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=3072)
    p.add_argument("--hidden", type=int, default=4096)
    p.add_argument("--intermediate", type=int, default=14336)
    p.add_argument("--vocab", type=int, default=128256)
    p.add_argument("--gemm-backend", choices=["auto", "tcgen05", "library"], default="auto")
    p.add_argument("--plain", action="store_true", help="run the steps without the activity profiler (for ncu)")
    p.add_argument("--prompt", action="store_true", help="the step of one whole prompt of --context tokens instead of a decode step")
    common(p)
    p.set_defaults(func=run_step_timeline, iters=3)
    p = sub.add_parser("latent-attention")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--rank", type=int, default=512)
    p.add_argument("--rot", type=int, default=64)
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--iters", type=int, default=10)
    p.set_defaults(func=run_latent_attention)
    p = sub.add_parser("linear-attention")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--key-dim", type=int, default=128)
    p.add_argument("--value-dim", type=int, default=128)
    p.add_argument("--iters", type=int, default=10)
    p.set_defaults(func=run_linear_attention)
    p = sub.add_parser("expert-product")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--experts", type=int, default=32)
    p.add_argument("--top", type=int, default=4)
    p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--expert-size", type=int, default=1024)
    p.add_argument("--iters", type=int, default=10)
    p.set_defaults(func=run_expert_product)
    p = sub.add_parser("sigmoid-attention")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--value-dim", type=int, default=128)
    p.add_argument("--chunk", type=int, default=512)
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--iters", type=int, default=10)
    p.set_defaults(func=run_sigmoid_attention)
    p = sub.add_parser("gated-recurrence")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--width", type=int, default=2048)
    p.add_argument("--iters", type=int, default=10)
    p.set_defaults(func=run_gated_recurrence)
    p = sub.add_parser("layer-tails")
    p.add_argument("--rows", type=int, default=2048)
    p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--depth", type=int, default=5)
    p.add_argument("--iters", type=int, default=10)
    p.set_defaults(func=run_layer_tails)
    p = sub.add_parser("pooled-window-attention")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--value-dim", type=int, default=128)
    p.add_argument("--window", type=int, default=512)
    p.add_argument("--pool", type=int, default=64)
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--iters", type=int, default=10)
    p.set_defaults(func=run_pooled_window_attention)
    p = sub.add_parser("biased-attention")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--context", type=int, default=2048)
    p.add_argument("--heads", type=int, default=16)
    p.add_argument("--kv-heads", type=int, default=8)
    p.add_argument("--head-dim", type=int, default=128)
    p.add_argument("--value-dim", type=int, default=128)
    p.add_argument("--bias-max", type=int, default=1024)
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--iters", type=int, default=10)
    p.set_defaults(func=run_biased_attention)
    p = sub.add_parser("hyper-streams")
    p.add_argument("--rows", type=int, default=2048)
    p.add_argument("--hidden", type=int, default=2048)
    p.add_argument("--streams", type=int, default=2)
    p.add_argument("--iters", type=int, default=10)
    p.set_defaults(func=run_hyper_streams)
    p = sub.add_parser("state-space")
    p.add_argument("--tokens", type=int, default=2048)
    p.add_argument("--batch", type=int, default=8)
    p.add_argument("--heads", type=int, default=64)
    p.add_argument("--head-dim", type=int, default=64)
    p.add_argument("--state", type=int, default=128)
    p.add_argument("--groups", type=int, default=1)
    p.add_argument("--taps", type=int, default=4)
    p.add_argument("--norm-groups", type=int, default=1)
    p.add_argument("--iters", type=int, default=10)
    p.set_defaults(func=run_state_space)
    args = parser.parse_args(argv)
    if not torch.cuda.is_available():
        raise SystemExit("bench_kernels needs a CUDA device")
    if args.ordinary_launches:
        ops.set_dependent_launch(False)
    with torch.inference_mode():
        args.func(args)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
