"""The Tibalorn design on the GPU against the plain implementation (tests/plain_tibalorn.py): each mechanism alone, the
residual stream layer by layer, whole prompts, token-by-token decoding, portions down to two tokens, mixed batches on
a tight pool with four slots, long decoding, keys at the edges of windows, blocks and pages, slots and pages used
again, greedy generation through the engine's entry point, and the trace program."""
import json
import math

import numpy as np
import pytest
import torch

import plain_tibalorn
import replay_util
from gpu_common import F32_ATOL, F32_RTOL, need_gpu, note_worst
from tibalorn_configs import CONFIGS, attention, dense, mamba2, write_model

pytestmark = pytest.mark.gpu
CUDA = torch.device("cuda")
# float32: every row within the bounds the Llama tests use.  bfloat16 (rows, keys, values and block means are kept in
# bfloat16 between kernels; the models are narrow, so a row's error is the sum of few roundings and scatters widely):
# nine rows in ten within BF16_REL of the largest logit of their sequence, every row within twice that, and half of
# the rows within a third of it.
BF16_REL = 0.06


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write_model(config, tmp_path_factory.mktemp(name), seed) for name, (config, seed) in CONFIGS.items()}


_plain: dict = {}


def plain(folder, tokens):
    key = (str(folder), tuple(tokens))
    if key not in _plain:
        if str(folder) not in _plain:
            _plain[str(folder)] = plain_tibalorn.read_model_folder(folder)
        config, weights = _plain[str(folder)]
        _plain[key] = plain_tibalorn.forward(config, weights, tokens).numpy()
    return _plain[key]


def requests_for(config, seed, lengths):
    g = torch.Generator().manual_seed(900 + seed)
    return {f"q{i}": torch.randint(0, config["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}


def compare(rows, folder, requests, dtype, what):
    assert rows, "nothing was compared"
    shares = []
    for (name, pos), got_list in rows.items():
        ref = plain(folder, requests[name])
        for got in got_list:
            got = np.asarray(got, dtype=np.float64)
            assert np.isfinite(got).all(), f"{name}@{pos}: non-finite logits"
            err = np.abs(got - ref[pos]).max()
            if dtype == "float32":
                bound = F32_ATOL + F32_RTOL * np.abs(ref[pos]).max()
                assert err <= bound, f"{what}: {name}@{pos} ({dtype}): max error {err:.3e} exceeds {bound:.3e}"
            else:
                bound = BF16_REL * np.abs(ref).max()
                assert err <= 2 * bound, f"{what}: {name}@{pos} ({dtype}): max error {err:.3e} exceeds {2 * bound:.3e}"
            shares.append(err / bound)
    shares = np.sort(np.asarray(shares))
    if dtype == "float32":
        note_worst(f"tibalorn {what} [{dtype}]", shares[-1])
    else:
        ninth, median = shares[int(0.9 * (len(shares) - 1))], shares[len(shares) // 2]
        assert ninth <= 1.0 and median <= 1 / 3, f"{what} ({dtype}): nine in ten rows within {ninth:.2f} of the bound, median {median:.2f}"
        note_worst(f"tibalorn {what}, nine rows in ten [{dtype}]", ninth)


def make_runner(folder, dtype, max_tokens, page_size=16, max_requests=4):
    from torchinferno_b200.engine.factory import load_model, make_runner as make
    model = load_model(folder, dtype=dtype)
    return make(model, page_size=page_size, max_tokens=max_tokens + page_size * max_requests, max_requests=max_requests)


def run_steps(runner, steps):
    from torchinferno_b200.engine.batch import StepEntry
    out = {}
    with torch.inference_mode():
        for step in steps:
            logits = runner.step([StepEntry(e["id"], e["tokens"], e["want"]) for e in step["entries"]])
            if logits.shape[0]:
                out[step["step"]] = logits.cpu().numpy()
            runner.end(step["end"])
            runner.cache.audit()
    return out


# ------------------------------------------------------------ whole models
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_residual_stream_after_every_layer(name, folders):
    need_gpu()
    from torchinferno_b200.engine.batch import StepEntry
    from torchinferno_b200.parts.block import PreNormBlock
    config, seed = CONFIGS[name]
    tokens = requests_for(config, seed, [45])["q0"]
    cfg, w = plain_tibalorn.read_model_folder(folders[name])
    _, want = plain_tibalorn.forward(cfg, w, tokens, keep_layers=True)
    runner = make_runner(folders[name], "float32", 64)
    seen, original = [], PreNormBlock.forward

    def recording(self, stream, ctx):
        original(self, stream, ctx)
        seen.append(stream.residual.clone() if stream.pending is None else stream.residual + stream.pending.float())
    PreNormBlock.forward = recording
    try:
        with torch.inference_mode():
            runner.step([StepEntry("a", tokens, [0])])
    finally:
        PreNormBlock.forward = original
    assert len(seen) == want.shape[0]
    for i, got in enumerate(seen):
        err = (got.cpu().double() - want[i]).abs().max()
        assert err <= 1e-4 * want[i].abs().max(), f"layer {i}: {err:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_tail_portions_and_mixed_batches(name, dtype, folders):
    need_gpu()
    config, seed = CONFIGS[name]
    requests = requests_for(config, seed, [1, 2, 37, 70, 131, 64, 33])
    page = {"TA": 16, "TB": 4, "TC": 8, "TD": 8, "TE": 2}[name]
    for kind, (steps, index) in {
            "whole": replay_util.trace_whole(requests), "tail": replay_util.trace_tail_decode(requests, tail=40),
            "portions": replay_util.trace_portions(requests, sizes=(2, 7, 16, 3, 33, 2, 5, 31, 32, 2, 64)),
            "mixed": replay_util.trace_mixed(requests, seed=seed)}.items():
        runner = make_runner(folders[name], dtype, replay_util.peak_tokens(steps), page_size=page)
        rows = replay_util.gather(run_steps(runner, steps), index)
        compare(rows, folders[name], requests, dtype, f"{name} {kind}")
        assert not runner.cache.live_requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["TA", "TB"])
def test_every_token_decoded_alone_from_the_first_and_long_decoding(name, dtype, folders):
    need_gpu()
    config, seed = CONFIGS[name]
    requests = requests_for(config, seed + 5, [150, 9])
    steps, index = replay_util.trace_tail_decode(requests, tail=10 ** 6)       # one token a step from position 0
    runner = make_runner(folders[name], dtype, replay_util.peak_tokens(steps), page_size=4)
    rows = replay_util.gather(run_steps(runner, steps), index)
    assert runner.counters["graph_steps"] > 100                              # the captured decode pass ran them
    compare(rows, folders[name], requests, dtype, f"{name} token by token")


def test_a_batch_of_unequal_requests_gives_each_what_it_gets_alone(folders):
    need_gpu()
    from torchinferno_b200.engine.batch import StepEntry
    config, seed = CONFIGS["TA"]
    reqs = requests_for(config, seed + 9, [150, 3, 69, 1])
    runner = make_runner(folders["TA"], "float32", 4 * 192, page_size=8)
    with torch.inference_mode():
        alone = {}
        for k, toks in reqs.items():
            alone[k] = runner.step([StepEntry(k + "a", toks, list(range(len(toks))))]).cpu()
            runner.end([k + "a"])
        # together: a portion of each, then the rest of each, in another order (slots and pages are used again)
        first = {k: max(1, len(t) // 2) for k, t in reqs.items()}
        got = {k: [] for k in reqs}
        out = runner.step([StepEntry(k, reqs[k][:first[k]], list(range(first[k]))) for k in reqs]).cpu()
        row = 0
        for k in reqs:
            got[k].append(out[row:row + first[k]]); row += first[k]
        rest = [k for k in reversed(list(reqs)) if len(reqs[k]) > first[k]]
        out = runner.step([StepEntry(k, reqs[k][first[k]:], list(range(len(reqs[k]) - first[k]))) for k in rest]).cpu()
        row = 0
        for k in rest:
            n = len(reqs[k]) - first[k]
            got[k].append(out[row:row + n]); row += n
        runner.end(list(reqs))
    for k in reqs:
        assert torch.allclose(torch.cat(got[k]), alone[k], atol=2e-6, rtol=2e-5), k


# ------------------------------------------------------- mechanisms alone
def _entries_batch(entries):
    from torchinferno_b200.engine.batch import EntryPlacement, build_batch
    places, row = [], 0
    for rid, slot, start, n in entries:
        places.append(EntryPlacement(rid, slot, row, n, start))
        row += n
    batch, _ = build_batch(places, [[0] * p.q_len for p in places], [[] for _ in places], [], CUDA)
    return batch


def _bind(part, stored, dtype, prefix):
    """Bind weights given in bfloat16-exact values (as a checkpoint would hold them); returns them in float64 by full name."""
    vectors = {ws.name for ws in part.weight_specs() if ws.role == "vector"}
    part.bind({k: (v.float() if dtype == torch.float32 or k in vectors else v.to(torch.bfloat16)).cuda() for k, v in stored.items()})
    return {prefix + k: v.double() for k, v in stored.items()}


def _random_weights(part, seed, dtype, prefix):
    from torchinferno_b200.weights.random_init import random_tensor
    return _bind(part, {ws.name: random_tensor(ws, seed, dtype=torch.bfloat16) for ws in part.weight_specs()}, dtype, prefix)


def _apply_tables(cache):
    from torchinferno_b200.kernels import ops
    for group, (idx, val) in zip(cache.groups, cache.drain_table_updates()):
        if idx:
            ops.scatter_i32(group.table_device, torch.tensor(idx, dtype=torch.int32).cuda(), torch.tensor(val, dtype=torch.int32).cuda())


def _two_cache_context(cache, entries):
    from torchinferno_b200.parts.base import KVBinding, LayerContext
    a, b = cache.kv_binding(0), cache.kv_binding(1)
    return LayerContext(batch=_entries_batch(entries), error_word=cache.error_word,
                        kv=KVBinding(a.pool, a.block_table, a.page_size, a.window, True, a.keys, a.values),
                        side_kv=KVBinding(b.pool, b.block_table, b.page_size, b.window, True, b.keys, b.values))


def _direct_attention(m, dtype, seed):
    """A pooled-window attention whose input row is [q | k | v | gate] itself: the projections pick their columns (the
    products are then exact in both number formats), so that a test sets queries, keys and values by hand.  Biases,
    temperatures, sinks and the output projection are random.  Returns (mixer, weights in float64, the columns' starts)."""
    from torchinferno_b200.parts.base import PartSpec, build_part
    from torchinferno_b200.weights.random_init import random_tensor
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    widths = {"q": H * d, "k": G * d, "v": G * dv, "g": H * dv}
    W = sum(widths.values())
    rot = m["rot"]
    law = rot.get("scaling")
    law = None if law is None else dict(law, rope_type="yarn")
    mixer = build_part("mixer", PartSpec("pooled_window_attention", {
        "hidden_size": W, "heads": H, "kv_heads": G, "dim": d, "value_dim": dv, "scale": m["scale"],
        "position": PartSpec("rotary", {"head_dim": d, "theta": rot["base"], "rot_dim": rot["dims"], "scaling": law}),
        "window": m["mask"]["size"], "pool": m["mask"]["pool"], "value_rotation_base": rot["base"], "bias": True, "sink": True,
        "temperature": True, "gate": True}), dtype=dtype, device=CUDA)
    stored = {ws.name: random_tensor(ws, seed, dtype=torch.bfloat16) for ws in mixer.weight_specs()}
    starts, at = {}, 0
    for name, width in widths.items():
        pick = torch.zeros(width, W)
        pick[torch.arange(width), at + torch.arange(width)] = 1.0
        assert stored[name].shape == pick.shape
        stored[name] = pick.to(torch.bfloat16)
        starts[name], at = at, at + width
    return mixer, _bind(mixer, stored, dtype, "mix."), starts


def _attention_cache(mixer, dtype, page, pages, max_requests, tokens):
    from torchinferno_b200.cache.manager import CacheManager
    cache = CacheManager([mixer.cache_spec(), mixer.side_cache_spec()], [None], page_size=page, num_pages=pages,
                         max_requests=max_requests, max_request_tokens=tokens, dtype=dtype, device=CUDA)
    for group in cache.groups:
        group.pool.fill_(float("nan"))       # (what was never written must never be read)
    return cache


def _run_portions(mixer, cache, name, x, portions, release=True):
    outs, at = [], 0
    for n in portions:
        start = cache.extend(name, n)
        _apply_tables(cache)
        outs.append(mixer.forward(x[at:at + n].cuda().contiguous(), _two_cache_context(cache, [(name, cache.slot(name), start, n)])))
        if release:
            cache.release_behind_window(name)
        at += n
    assert at == x.shape[0] and int(cache.error_word) == 0
    cache.audit()
    return torch.cat(outs).cpu().double()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,size,pool,page", [
    (4, 2, 16, 24, 20, 6, 8), (3, 1, 40, 8, 7, 3, 4), (2, 2, 64, 64, 33, 16, 16), (2, 1, 8, 4, 5, 1, 2), (1, 1, 12, 6, 4, 9, 4),
    (6, 2, 32, 32, 16, 16, 16),
    # sixteen and eight query heads on one key head: a single token, or a portion of two, fills the sixteen rows up to
    # which the warps of the tensor-core kernel take a tile each
    (16, 1, 16, 16, 9, 4, 8), (8, 1, 24, 8, 70, 5, 16)])
def test_pooled_window_attention_alone_at_the_edges_of_windows_blocks_and_pages(dtype, heads, kv_heads, dim, vdim, size, pool, page):
    """A prompt in portions, then single tokens, in a pool whose pages were used before and go back as the window passes.
    Some tokens carry values thirty times the usual size, and whole blocks do: a query that sees a token one step too long
    or too short, or a block one query too early or too late, in a prompt or decoded alone, is far off; so is one that
    reads a wrong page or a block mean that was made from the wrong tokens."""
    need_gpu()
    m = attention(heads, kv_heads, dim, vdim, size, pool, 0.3, rot_dims=dim // 2 if dim % 4 == 0 else dim, base=1000.0,
                  scaling=(4.0, 64, 8.0, 1.0))
    mixer, w, starts = _direct_attention(m, dtype, seed=3)
    T = 3 * size + 4 * pool + 19
    g = torch.Generator().manual_seed(size * 100 + pool)
    x = torch.randn(T, mixer.hidden_size, generator=g)
    x[:, starts["q"]:starts["k"]] *= 2.0 / math.sqrt(dim)            # (scores of about one: no key takes all the weight)
    v0, v1 = starts["v"], starts["v"] + kv_heads * vdim
    loud = [size + 1, 2 * size, 2 * size + pool + 3]
    for p in loud:
        x[p, v0:v1] *= 30
    b_loud = (size + 2 * pool) // pool + 1                           # a whole block of large values
    x[b_loud * pool:(b_loud + 1) * pool, v0:v1] *= 30
    x = x.to(torch.bfloat16).to(dtype)
    pos = torch.arange(T)
    want = plain_tibalorn.attention_mixer(x.double(), w, "mix.", m, pos)
    # the test can tell: a window one token longer or shorter gives another answer where a loud token enters or leaves it
    for other in (size + 1, size - 1):
        if other < 1 or pool == 1:      # (with blocks of one token, what leaves the window comes back at once as its own block)
            continue
        off = plain_tibalorn.attention_mixer(x.double(), w, "mix.", dict(m, mask={"size": other, "pool": pool}), pos)
        edge = [p + size - 1 for p in loud] + [p + size for p in loud]
        assert max((off[i] - want[i]).abs().max() / want[i].abs().max() for i in edge if i < T) > 0.1
    cache = _attention_cache(mixer, dtype, page, -(-T // page) + 6, 3, T + page)
    cache.open("old"), cache.extend("old", 2 * page + 1), cache.open("warm"), cache.extend("warm", page + 1)
    cache.close("old")                  # its pages go to "r", out of order
    cache.open("r")
    portions = [size - 1, 2, pool, 1, 1, size + pool + 3, 2]
    portions += [1] * (T - sum(portions))
    got = _run_portions(mixer, cache, "r", x, portions)
    tol = 2e-5 if dtype == torch.float32 else BF16_REL
    err = (got - want).abs().max(dim=1).values / want.abs().max()
    assert err.max() <= tol, (int(err.argmax()), float(err.max()))
    # the window let pages go while the request lived, and the blocks' cache grew pool times slower than the tokens'
    assert sum(p >= 0 for p in cache.block_table("r", 0)) <= -(-max(size, pool) // page) + 1
    assert sum(p >= 0 for p in cache.block_table("r", 1)) == -(-(T // pool) // page)
    # a second request in the slot and pages the first one leaves: nothing of the first shows
    cache.close("r"), cache.close("warm")
    cache.open("s")
    again = _run_portions(mixer, cache, "s", x[:size + pool + 5], [size + pool + 4, 1])
    assert ((again - want[:size + pool + 5]).abs().max() / want.abs().max()) <= tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pooled_window_attention_finds_a_far_block_among_many_and_two_requests_side_by_side(dtype):
    """700 tokens over pages of 16, a window of 40 and blocks of 8: the token at position 3 has a value a hundred times
    the usual size and a key that the last queries match in the part of the head that is not rotated, so its block's
    mean stands out among 80 blocks.  Decoded tokens and a prompt's tail must both see it, also with a second,
    shorter request in the same steps."""
    need_gpu()
    T, far, size, pool, d, dv = 700, 3, 40, 8, 16, 16
    m = attention(2, 1, d, dv, size, pool, 0.5, rot_dims=4, base=100.0)
    mixer, w, starts = _direct_attention(m, dtype, seed=9)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(T, mixer.hidden_size, generator=g) * 0.5
    other = torch.randn(100, mixer.hidden_size, generator=g) * 0.5
    u = torch.zeros(d)
    u[6:] = 1.0                                            # a direction outside the rotated part
    x[far, starts["k"]:starts["k"] + d] = 12 * u
    x[far, starts["v"]:starts["v"] + dv] *= 100
    for i in range(T - 12, T):                             # both heads of the last queries look that way
        x[i, starts["q"]:starts["q"] + 2 * d] += torch.cat([u, u])
    x, other = x.to(torch.bfloat16).to(dtype), other.to(torch.bfloat16).to(dtype)
    want = plain_tibalorn.attention_mixer(x.double(), w, "mix.", m, torch.arange(T))
    want_other = plain_tibalorn.attention_mixer(other.double(), w, "mix.", m, torch.arange(100))
    lost = x.clone()
    lost[far, starts["v"]:starts["v"] + dv] = 0
    without = plain_tibalorn.attention_mixer(lost.double(), w, "mix.", m, torch.arange(T))
    assert (without[-1] - want[-1]).abs().max() > 0.3 * want[-1].abs().max()
    cache = _attention_cache(mixer, dtype, 16, 44, 2, 720)        # (the tokens' pages go back as the window passes)
    slot_r, slot_o = cache.open("r"), cache.open("o")
    outs, outs_other, at, oat = [], [], 0, 0
    for n, k in [(2, 0), (300, 50), (390, 1), (1, 1), (1, 0), (1, 40), (1, 1)] + [(1, 0)] * 4:
        entries = [("r", slot_r, cache.extend("r", n), n)] + ([("o", slot_o, cache.extend("o", k), k)] if k else [])
        _apply_tables(cache)
        rows = torch.cat([x[at:at + n]] + ([other[oat:oat + k]] if k else [])).cuda().contiguous()
        out = mixer.forward(rows, _two_cache_context(cache, entries))
        outs.append(out[:n]), outs_other.append(out[n:])
        cache.release_behind_window("r"), cache.release_behind_window("o")
        at, oat = at + n, oat + k
    assert at == T and int(cache.error_word) == 0
    got, got_other = torch.cat(outs).cpu().double(), torch.cat(outs_other).cpu().double()
    tol = 2e-5 if dtype == torch.float32 else BF16_REL
    assert (got - want).abs().max() <= tol * want.abs().max()
    assert (got_other - want_other[:oat]).abs().max() <= tol * want_other.abs().max()


def test_a_sink_takes_weight_and_gives_nothing():
    """Sinks set by hand: a head whose sink lies far above every score gives (nearly) nothing, one whose sink lies far
    below gives the plain softmax's sum; the first token of a sequence, which sees one key only, shows it most."""
    need_gpu()
    m = attention(2, 2, 8, 8, 6, 2, 0.4, rot_dims=8, base=10.0)
    mixer, w, starts = _direct_attention(m, torch.float32, seed=5)
    mixer.sink.copy_(torch.tensor([30.0, -30.0]))
    w["mix.sink"] = torch.tensor([30.0, -30.0], dtype=torch.float64)
    mixer.o_weight = type(mixer.o_weight)(torch.eye(16, device=CUDA), few_rows_tcgen05=None)
    w["mix.o"] = torch.eye(16, dtype=torch.float64)
    x = torch.randn(30, mixer.hidden_size, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).float()
    want = plain_tibalorn.attention_mixer(x.double(), w, "mix.", m, torch.arange(30))
    cache = _attention_cache(mixer, torch.float32, 4, 12, 1, 64)
    cache.open("r")
    got = _run_portions(mixer, cache, "r", x, [1, 12, 1, 16])
    assert (got - want).abs().max() <= 2e-5 * want.abs().max()
    assert got[:, :8].abs().max() < 1e-6 * got[:, 8:].abs().max()          # the first head's weight all went to its sink
    assert got[0, 8:].abs().max() > 0.01


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,vdim,state,groups,conv,parts", [(4, 8, 12, 2, 3, 2), (1, 6, 3, 1, 2, 1), (3, 16, 64, 3, 4, 3), (2, 34, 9, 1, 8, 1),
                                                                (6, 5, 7, 3, 1, 2), (8, 64, 128, 1, 4, 1)])
def test_state_space_mixer_alone_in_portions_over_its_state(dtype, heads, vdim, state, groups, conv, parts):
    """Portions that end just before, at and just after the kernels' runs of 16 and 64 tokens, portions shorter than the
    convolution's reach (its carried inputs then move along by less than their number), long ones (which the scan cuts
    into runs) beside single tokens and beside other long ones, single tokens; a slot used again starts from zero."""
    need_gpu()
    from torchinferno_b200.cache.manager import CacheManager
    from torchinferno_b200.parts.base import LayerContext, PartSpec, build_part
    W, eps = 48, 1e-5
    m = mamba2(heads, vdim, state, groups=groups, conv=conv, norm_groups=parts)
    mixer = build_part("mixer", PartSpec("state_space_duality", {
        "hidden_size": W, "heads": heads, "head_dim": vdim, "state_dim": state, "groups": groups, "taps": conv, "norm_groups": parts,
        "eps": eps}), dtype=dtype, device=CUDA)
    w = _random_weights(mixer, 4, dtype, "mix.")
    g = torch.Generator().manual_seed(state)
    plan = ((63, 0), (1, 7), (2, 0), (1, 1), (1, 2), (64, 1), (65, 0), (1, 64), (15, 3), (17, 0), (200, 2), (1, 0), (1, 8), (130, 70))
    T = sum(n for n, _ in plan)
    x = torch.randn(T, W, generator=g).to(torch.bfloat16).to(dtype)
    other = torch.randn(sum(k for _, k in plan), W, generator=g).to(torch.bfloat16).to(dtype)
    want = plain_tibalorn.mamba2_mixer(x.double(), w, "mix.", m, eps)
    want_other = plain_tibalorn.mamba2_mixer(other.double(), w, "mix.", m, eps)
    # the state a request leaves is what the next portion starts from: the last portion from a zero state differs
    assert (plain_tibalorn.mamba2_mixer(x.double()[T - 130:], w, "mix.", m, eps)[0] - want[T - 130]).abs().max() > 0.02 * want.abs().max()
    cache = CacheManager([], [mixer.state_spec()], page_size=4, num_pages=4, max_requests=2, max_request_tokens=10 ** 6,
                         dtype=dtype, device=CUDA)
    cache.open("warm"), cache.close("warm")
    slot_r, slot_o = cache.open("r"), cache.open("o")
    outs, outs_other, pos, opos = [], [], 0, 0
    for n, k in plan:
        entries = [("r", slot_r, pos, n)] + ([("o", slot_o, opos, k)] if k else [])
        rows = torch.cat([x[pos:pos + n]] + ([other[opos:opos + k]] if k else [])).cuda().contiguous()
        out = mixer.forward(rows, LayerContext(batch=_entries_batch(entries), state=cache.states[0]))
        outs.append(out[:n]), outs_other.append(out[n:])
        pos, opos = pos + n, opos + k
    got, got_other = torch.cat(outs).cpu().double(), torch.cat(outs_other).cpu().double()
    tol = 2e-5 if dtype == torch.float32 else BF16_REL
    assert (got - want).abs().max() <= tol * want.abs().max()
    assert (got_other - want_other).abs().max() <= tol * want_other.abs().max()
    cache.close("o")
    assert cache.open("n") == slot_o
    out = mixer.forward(other[:5].cuda().contiguous(), LayerContext(batch=_entries_batch([("n", slot_o, 0, 5)]), state=cache.states[0]))
    assert (out.cpu().double() - want_other[:5]).abs().max() <= tol * want_other.abs().max()


@pytest.mark.parametrize("cut", [False, True])
def test_the_scan_keeps_a_first_token_through_a_long_quiet_run_and_forgets_at_the_rate_it_is_given(cut):
    """Step sizes made by hand: the first token writes the state, the 500 that follow have steps of about 1e-9 (they
    neither write nor let it decay), in portions and single tokens.  A state that is reset, scaled or lost at a run's or
    a portion's edge shows in the last outputs.  A second head decays by a known factor per token.  ``cut``: the kernel
    is told the portions' lengths, so it cuts the long ones into runs that it walks side by side."""
    need_gpu()
    from torchinferno_b200.kernels import ops
    H, P, N, T = 2, 12, 10, 501
    g = torch.Generator().manual_seed(7)
    x, B, C = torch.randn(T, H, P, generator=g), torch.randn(T, 1, N, generator=g), torch.randn(T, 1, N, generator=g)
    raw = torch.full((T, H), -20.0)
    raw[0] = 3.0
    raw[:, 1] = 0.0                                            # the second head: softplus(0) = ln 2 at every token
    a_log, d_skip, dt_bias = torch.tensor([1.0, -1.0]), torch.tensor([0.0, 0.5]), torch.zeros(H)
    dt = plain_tibalorn.softplus(raw.double())
    want, S = plain_tibalorn.state_space_scan(x.double(), B.double(), C.double(), dt, a_log.double(), d_skip.double())
    quiet = torch.einsum("np,n->p", float(dt[0, 0]) * B[0, 0].double()[:, None] * x[0, 0].double()[None, :], C[T - 1, 0].double())
    assert (want[T - 1, 0] - quiet).abs().max() < 1e-5 * quiet.abs().max()      # the first token is all the first head has
    xbc = torch.cat([x.reshape(T, H * P), B.reshape(T, N), C.reshape(T, N)], dim=1).cuda().contiguous()
    state = torch.zeros(3, H * N * P + 5, device=CUDA)
    state[0], state[2] = 5.0, -3.0                             # (other slots' state must neither leak nor change)
    y = torch.empty(T, H * P, device=CUDA)
    at = 0
    for n in (1, 15, 16, 17, 63, 64, 129, 1, 1, 194):
        q_start = torch.tensor([0, n], dtype=torch.int32, device=CUDA)
        ops.ssd_scan(xbc[at:at + n], raw[at:at + n].cuda().contiguous(), 0, dt_bias.cuda(), a_log.cuda(), d_skip.cuda(), state, q_start,
                     torch.tensor([1], dtype=torch.int32, device=CUDA), y[at:at + n], 1, heads=H, groups=1, state_dim=N, head_dim=P,
                     max_q_len=n if cut else None)
        at += n
    assert at == T and (y.cpu().double() - want.reshape(T, H * P)).abs().max() <= 1e-5 * want.abs().max()
    assert (state[1, :H * N * P].cpu().double() - S.reshape(-1)).abs().max() <= 1e-5 * S.abs().max()
    assert float((state[0] - 5.0).abs().max()) == 0.0 and float((state[2] + 3.0).abs().max()) == 0.0
    assert float(state[1, H * N * P:].abs().max()) == 0.0      # what lies behind S in the slot is not the scan's


@pytest.mark.parametrize("taps", [1, 2, 3, 4, 8])
def test_short_convolution_carries_its_last_inputs_through_portions_of_any_length(taps):
    need_gpu()
    from torchinferno_b200.kernels import ops
    C, T = 37, 150
    g = torch.Generator().manual_seed(taps)
    u, weight, bias = torch.randn(T, C + 5, generator=g), torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    want = plain_tibalorn.silu(plain_tibalorn.short_convolution(u[:, 3:3 + C].double(), weight.double(), bias.double()))
    state = torch.zeros(2, 11 + (taps - 1) * C, device=CUDA)
    state[0] = 9.0
    out = torch.empty(T, C, device=CUDA)
    at = 0
    for n in (1, 1, 2, 1, 3, 5, 1, 64, 1, 2, 65, 4):
        q_start = torch.tensor([0, n], dtype=torch.int32, device=CUDA)
        ops.short_conv(u[at:at + n].cuda().contiguous(), 3, weight.cuda(), bias.cuda(), state, 11, q_start,
                       torch.tensor([1], dtype=torch.int32, device=CUDA), out[at:at + n], 1, n, silu=True)
        at += n
    assert at == T and (out.cpu().double() - want).abs().max() <= 1e-5
    assert float((state[0] - 9.0).abs().max()) == 0.0 and float(state[1, :11].abs().max()) == 0.0
    if taps > 1:
        assert torch.equal(state[1, 11:].cpu().view(taps - 1, C), u[T - taps + 1:, 3:3 + C])


@pytest.mark.parametrize("width,parts,rows", [(32, 2, 7), (30, 3, 9), (192, 1, 300), (4096, 8, 5), (6, 6, 3)])
def test_gate_then_norm_in_parts_and_the_small_row_kernels(width, parts, rows):
    need_gpu()
    from torchinferno_b200.kernels import ops
    g = torch.Generator().manual_seed(width + parts)
    y, z, weight = torch.randn(rows, width, generator=g) * 3, torch.randn(rows, width + 9, generator=g), torch.randn(width, generator=g)
    want = plain_tibalorn.group_rms(y.double() * plain_tibalorn.silu(z[:, 4:4 + width].double()), parts, 1e-5) * weight.double()
    out = torch.empty(rows, width, device=CUDA)
    ops.gated_group_norm(y.cuda(), z.cuda(), 4, weight.cuda(), 1e-5, out, parts)
    assert (out.cpu().double() - want).abs().max() <= 1e-5 * want.abs().max()
    # gate before norm is not norm before gate
    other = plain_tibalorn.group_rms(y.double(), parts, 1e-5) * plain_tibalorn.silu(z[:, 4:4 + width].double()) * weight.double()
    assert width // parts == 1 or (other - want).abs().max() > 0.05 * want.abs().max()
    h = torch.randn(rows, width, generator=g)
    for dtype in (torch.float32, torch.bfloat16):
        hd = h.to(dtype).cuda()
        got = ops.relu_squared(hd, torch.empty_like(hd))
        ref = torch.relu(h.to(dtype).double()).pow(2)
        assert (got.cpu().double() - ref).abs().max() <= (1e-6 if dtype == torch.float32 else 0.01) * ref.abs().max()
    logits = (torch.randn(rows, width, generator=g) * 40).cuda()
    ref = 30.0 * torch.tanh(logits.cpu().double() / 30.0)
    assert (ops.softcap_(logits, 30.0).cpu().double() - ref).abs().max() <= 1e-5


def test_the_feed_forward_squares_what_relu_leaves():
    need_gpu()
    from torchinferno_b200.parts.base import LayerContext, PartSpec, build_part
    for dtype in (torch.float32, torch.bfloat16):
        part = build_part("feed_forward", PartSpec("dense", {"hidden_size": 40, "intermediate_size": 24, "activation": "relu2",
                                                             "up_name": "up", "down_name": "down"}), dtype=dtype, device=CUDA)
        w = _random_weights(part, 6, dtype, "mlp.")
        x = torch.randn(11, 40, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).to(dtype)
        want = plain_tibalorn.feed_forward(x.double(), w, "mlp.")
        got = part.forward(x.cuda(), LayerContext(batch=_entries_batch([("r", 0, 0, 11)]))).cpu().double()
        assert (got - want).abs().max() <= (2e-5 if dtype == torch.float32 else BF16_REL) * want.abs().max()


# ------------------------------------------------ entry point and programs
def test_greedy_generation_through_the_engine_and_its_scheduler(folders):
    need_gpu()
    from torchinferno_b200.config.engine_config import EngineConfig
    from torchinferno_b200.engine.engine import InferenceEngine
    from torchinferno_b200.engine.types import GenerateRequest, SamplingConfig
    config, seed = CONFIGS["TA"]
    cfg, w = plain_tibalorn.read_model_folder(folders["TA"])
    prompts = list(requests_for(config, seed + 2, [5, 41, 1, 18, 66]).values())
    new = 30                                                # (decoding passes the window and completes blocks)
    for dtype in ("float32", "bfloat16"):
        with InferenceEngine.from_config(EngineConfig(model=str(folders["TA"]), dtype=dtype, page_size=8, max_batch_size=3,
                                                      prefill_chunk_size=16, max_num_batched_tokens=48, kv_cache_tokens=512)) as engine:
            outs = engine.generate_many([GenerateRequest(f"g{i}", prompt_token_ids=p, sampling=SamplingConfig(new))
                                         for i, p in enumerate(prompts)])
        for prompt, out in zip(prompts, outs):
            tokens = list(out.token_ids)
            assert len(tokens) == new
            logits = plain_tibalorn.forward(cfg, w, (prompt + tokens)[:-1])
            for i, tok in enumerate(tokens):
                row = logits[len(prompt) + i - 1]
                best = row.topk(2)
                if dtype == "float32" and float(best.values[0] - best.values[1]) > 1e-4 * float(row.abs().max()):
                    assert tok == int(best.indices[0])
                else:
                    assert tok in best.indices.tolist()


def test_the_trace_program_replays_a_tibalorn_folder(folders, tmp_path):
    need_gpu()
    import subprocess
    import sys
    config, seed = CONFIGS["TE"]
    requests = requests_for(config, seed + 3, [30, 75, 2])
    steps, index = replay_util.trace_mixed(requests, seed=3)
    out_dir = tmp_path / "out"
    cmd = [sys.executable, str(replay_util.ROOT / "bin" / "trace_run"), "--model", str(folders["TE"]), "--dtype", "float32",
           "--out", str(out_dir), "--max-tokens", str(replay_util.peak_tokens(steps))]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for step in steps:
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
            assert proc.stdout.readline().strip() == f"done {step['step']}"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    results = {}
    for step in steps:
        wanted = sum(len(e["want"]) for e in step["entries"])
        if wanted:
            results[step["step"]] = np.fromfile(out_dir / f"{step['step']}.f32", dtype="<f4").reshape(wanted, config["vocab"])
    compare(replay_util.gather(results, index), folders["TE"], requests, "float32", "TE trace program")


# ------------------------------------------------------- sizes drawn at random
def _random_config(rng):
    """A small Tibalorn configuration with sizes drawn from lists that mix multiples of 8, 16, 64 with odd ones."""
    pick = rng.choice
    layers = []
    for _ in range(pick([2, 3, 4])):
        mlp = pick([None, dense(pick([8, 24, 36, 70]))])
        if rng.random() < 0.4:
            heads = pick([1, 2, 3, 4, 6])
            groups = pick([g for g in (1, 2, 3) if heads % g == 0])
            vdim = pick([4, 5, 8, 16, 33])
            parts = pick([p for p in (1, 2, 3, heads) if (heads * vdim) % p == 0])
            layers.append({"type": "mamba2", "mixer": mamba2(heads, vdim, pick([1, 4, 9, 16, 40]), groups=groups,
                                                             conv=pick([1, 2, 4, 5]), norm_groups=parts), "mlp": mlp})
            continue
        kv_heads, dim = pick([1, 2, 3]), pick([4, 8, 24, 40])
        scaling = pick([None, (pick([2.0, 4.0, 16.0]), pick([16, 64, 4096]), pick([4.0, 32.0]), pick([0.5, 1.0, 2.0]))])
        layers.append({"type": "attention", "mlp": mlp, "mixer": attention(
            kv_heads * pick([1, 2, 4]), kv_heads, dim, pick([2, 6, 8, 20, 40]), pick([1, 3, 16, 50, 4096]), pick([1, 2, 5, 16, 64]),
            pick([0.1, 0.3]), pick([2, dim // 2, dim]) // 2 * 2 or 2, base=pick([100.0, 10000.0, 1e6]), scaling=scaling)})
    return {"architecture": "Tibalorn", "vocab": pick([50, 97, 128]), "width": pick([24, 40, 72, 96, 136]),
            "norm": {"eps": pick([1e-6, 1e-5])}, "embedding": {"scale": pick([1.0, 2.5, 6.0])},
            "logit_softcap": pick([None, 5.0, 30.0]), "layers": layers}


@pytest.mark.parametrize("draw", range(8))
def test_sizes_drawn_at_random(draw, tmp_path):
    """Whole prompts, portions and token-by-token decoding of models whose every size was drawn at random, in both
    number formats."""
    need_gpu()
    import random
    rng = random.Random(7300 + draw)
    config = _random_config(rng)
    write_model(config, tmp_path, seed=draw)
    requests = requests_for(config, 50 + draw, [41, 3, 70])
    for dtype in ("float32", "bfloat16"):
        for kind, (steps, index) in {"whole": replay_util.trace_whole(requests), "tail": replay_util.trace_tail_decode(requests, tail=12),
                                     "portions": replay_util.trace_portions(requests, sizes=(2, 31, 3, 33, 2, 16))}.items():
            runner = make_runner(tmp_path, dtype, replay_util.peak_tokens(steps), page_size=rng.choice([4, 16]))
            rows = replay_util.gather(run_steps(runner, steps), index)
            compare(rows, tmp_path, requests, dtype, f"draw {draw} {kind}")
