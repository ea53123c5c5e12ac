"""A plain, slow Vofidra forward pass for the tests: whole sequences, no cache, one function per mechanism.

Vofidra is a decoder-only design whose residual is carried in several streams that every sublayer reads through one
weighted sum and writes back through a small mixing matrix; whose norm is tanh(alpha x) w + b; whose mixers are an
attention over a low-rank latent (queries through a latent of their own, one rotated key part shared by all heads,
a sigmoid gate per head) or a grouped attention without rotation (RMS-normed queries and keys, a query temperature
that grows with the logarithm of the position, and a learned bias per head and distance bucket); whose feed-forward
is a gated unit, dense or routed (softmax scores, a correction that only steers the choice, groups of experts of
which the best are kept, experts that hand their input through unchanged); and whose logits pass a tanh cap.  This
file shares no code with ``torchinferno_b200``: it reads config.json and model.safetensors itself and computes on the
CPU in float64, so that its own rounding does not count against the engine.

Notation: T tokens, W the model width, S streams, x the streams [S, T, W].
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

F = torch.float64


def read_model_folder(folder, dtype=F):
    from safetensors import safe_open
    folder = Path(folder)
    config = json.loads((folder / "config.json").read_text())
    weights = {}
    with safe_open(str(folder / "model.safetensors"), framework="pt", device="cpu") as handle:
        for name in handle.keys():
            t = handle.get_tensor(name)
            weights[name] = t.to(dtype) if t.is_floating_point() else t
    return config, weights


# ------------------------------------------------------------- small pieces
def tanh_norm(x, w, name):
    """tanh(alpha x) * weight + bias, element by element: no statistic of the row enters.  ``name`` + '.alpha' is a scalar, ``name`` + '.b' the bias."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def rms_norm(x, weight, eps):
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight


def silu(x):
    return x * torch.sigmoid(x)


def turn_halves(x, positions, dims, base):
    """Turn the pairs (i, i + dims / 2) of the first ``dims`` elements of x [T, heads, d] by position * base^(-2i / dims):
    (u, v) -> (u cos - v sin, v cos + u sin); the rest pass unchanged."""
    half = dims // 2
    freq = torch.tensor(float(base), dtype=F) ** (-2 * torch.arange(half, dtype=F) / dims)
    angle = positions.to(F)[:, None] * freq[None, :]
    cos, sin = angle.cos()[:, None, :], angle.sin()[:, None, :]
    lo, hi = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = lo * cos - hi * sin
    out[..., half:dims] = hi * cos + lo * sin
    return out


def causal_softmax(scores):
    """scores [H, T, T] (query i, key j) -> weights with j <= i only."""
    T = scores.shape[-1]
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    return torch.softmax(scores.masked_fill(~mask, -math.inf), dim=-1)


# ---------------------------------------------------------------- streams
def read_streams(x, into):
    """u = sum_s into[s] x_s."""
    return torch.einsum("s,stw->tw", into, x)


def write_streams(x, mix, out, y):
    """x_t <- sum_s mix[s, t] x_s + out[t] y, every stream from the values before the write."""
    return torch.einsum("st,snw->tnw", mix, x) + out[:, None, None] * y[None]


# ------------------------------------------------------------------- mixers
def latent_attention(h, w, p, m, positions, eps):
    """Attention over a latent: c_q = rms(W_dq h), q = W_uq c_q laid out per head as [dim plain ; rot_dim rotated];
    W_dkv h gives the latent c (first kv_rank rows, RMS-normed) and one rotated key part for all heads; head j's plain
    key is W_uk_j c and its value W_uv_j c; the head's sum is multiplied by sigmoid(W_g h)_j."""
    T, H, d, r, dv, rank = h.shape[0], m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, d + r)
    dkv = h @ w[p + "dkv"].T
    c = rms_norm(dkv[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = turn_halves(dkv[:, None, rank:], positions, m["rot"]["dims"], m["rot"]["base"])      # [T, 1, r]
    q_rot = turn_halves(q[..., d:], positions, m["rot"]["dims"], m["rot"]["base"])
    k_plain = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    scores = (torch.einsum("ihd,jhd->hij", q[..., :d], k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot[:, 0])) * m["scale"]
    heads = torch.einsum("hij,jhd->ihd", causal_softmax(scores), v)
    gate = torch.sigmoid(h @ w[p + "g"].T)                                                        # [T, H]
    return (heads * gate[..., None]).reshape(T, H * dv) @ w[p + "o"].T


def distance_bucket(n, buckets, far):
    """n for n < buckets / 2, else min(buckets - 1, buckets / 2 + floor(ln(n / half) / ln(far / half) * (buckets - half)))."""
    half = buckets // 2
    if n < half:
        return n
    return min(buckets - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (buckets - half))))


def query_temperature(positions, coef, every):
    """1 + coef * ln(floor((p + 1) / every) + 1)."""
    return 1.0 + coef * torch.log(torch.floor((positions.to(F) + 1) / every) + 1)


def biased_attention(h, w, p, m, positions, eps):
    """Grouped attention without rotation: per-head RMS norm of q and k (one weight for all heads), q times the
    temperature of its position, score = q . k * scale + rel[bucket(i - j), head], causal softmax."""
    T, H, G, d, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ w[p + "q"].T).view(T, H, d), w[p + "q.norm"], eps)
    k = rms_norm((h @ w[p + "k"].T).view(T, G, d), w[p + "k.norm"], eps)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    q = q * query_temperature(positions, m["q_temp"]["coef"], m["q_temp"]["every"])[:, None, None]
    rel = w[p + "rel"]                                                                            # [buckets, H]
    kh, vh = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kh) * m["scale"]
    distance = (positions[:, None] - positions[None, :]).clamp(min=0)                             # [T, T]; j > i is masked anyway
    row_of = torch.tensor([distance_bucket(n, rel.shape[0], m["bias_max"]) for n in range(int(distance.max()) + 1)])
    bias = rel[row_of[distance]].permute(2, 0, 1)                                                 # [H, T, T]
    heads = torch.einsum("hij,jhd->ihd", causal_softmax(scores + bias), vh)
    return heads.reshape(T, H * dv) @ w[p + "o"].T


# ------------------------------------------------------------ feed-forward
def gated_unit(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p, router, gaps=None):
    """(ids [T, top], weights [T, top]): softmax scores over experts and identity experts; the choice adds the correction
    and is made among the members of the ``keep`` best of ``count`` equal runs of adjacent outputs (a run ranks by its best corrected score);
    the weights are the chosen scores without the correction, divided by their sum + 1e-20.  ``gaps`` (a list) receives
    per token the smallest margin by which a choice was made: between the last group kept and the first one dropped, and
    between the last output chosen and the first one left."""
    n = router["experts"] + router["identity"]
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"]
    count, keep = router["groups"]["count"], router["groups"]["keep"]
    group_score = choice.view(-1, count, n // count).max(dim=-1).values
    ranked = group_score.sort(dim=-1, descending=True)
    kept = torch.zeros_like(group_score, dtype=torch.bool)
    kept.scatter_(1, ranked.indices[:, :keep], True)
    choice = choice.masked_fill(~kept.repeat_interleave(n // count, dim=1), -math.inf)
    order = choice.sort(dim=-1, descending=True)
    ids = order.indices[:, :router["top"]]
    if gaps is not None:
        for t in range(h.shape[0]):
            margin = math.inf
            if keep < count:
                margin = float(ranked.values[t, keep - 1] - ranked.values[t, keep])
            if router["top"] < n and order.values[t, router["top"]] > -math.inf:
                margin = min(margin, float(order.values[t, router["top"] - 1] - order.values[t, router["top"]]))
            gaps.append(margin)
    chosen = s.gather(1, ids)
    return ids, chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20)


def routed_units(h, w, p, mlp, gaps=None):
    router = mlp["router"]
    ids, weights = route(h, w, p, router, gaps)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), weights[t]):
            out[t] += a * (h[t] if e >= router["experts"] else gated_unit(h[t:t + 1], w, f"{p}e{e}.")[0])
    return out


# -------------------------------------------------------------------- model
def forward(config, w, tokens, return_layers=False, gaps=None):
    """Logits [T, vocab] of one sequence from its first token (and the sum of the streams after every layer).  ``gaps`` (a
    list of one list per token) receives the margins of every router's choice for that token."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    eps, S = config["norm"]["eps"], config["streams"]
    x = w["embed"][tokens][None].repeat(S, 1, 1)
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        u = tanh_norm(read_streams(x, w[p + "hc1.in"]), w, p + "norm1")
        mixer = latent_attention if layer["type"] == "latent_attention" else biased_attention
        x = write_streams(x, w[p + "hc1.mix"], w[p + "hc1.out"], mixer(u, w, p + "mix.", layer["mixer"], positions, eps))
        if layer["mlp"] is not None:
            u = tanh_norm(read_streams(x, w[p + "hc2.in"]), w, p + "norm2")
            margins = [] if gaps is not None else None
            y = gated_unit(u, w, p + "mlp.") if layer["mlp"]["kind"] == "dense" else routed_units(u, w, p + "mlp.", layer["mlp"], margins)
            for t, margin in enumerate(margins or []):
                gaps[t].append(margin)
            x = write_streams(x, w[p + "hc2.mix"], w[p + "hc2.out"], y)
        after.append(x.sum(dim=0))
    logits = tanh_norm(x.sum(dim=0), w, "final.norm") @ w["head"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(after)) if return_layers else logits
