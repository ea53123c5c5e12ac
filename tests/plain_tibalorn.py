"""A plain, slow Tibalorn forward pass for the tests: whole sequences, no cache, one function per mechanism.

Tibalorn is a decoder-only design of pre-norm layers (layer norms with weight and bias) whose mixers are either a
Mamba-2 recurrence (a short causal convolution, then a state of N x P numbers per head that decays by a
data-dependent factor) or an attention over a sliding window plus one averaged key and value for every block of
tokens that lies wholly behind the window, with rotary positions on part of a head under a YaRN frequency law,
values that are rotated by their own position and turned back at the query's, a learned number per head in the
softmax's denominator, a temperature per head and an element-wise output gate.  The feed-forward is W_down relu(W_up
h)^2; the head is the embedding table, and the logits pass a tanh cap.  This file shares no code with
``torchinferno_b200``: it reads config.json and model.safetensors itself and computes on the CPU in float64, token by
token where the design is a recurrence, so that its own rounding does not count against the engine.

Notation: T tokens, W the model width, x the residual stream [T, W].
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
def layer_norm(x, w, name, eps):
    """(x - mean) / sqrt(mean((x - mean)^2) + eps) * weight + bias; the bias is the tensor ``name`` + '.b'."""
    mean = x.mean(dim=-1, keepdim=True)
    var = (x - mean).pow(2).mean(dim=-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * w[name] + w[name + ".b"]


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.clamp(x, min=0) + torch.log1p(torch.exp(-x.abs()))


def yarn_frequencies(dims, base, scaling):
    """(frequencies [dims / 2], amplitude).  Plain: base^(-2i / dims), amplitude 1.  With a scaling law (factor,
    original, fast, slow): d(t) = dims ln(original / (2 pi t)) / (2 ln base); lo = max(floor(d(fast)), 0),
    hi = min(ceil(d(slow)), dims - 1); r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1); the frequency is
    f_i / factor where r_i = 1, f_i where r_i = 0 and the blend between; amplitude 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=F)
    freq = torch.tensor(float(base), dtype=F) ** (-2 * i / dims)
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def d(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(d(float(scaling["fast"]))), 0)
    hi = min(math.ceil(d(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return freq / factor * ramp + freq * (1 - ramp), 0.1 * math.log(factor) + 1.0


def turn_halves(x, angle, dims, amplitude=1.0):
    """Turn the pairs (i, i + dims / 2) of the first ``dims`` elements of x [T, heads, d] by angle [T, dims / 2]:
    (u, v) -> (u cos - v sin, v cos + u sin), cos and sin times ``amplitude``; the rest pass unchanged."""
    half = dims // 2
    cos, sin = angle.cos()[:, None, :] * amplitude, angle.sin()[:, None, :] * amplitude
    lo, hi = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = lo * cos - hi * sin
    out[..., half:dims] = hi * cos + lo * sin
    return out


def value_angles(positions, vdim, base):
    m = torch.arange(vdim // 2, dtype=F)
    return positions.to(F)[:, None] * (torch.tensor(float(base), dtype=F) ** (-2 * m / vdim))[None, :]


# ------------------------------------------------------------------- mixers
def pooled_window_weights(scores_tokens, scores_blocks, positions, size, pool, sink):
    """Softmax over what each query sees, with ``sink`` [H] in the denominator.

    scores_tokens [H, T, T] (query i, key j), scores_blocks [H, T, B] (query i, block b of ``pool`` tokens).  Query i
    sees token j iff 0 <= i - j < size, and block b iff its last token b * pool + pool - 1 <= i - size.  Returns the
    weights of tokens [H, T, T] and of blocks [H, T, B]."""
    i = positions[:, None]
    see_tokens = (i - positions[None, :] >= 0) & (i - positions[None, :] < size)
    last = torch.arange(scores_blocks.shape[-1]) * pool + pool - 1
    see_blocks = last[None, :] <= i - size
    both = torch.cat([scores_tokens.masked_fill(~see_tokens, -math.inf), scores_blocks.masked_fill(~see_blocks, -math.inf)], dim=-1)
    top = torch.maximum(both.max(dim=-1).values, sink[:, None].expand(both.shape[:2]))
    e = torch.exp(both - top[..., None])
    weights = e / (e.sum(dim=-1) + torch.exp(sink[:, None] - top))[..., None]
    T = scores_tokens.shape[-1]
    return weights[..., :T], weights[..., T:]


def windowed_pooled_attention(q, k, v, positions, size, pool, factor, sink):
    """q [T, H, d] and k [T, G, d], v [T, G, dv] as a cache would hold them, of one sequence from its first token on.
    Block b is the mean of the keys (values) of positions b * pool .. b * pool + pool - 1; query head h reads key head
    h // (H / G); ``factor`` [H] multiplies the scores.  Returns the heads' sums [T, H, dv]."""
    T, H, G = q.shape[0], q.shape[1], k.shape[1]
    B = T // pool
    k_blocks = k[:B * pool].reshape(B, pool, G, k.shape[2]).mean(dim=1)
    v_blocks = v[:B * pool].reshape(B, pool, G, v.shape[2]).mean(dim=1)
    rep = H // G
    kh, vh = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    kbh, vbh = k_blocks.repeat_interleave(rep, dim=1), v_blocks.repeat_interleave(rep, dim=1)
    s_tokens = torch.einsum("ihd,jhd->hij", q, kh) * factor[:, None, None]
    s_blocks = torch.einsum("ihd,bhd->hib", q, kbh) * factor[:, None, None]
    p_tokens, p_blocks = pooled_window_weights(s_tokens, s_blocks, positions, size, pool, sink)
    return torch.einsum("hij,jhd->ihd", p_tokens, vh) + torch.einsum("hib,bhd->ihd", p_blocks, vbh)


def attention_mixer(h, w, prefix, m, positions):
    """h: [T, W] normed input of one sequence whose positions are 0 .. T - 1."""
    T, H, G, d, dv = h.shape[0], m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    rot, mask = m["rot"], m["mask"]
    q = (h @ w[prefix + "q"].T + w[prefix + "q.b"]).view(T, H, d)
    k = (h @ w[prefix + "k"].T + w[prefix + "k.b"]).view(T, G, d)
    v = (h @ w[prefix + "v"].T + w[prefix + "v.b"]).view(T, G, dv)
    freq, amplitude = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
    angle = positions.to(F)[:, None] * freq[None, :]
    q, k = turn_halves(q, angle, rot["dims"], amplitude), turn_halves(k, angle, rot["dims"], amplitude)
    turn = value_angles(positions, dv, rot["base"])
    v = turn_halves(v, turn, dv)                             # a value is kept turned by its own position
    out = windowed_pooled_attention(q, k, v, positions, mask["size"], mask["pool"], float(m["scale"]) * w[prefix + "temp"],
                                    w[prefix + "sink"])
    out = turn_halves(out, -turn, dv)                        # and the sum is turned back by the query's
    gate = torch.sigmoid(h @ w[prefix + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[prefix + "o"].T


def short_convolution(u, weight, bias):
    """Causal convolution per channel: out_t = bias + sum_k weight[:, k] u_(t - taps + 1 + k), zeros before the start."""
    T, taps = u.shape[0], weight.shape[1]
    padded = torch.cat([torch.zeros((taps - 1, u.shape[1]), dtype=u.dtype), u], dim=0)
    out = bias.expand(T, -1).clone()
    for k in range(taps):
        out = out + padded[k:k + T] * weight[:, k]
    return out


def group_rms(y, parts, eps):
    T, width = y.shape
    y = y.reshape(T, parts, width // parts)
    return (y / torch.sqrt(y.pow(2).mean(dim=-1, keepdim=True) + eps)).reshape(T, width)


def state_space_scan(x, B, C, dt, a_log, d_skip, start=None):
    """The recurrence alone, token by token.  x [T, H, P], B and C [T, G, N], dt [T, H] (already positive), per head
    (its group g = head // (H / G)) a state S [N, P] that starts at zero (or at ``start`` [H, N, P]):
    S_t = exp(-exp(a_log) dt_t) S_(t-1) + dt_t B_t x_t^T;   y_t = S_t^T C_t + d_skip x_t.  Returns (y [T, H, P], S)."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    decay = torch.exp(-torch.exp(a_log) * dt)
    S = torch.zeros((H, N, P), dtype=x.dtype) if start is None else start.clone()
    y = torch.empty((T, H, P), dtype=x.dtype)
    group = torch.arange(H) // (H // G)
    for t in range(T):
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * B[t][group][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, C[t][group]) + d_skip[:, None] * x[t]
    return y, S


def mamba2_mixer(h, w, prefix, m, eps):
    """[z | x | B | C | dt] = W_in h; x, B, C pass the convolution and silu; dt = softplus(dt + dt_bias); the scan; the
    heads side by side times silu(z), normed in ``norm_groups`` parts, times a weight, then W_o."""
    T, H, P, N, G = h.shape[0], m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w[prefix + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_convolution(xbc, w[prefix + "conv"], w[prefix + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    y, _ = state_space_scan(x, B, C, softplus(dt + w[prefix + "dt_bias"]), w[prefix + "A_log"], w[prefix + "D"])
    y = y.reshape(T, inner) * silu(z)
    return (group_rms(y, m["norm_groups"], eps) * w[prefix + "norm"]) @ w[prefix + "o"].T


def feed_forward(h, w, prefix):
    return torch.relu(h @ w[prefix + "up"].T).pow(2) @ w[prefix + "down"].T


# -------------------------------------------------------------------- model
def forward(config, w, tokens, keep_layers=False):
    """Logits [T, vocab] of one sequence (and, with ``keep_layers``, the residual stream after every layer)."""
    eps = float(config["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.shape[0])
    x = w["embed"][tokens] * float(config["embedding"]["scale"])
    kept = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = layer_norm(x, w, p + "norm1", eps)
        if layer["type"] == "attention":
            x = x + attention_mixer(h, w, p + "mix.", layer["mixer"], positions)
        elif layer["type"] == "mamba2":
            x = x + mamba2_mixer(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(f"unknown mixer {layer['type']!r}")
        if layer.get("mlp") is not None:
            x = x + feed_forward(layer_norm(x, w, p + "norm2", eps), w, p + "mlp.")
        kept.append(x.clone())
    logits = layer_norm(x, w, "final.norm", eps) @ w["embed"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = float(cap) * torch.tanh(logits / float(cap))
    return (logits, torch.stack(kept)) if keep_layers else logits
