"""Small Vofidra configurations for the tests: sizes that differ from one another in every place, values that happen
to be 1 or equal to one another, both kinds of layer in several orders, every kind of feed-forward."""
from __future__ import annotations


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0, rot_dims=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
            "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}


def attention(heads, kv_heads, dim, vdim, scale, bias_max, buckets, coef=0.5, every=16):
    # ("buckets" is read for random weights only: a checkpoint's table says how many rows it has)
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max,
            "buckets": buckets, "q_temp": {"coef": coef, "every": every}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, identity, top, ff, count=1, keep=1):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": count, "keep": keep}}}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# two streams; grouped heads with values wider than keys; a bias table of 16 rows whose last distance (40) lies inside the
# prompts; a temperature that steps every 8 positions; experts in four groups of which two are kept, two of the eight
# router outputs without tensors; a latent layer first and last
VA = {
    "architecture": "Vofidra", "vocab": 101, "width": 64, "streams": 2, "norm": {"eps": 1e-5}, "logit_softcap": 8.0,
    "layers": [
        layer("latent_attention", latent(4, 8, 8, 12, 24, 20, 0.25, base=1000.0), dense(40)),
        layer("attention", attention(4, 2, 16, 24, 0.2, 40, 16, coef=0.3, every=8), moe(6, 2, 3, 20, count=4, keep=2)),
        layer("attention", attention(2, 2, 8, 8, 0.35, 9, 6, coef=1.0, every=1), dense(24)),
        layer("latent_attention", latent(2, 16, 4, 8, 12, 40, 0.2, base=50.0), moe(4, 0, 2, 12, count=2, keep=1)),
    ],
}
# one stream, one head, sizes that are no multiple of 8, an odd vocabulary, an attention first, a layer without
# feed-forward, every expert chosen, a single group, a last distance beyond any prompt, rotary on part of the rotated width
VB = {
    "architecture": "Vofidra", "vocab": 131, "width": 44, "streams": 1, "norm": {"eps": 1e-6}, "logit_softcap": 50.0,
    "layers": [
        layer("attention", attention(1, 1, 12, 20, 0.3, 5000, 32, coef=0.25, every=64), None),
        layer("latent_attention", latent(1, 6, 6, 20, 10, 7, 0.4, base=200000.0, rot_dims=4), moe(3, 0, 3, 6)),
        layer("attention", attention(3, 1, 6, 2, 0.4, 3, 2, coef=0.0, every=5), dense(8)),
    ],
}
# three streams; nothing is a multiple of 4: width 50, heads of 6 and 10, a latent of 14 + 2, a feed-forward of 9, a vocabulary
# of 53; as many experts without tensors as with; top 1
VC = {
    "architecture": "Vofidra", "vocab": 53, "width": 50, "streams": 3, "norm": {"eps": 1e-5}, "logit_softcap": 5.0,
    "layers": [
        layer("latent_attention", latent(3, 6, 2, 10, 14, 9, 0.4, base=300.0), moe(3, 3, 2, 9, count=3, keep=2)),
        layer("attention", attention(6, 3, 10, 6, 0.3, 21, 6, coef=0.7, every=3), moe(5, 1, 1, 3, count=2, keep=1)),
    ],
}
# four streams, only attention: six query heads on one key head, keys wider than values, a head of 40 (no multiple of 16),
# as many key heads as query heads, a table of two rows; no cap on the logits
VD = {
    "architecture": "Vofidra", "vocab": 97, "width": 96, "streams": 4, "norm": {"eps": 1e-5}, "logit_softcap": None,
    "layers": [
        layer("attention", attention(6, 1, 40, 16, 0.15, 200, 32, coef=0.5, every=32), dense(64)),
        layer("attention", attention(3, 3, 32, 32, 0.2, 2, 2, coef=2.0, every=50), moe(7, 1, 1, 16, count=2, keep=1)),
        layer("attention", attention(6, 1, 40, 16, 0.15, 33, 10, coef=0.1, every=2), None),
    ],
}
# only latent attention, with a latent of 64 + 16 (the shapes the tensor-core kernel takes) beside a small one
VE = {
    "architecture": "Vofidra", "vocab": 64, "width": 128, "streams": 2, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
    "layers": [
        layer("latent_attention", latent(8, 16, 16, 16, 64, 32, 0.18, base=10000.0), dense(48)),
        layer("latent_attention", latent(2, 8, 2, 4, 6, 3, 0.3, base=10.0), None),
        layer("latent_attention", latent(4, 32, 16, 24, 64, 48, 0.12, base=1e6), moe(10, 5, 4, 32, count=5, keep=3)),
    ],
}
CONFIGS = {"VA": (VA, 41), "VB": (VB, 42), "VC": (VC, 43), "VD": (VD, 44), "VE": (VE, 45)}


def write_model(config, folder, seed, embed_gain=40.0, head_gain=25.0):
    """A folder with random weights.  The table's rows are made ``embed_gain`` times the usual size, so that the tanh of
    the norms bends, and the head's ``head_gain`` times, so that the logits reach the range where their cap bends them."""
    from safetensors.torch import load_file, save_file
    from torchinferno_b200.weights.random_init import write_random_model
    folder = write_random_model(config, folder, seed)
    path = str(folder) + "/model.safetensors"
    tensors = load_file(path)
    tensors["embed"] = (tensors["embed"].float() * embed_gain).to(tensors["embed"].dtype)
    tensors["head"] = (tensors["head"].float() * head_gain).to(tensors["head"].dtype)
    save_file(tensors, path)
    return folder
