"""Small Tibalorn configurations for the tests: sizes that differ from one another in every place, values that happen
to be 1 or equal to one another, both kinds of layer in several orders, windows and blocks of many sizes."""
from __future__ import annotations


def attention(heads, kv_heads, dim, vdim, size, pool, scale, rot_dims, base=10000.0, scaling=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling is not None:
        factor, original, fast, slow = scaling
        rot["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": {"size": size, "pool": pool}, "rot": rot}


def mamba2(heads, vdim, state, groups=1, conv=4, norm_groups=1):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


# grouped heads, values wider than keys, rotary on half a head under a scaling law whose ramp covers some pairs only,
# a window of 20 with blocks of 6 (neither divides the pages used), a recurrence with two groups and two norm parts
# between two attentions of different masks, a feed-forward after a recurrence and none after an attention
TA = {
    "architecture": "Tibalorn", "vocab": 101, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 4.0},
    "logit_softcap": 8.0,
    "layers": [
        layer("attention", attention(4, 2, 16, 24, 20, 6, 0.2, 8, base=1000.0, scaling=(4.0, 64, 8.0, 1.0)), dense(40)),
        layer("mamba2", mamba2(4, 8, 12, groups=2, conv=3, norm_groups=2), dense(24)),
        layer("attention", attention(2, 2, 8, 8, 7, 3, 0.35, 8, base=50.0, scaling=(2.0, 16, 4.0, 0.5)), None),
        layer("mamba2", mamba2(2, 20, 5, conv=4), None),
    ],
}
# one head, sizes that are no multiple of 8, an odd vocabulary, a recurrence first, no scaling law, blocks of one token
# (every token behind the window is seen again as its own block), a window of one token, blocks longer than the window
TB = {
    "architecture": "Tibalorn", "vocab": 131, "width": 44, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0},
    "logit_softcap": 50.0,
    "layers": [
        layer("mamba2", mamba2(1, 6, 3, conv=2), None),
        layer("attention", attention(1, 1, 12, 20, 16, 1, 0.5, 12, base=200000.0), dense(20)),
        layer("attention", attention(1, 1, 12, 20, 1, 4, 0.4, 2), dense(8)),
        layer("attention", attention(3, 1, 6, 2, 5, 33, 0.3, 6, base=100.0, scaling=(8.0, 32, 2.0, 1.0)), None),
    ],
}
# only state, no keys at all: as many groups as heads, a convolution of one tap (nothing carried) and one of eight,
# a norm part per head
TC = {
    "architecture": "Tibalorn", "vocab": 60, "width": 40, "norm": {"eps": 1e-6}, "embedding": {"scale": 3.0},
    "logit_softcap": 15.0,
    "layers": [
        layer("mamba2", mamba2(3, 8, 16, groups=3, conv=1, norm_groups=3), dense(12)),
        layer("mamba2", mamba2(2, 34, 9, groups=1, conv=8, norm_groups=1), None),
    ],
}
# only attention: six query heads on one key head, keys wider than values, a head of 40 (no multiple of 16), a window
# longer than any prompt of the tests (no block is ever seen) beside a window of 2 with blocks of 2; no cap on the logits
TD = {
    "architecture": "Tibalorn", "vocab": 97, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 5.0},
    "logit_softcap": None,
    "layers": [
        layer("attention", attention(6, 1, 40, 16, 1000, 16, 0.15, 40, scaling=(2.0, 128, 32.0, 1.0)), dense(64)),
        layer("attention", attention(3, 3, 32, 32, 2, 2, 0.2, 32, base=100.0), dense(8)),
        layer("attention", attention(6, 1, 40, 16, 33, 10, 0.15, 20), None),
    ],
}
# nothing is a multiple of 4: width 50, heads of 6 and 10, a state of 7 with heads of 5, a feed-forward of 9, a vocabulary of 53
TE = {
    "architecture": "Tibalorn", "vocab": 53, "width": 50, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
    "logit_softcap": 5.0,
    "layers": [
        layer("attention", attention(3, 3, 6, 10, 9, 5, 0.4, 2), dense(9)),
        layer("mamba2", mamba2(6, 5, 7, groups=3, conv=5, norm_groups=2), dense(3)),
        layer("attention", attention(6, 3, 6, 10, 21, 7, 0.4, 6, base=300.0, scaling=(3.0, 40, 4.0, 2.0)), None),
    ],
}
CONFIGS = {"TA": (TA, 31), "TB": (TB, 32), "TC": (TC, 33), "TD": (TD, 34), "TE": (TE, 35)}


def write_model(config, folder, seed, embed_gain=12.0):
    """A folder with random weights.  The table's rows, which are also the head's, are made ``embed_gain`` times the
    usual size, so that the logits reach the range where their cap bends them."""
    from safetensors.torch import load_file, save_file
    from torchinferno_b200.weights.random_init import write_random_model
    folder = write_random_model(config, folder, seed)
    path = str(folder) + "/model.safetensors"
    tensors = load_file(path)
    tensors["embed"] = (tensors["embed"].float() * embed_gain).to(tensors["embed"].dtype)
    save_file(tensors, path)
    return folder
