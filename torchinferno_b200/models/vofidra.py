"""Vofidra as a description made of parts.

The residual is carried in ``streams`` copies; every layer is a ``hyper_connection`` block: each sublayer reads the
streams through a weighted sum, norms it with a tanh norm (``tanh(alpha x) w + b``) and writes its output back through a
small matrix.  The mixer is an attention over a low-rank latent (``latent_attention``: queries through a latent of their
own, rotary pairs (i, i + dims / 2) on a key part all heads share, a sigmoid gate per head) or a grouped attention
without rotation (``biased_attention``: RMS-normed queries and keys, a query temperature, a learned bias per head and
distance bucket).  The feed-forward is a gated unit with SiLU, dense (``swiglu``) or routed (``routed_experts``: softmax
scores, a correction for the choice, groups of experts, experts that hand their input through), or absent.  The model's
norm reads the sum of the streams, and the logits pass c * tanh(. / c).  Tensor names: ``embed``, ``head``,
``final.norm`` (+ ``.b``, ``.alpha``), and per layer ``l<i>.norm1`` / ``norm2`` (+ ``.b``, ``.alpha``),
``l<i>.hc1.*`` / ``hc2.*``, ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from torchinferno_b200.config.registry import ArchitectureEntry, register_architecture
from torchinferno_b200.config.vofidra_config import MAX_POSITIONS, VofidraConfig, VofidraLayer
from torchinferno_b200.models.spec import BlockSpec, LayerCall, ModelSpec
from torchinferno_b200.parts.base import PartSpec

ROUTER_WEIGHT_EPS = 1e-20       # added to the sum of the chosen scores before they are divided by it


def _mixer(layer: VofidraLayer, config: VofidraConfig, buckets: int | None) -> PartSpec:
    m = layer.mixer
    if layer.type == "latent_attention":
        return PartSpec("latent_attention", {
            "hidden_size": config.width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "value_dim": m["vdim"],
            "kv_rank": m["kv_rank"], "q_rank": m["q_rank"], "scale": float(m["scale"]), "rot_base": float(m["rot"]["base"]),
            "rot_dims": m["rot"]["dims"], "pairing": "half", "eps": config.eps, "gate": "head"}, prefix="mix.")
    return PartSpec("biased_attention", {
        "hidden_size": config.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "value_dim": m["vdim"],
        "scale": float(m["scale"]), "buckets": buckets, "bias_max": m["bias_max"], "qk_norm_eps": config.eps,
        "temp_coef": float(m["q_temp"]["coef"]), "temp_every": m["q_temp"]["every"]}, prefix="mix.")


def _feed_forward(layer: VofidraLayer, config: VofidraConfig) -> PartSpec | None:
    mlp = layer.mlp
    if mlp is None:
        return None
    if mlp["kind"] == "dense":
        return PartSpec("swiglu", {"hidden_size": config.width, "intermediate_size": mlp["ff"], "gate_name": "gate",
                                   "up_name": "up", "down_name": "down"}, prefix="mlp.")
    router = mlp["router"]
    return PartSpec("routed_experts", {
        "hidden_size": config.width, "experts": router["experts"], "identity": router["identity"], "top": router["top"],
        "expert_size": mlp["expert"]["ff"], "activation": "swiglu", "scores": "softmax", "normalize": True,
        "norm_eps": ROUTER_WEIGHT_EPS, "correction": True, "groups": (router["groups"]["count"], router["groups"]["keep"])},
        prefix="mlp.")


def default_bias_rows(bias_max: int) -> int:
    """Rows of an attention layer's bias table when nothing else says (random weights; a checkpoint's own table decides
    for itself): the largest power of two up to 32 that ``bias_max`` still exceeds the half of."""
    rows = 2
    while rows * 2 <= 32 and rows < bias_max:
        rows *= 2
    return rows


def build_vofidra(config: VofidraConfig) -> ModelSpec:
    def norm(name: str, prefix: str = "") -> PartSpec:
        return PartSpec("tanh", {"width": config.width, "weight_name": name}, prefix=prefix)

    blocks, schedule = [], []
    for i, layer in enumerate(config.layers):
        buckets = None
        if layer.type == "attention":
            buckets = layer.mixer.get("buckets") or default_bias_rows(layer.mixer["bias_max"])
        feed_forward = _feed_forward(layer, config)
        block = PartSpec("hyper_connection", {
            "streams": config.streams, "mixer": _mixer(layer, config, buckets), "mixer_norm": norm("norm1"),
            "feed_forward": feed_forward, "feed_forward_norm": None if feed_forward is None else norm("norm2")})
        blocks.append(BlockSpec(block, f"l{i}."))
        schedule.append(LayerCall(i, i))         # every mixer keeps keys: a cache layer each
    return ModelSpec(
        architecture="Vofidra", hidden_size=config.width, vocab_size=config.vocab, max_positions=MAX_POSITIONS,
        embedding_name="embed", layers=tuple(blocks), schedule=tuple(schedule), final_norm=norm("norm", "final."),
        head_name="head", tie_head_to_embedding=False, config=config.to_dict(), logit_softcap=config.logit_softcap,
        streams=config.streams)


VOFIDRA = register_architecture(ArchitectureEntry(
    name="Vofidra", model_types=("vofidra",), config_class=VofidraConfig, build=build_vofidra))
