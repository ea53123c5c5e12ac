"""Tibalorn as a description made of parts.

The embedding output is multiplied by a constant.  Every layer is a pre-norm block with layer norms (weight and
bias): x <- x + mixer(norm1(x)), then, where the layer has a feed-forward, x <- x + ff(norm2(x)).  The mixer is a
Mamba-2 recurrence (``state_space_duality``: a short causal convolution and a decaying state per request) or an
attention over a sliding window plus one averaged key and value per block of tokens that lies wholly behind the
window (``pooled_window_attention``: rotary positions under a YaRN law on part of a head, values rotated by their
position and turned back at the query's, a learned number per head in the softmax's denominator, a temperature per
head, an element-wise output gate).  The feed-forward is W_down relu(W_up h)^2.  The model's norm is a layer norm, the
head is the embedding table, and the logits pass c * tanh(. / c).  Tensor names: ``embed``, ``final.norm`` (+ ``.b``),
and per layer ``l<i>.norm1`` / ``norm2`` (+ ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.*``.
"""
from __future__ import annotations

from torchinferno_b200.config.registry import ArchitectureEntry, register_architecture
from torchinferno_b200.config.tibalorn_config import MAX_POSITIONS, TibalornConfig, TibalornLayer
from torchinferno_b200.models.spec import BlockSpec, LayerCall, ModelSpec
from torchinferno_b200.parts.base import PartSpec


def _mixer(layer: TibalornLayer, config: TibalornConfig) -> PartSpec:
    m = layer.mixer
    if layer.type == "mamba2":
        return PartSpec("state_space_duality", {
            "hidden_size": config.width, "heads": m["heads"], "head_dim": m["vdim"], "state_dim": m["state"],
            "groups": m["groups"], "taps": m["conv"], "norm_groups": m["norm_groups"], "eps": config.eps}, prefix="mix.")
    rot = m["rot"]
    scaling = rot.get("scaling")
    law = None if scaling is None else {
        "rope_type": "yarn", "factor": float(scaling["factor"]), "original": float(scaling["original"]),
        "fast": float(scaling["fast"]), "slow": float(scaling["slow"])}
    position = PartSpec("rotary", {"head_dim": m["dim"], "theta": float(rot["base"]), "rot_dim": rot["dims"], "scaling": law})
    return PartSpec("pooled_window_attention", {
        "hidden_size": config.width, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "value_dim": m["vdim"],
        "scale": float(m["scale"]), "position": position, "window": m["mask"]["size"], "pool": m["mask"]["pool"],
        "value_rotation_base": float(rot["base"]), "bias": True, "sink": True, "temperature": True, "gate": True},
        prefix="mix.")


def _feed_forward(layer: TibalornLayer, config: TibalornConfig) -> PartSpec | None:
    if layer.mlp is None:
        return None
    return PartSpec("dense", {"hidden_size": config.width, "intermediate_size": layer.mlp["ff"], "activation": "relu2",
                              "up_name": "up", "down_name": "down"}, prefix="mlp.")


def build_tibalorn(config: TibalornConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("layernorm", {"width": config.width, "eps": config.eps, "weight_name": name})

    blocks, schedule = [], []
    caches = 0
    for i, layer in enumerate(config.layers):
        feed_forward = _feed_forward(layer, config)
        block = PartSpec("prenorm", {
            "mixer": _mixer(layer, config), "mixer_norm": norm("norm1"), "feed_forward": feed_forward,
            "feed_forward_norm": None if feed_forward is None else norm("norm2")})
        blocks.append(BlockSpec(block, f"l{i}."))
        if layer.type == "attention":       # the tokens' keys and values, and beside them the blocks' averages
            schedule.append(LayerCall(i, caches, side_cache=caches + 1))
            caches += 2
        else:
            schedule.append(LayerCall(i, None))
    return ModelSpec(
        architecture="Tibalorn", hidden_size=config.width, vocab_size=config.vocab, max_positions=MAX_POSITIONS,
        embedding_name="embed", layers=tuple(blocks), schedule=tuple(schedule),
        final_norm=PartSpec("layernorm", {"width": config.width, "eps": config.eps, "weight_name": "norm"}, prefix="final."),
        head_name=None, tie_head_to_embedding=True, config=config.to_dict(),
        embedding_scale=config.embedding_scale, logit_softcap=config.logit_softcap)


TIBALORN = register_architecture(ArchitectureEntry(
    name="Tibalorn", model_types=("tibalorn",), config_class=TibalornConfig, build=build_tibalorn))
