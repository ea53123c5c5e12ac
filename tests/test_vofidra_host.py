"""Host-side tests of the Vofidra design: its configuration, its description made of parts, the tensors it expects,
and properties of the plain implementation the GPU tests compare with."""
import copy
import math

import pytest
import torch

import plain_vofidra
from vofidra_configs import CONFIGS, VA, VB, VC, VD, VE


def test_the_registry_resolves_the_design():
    from torchinferno_b200.config.registry import registered_architectures, resolve_architecture
    assert "Vofidra" in registered_architectures()
    assert resolve_architecture({"architecture": "Vofidra"}).name == "Vofidra"
    with pytest.raises(ValueError):
        resolve_architecture({"architecture": "Vofidra", "architectures": ["LlamaForCausalLM"]})


def test_config_errors_name_what_is_missing_or_wrong():
    from torchinferno_b200.config.model_config import ConfigError
    from torchinferno_b200.config.vofidra_config import VofidraConfig
    for config in (VA, VB, VC, VD, VE):
        VofidraConfig.from_dict(config)
    for path, value in ((("width",), None), (("streams",), None), (("streams",), 0), (("norm", "eps"), 0.0),
                        (("layers", 0, "type"), "conv"), (("layers", 0, "mixer", "q_rank"), None),
                        (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "rot", "dims"), 18),
                        (("layers", 0, "mixer", "scale"), None), (("layers", 1, "mixer", "kv_heads"), 3),
                        (("layers", 1, "mixer", "bias_max"), None), (("layers", 1, "mixer", "q_temp"), None),
                        (("layers", 1, "mixer", "q_temp", "every"), 0), (("layers", 1, "mlp", "router", "top"), 5),
                        (("layers", 1, "mlp", "router", "groups", "count"), 3), (("layers", 1, "mlp", "router", "groups", "keep"), 5),
                        (("layers", 1, "mlp", "router", "identity"), None), (("layers", 1, "mlp", "expert"), None),
                        (("layers", 0, "mlp", "kind"), "glu"), (("logit_softcap",), -1.0)):
        bad = copy.deepcopy(VA)
        node = bad
        for key in path[:-1]:
            node = node[key]
        if value is None:
            del node[path[-1]]
        else:
            node[path[-1]] = value
        with pytest.raises(ConfigError):
            VofidraConfig.from_dict(bad)


def test_the_description_names_streams_blocks_and_a_cache_layer_per_mixer():
    from torchinferno_b200.config.vofidra_config import VofidraConfig
    from torchinferno_b200.models.vofidra import build_vofidra, default_bias_rows
    spec = build_vofidra(VofidraConfig.from_dict(VA))
    assert spec.streams == 2 and spec.logit_softcap == 8.0 and spec.cache_layers == 4 and not spec.tie_head_to_embedding
    assert [(c.layer, c.cache, c.writes_cache) for c in spec.schedule] == [(i, i, True) for i in range(4)]
    assert all(layer.block.kind == "hyper_connection" and layer.block.params["streams"] == 2 for layer in spec.layers)
    assert [layer.block.params["mixer"].kind for layer in spec.layers] == ["latent_attention", "biased_attention", "biased_attention", "latent_attention"]
    assert spec.layers[1].block.params["feed_forward"].params["groups"] == (4, 2)
    assert build_vofidra(VofidraConfig.from_dict(VB)).layers[0].block.params["feed_forward"] is None
    assert build_vofidra(VofidraConfig.from_dict(VD)).logit_softcap is None
    assert [default_bias_rows(d) for d in (2, 3, 9, 17, 120, 5000)] == [2, 4, 16, 32, 32, 32]


def test_expected_tensors_and_requirements():
    from torchinferno_b200.weights.random_init import build_model
    model = build_model(VA, dtype=torch.float32, device="cpu")
    names = model.expected_tensors()
    assert names["l0.mix.dq"].shape == (20, 64) and names["l0.mix.dq.norm"].shape == (20,) and names["l0.mix.uq"].shape == (64, 20)
    assert names["l0.mix.dkv"].shape == (32, 64) and names["l0.mix.dkv.norm"].shape == (24,) and names["l0.mix.uk"].shape == (32, 24)
    assert names["l0.mix.uv"].shape == (48, 24) and names["l0.mix.g"].shape == (4, 64) and names["l0.mix.o"].shape == (64, 48)
    assert names["l1.mix.q"].shape == (64, 64) and names["l1.mix.k"].shape == (32, 64) and names["l1.mix.v"].shape == (48, 64)
    assert names["l1.mix.q.norm"].shape == (16,) and names["l1.mix.k.norm"].shape == (16,) and names["l1.mix.rel"].shape == (16, 4)
    assert names["l1.mix.rel"].free_dims == (0,) and names["l1.mix.o"].shape == (64, 96)
    assert names["l1.mlp.router"].shape == (8, 64) and names["l1.mlp.correction"].shape == (8,) and "l1.mlp.e6.up" not in names
    assert names["l1.mlp.e5.gate"].shape == (20, 64) and names["l1.mlp.e5.down"].shape == (64, 20)
    assert names["l0.mlp.gate"].shape == (40, 64) and names["l0.hc1.mix"].shape == (2, 2) and names["l3.hc2.in"].shape == (2,)
    assert names["l2.norm1.alpha"].shape == () and {"embed", "head", "final.norm", "final.norm.b", "final.norm.alpha"} <= set(names)
    single = build_model(VB, dtype=torch.float32, device="cpu").expected_tensors()
    assert "l0.norm2" not in single and "l0.hc2.in" not in single and single["l0.hc1.mix"].shape == (1, 1)
    caches, states = model.cache_requirements(), model.state_requirements()
    assert [(c.kv_heads, c.head_dim, c.value_width) for c in caches] == [(1, 32, 0), (2, 16, 24), (2, 8, 8), (1, 16, 0)]
    assert states == [None] * 4 and model.capturable()


def test_a_random_model_folder_holds_exactly_the_expected_tensors(tmp_path):
    from torchinferno_b200.weights.random_init import build_model, write_random_model
    write_random_model(VC, tmp_path, seed=3)
    config, weights = plain_vofidra.read_model_folder(tmp_path)
    assert set(weights) == set(build_model(VC, dtype=torch.float32, device="cpu").expected_tensors())
    assert config["layers"] == VC["layers"]
    assert float((weights["l1.norm1"] - 1).abs().max()) > 0.01 and float(weights["l1.norm1.b"].abs().max()) > 0.01
    mix = weights["l0.hc1.mix"]
    assert mix.shape == (3, 3) and float((mix - torch.eye(3)).abs().max()) > 0.01 and float(mix.diagonal().min()) > 0.3


def test_a_file_may_size_a_dimension_that_the_description_leaves_free(tmp_path):
    """The loader compares shapes except in the dimensions a part leaves to the file, and only there."""
    from safetensors.torch import load_file, save_file
    from torchinferno_b200.weights.loader import WeightError, load_weights
    from torchinferno_b200.weights.random_init import build_model, write_random_model
    config = copy.deepcopy(VD)
    write_random_model(config, tmp_path, seed=1)
    path = str(tmp_path / "model.safetensors")
    tensors = load_file(path)
    tensors["l0.mix.rel"] = torch.randn(12, 6).to(torch.bfloat16)          # (the description says 32 rows)
    save_file(tensors, path)
    model = build_model(config, dtype=torch.float32, device="cpu")
    load_weights(model, tmp_path)
    assert model.blocks[0].mixer.buckets == 12 and model.blocks[0].mixer.bias_by_distance.shape == (6, 201)
    tensors["l0.mix.rel"] = torch.randn(12, 5).to(torch.bfloat16)          # (heads are not the file's to say)
    save_file(tensors, path)
    with pytest.raises(WeightError):
        load_weights(build_model(config, dtype=torch.float32, device="cpu"), tmp_path)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_plain_implementation_is_causal(name, tmp_path):
    from vofidra_configs import write_model
    config, seed = CONFIGS[name]
    write_model(config, tmp_path, seed=seed)
    cfg, w = plain_vofidra.read_model_folder(tmp_path)
    tokens = torch.randint(0, cfg["vocab"], (53,)).tolist()
    whole, layers = plain_vofidra.forward(cfg, w, tokens, return_layers=True)
    assert torch.isfinite(whole).all() and whole.abs().max() > 1.0 and layers.shape[:2] == (len(cfg["layers"]), 53)
    assert torch.allclose(plain_vofidra.forward(cfg, w, tokens[:19]), whole[:19], atol=1e-12, rtol=1e-10)
    if cfg.get("logit_softcap"):
        assert whole.abs().max() < cfg["logit_softcap"]


def test_plain_mechanisms_against_closed_forms():
    g = torch.Generator().manual_seed(5)
    # streams: one stream with unit coefficients is the ordinary residual sum; the mix matrix is indexed [from, to]
    x = torch.randn(1, 4, 3, generator=g, dtype=torch.float64)
    y = torch.randn(4, 3, generator=g, dtype=torch.float64)
    one = torch.ones(1, dtype=torch.float64)
    assert torch.equal(plain_vofidra.write_streams(x, one.view(1, 1), one, y), x + y)
    x = torch.randn(2, 4, 3, generator=g, dtype=torch.float64)
    mix = torch.tensor([[1.0, 5.0], [0.0, 1.0]], dtype=torch.float64)       # stream 0 feeds stream 1, not the other way
    new = plain_vofidra.write_streams(x, mix, torch.zeros(2, dtype=torch.float64), y)
    assert torch.allclose(new[0], x[0]) and torch.allclose(new[1], 5 * x[0] + x[1])
    assert torch.allclose(plain_vofidra.read_streams(x, torch.tensor([2.0, -1.0], dtype=torch.float64)), 2 * x[0] - x[1])
    # the tanh norm takes no statistic of the row: a row and its double differ, and a large entry saturates at weight + bias
    w = {"n": torch.full((3,), 2.0, dtype=torch.float64), "n.b": torch.full((3,), 0.5, dtype=torch.float64),
         "n.alpha": torch.tensor(0.5, dtype=torch.float64)}
    row = torch.tensor([[0.2, -1.0, 400.0]], dtype=torch.float64)
    out = plain_vofidra.tanh_norm(row, w, "n")
    assert abs(float(out[0, 2]) - 2.5) < 1e-12 and abs(float(out[0, 0]) - (2 * math.tanh(0.1) + 0.5)) < 1e-12
    assert not torch.allclose(plain_vofidra.tanh_norm(2 * row, w, "n"), out)
    # pairs (i, i + dims / 2): with dims 4 of 6, elements 0 and 2 turn together, 4 and 5 pass
    v = torch.tensor([[[1.0, 0.0, 0.0, 0.0, 7.0, 9.0]]], dtype=torch.float64)
    turned = plain_vofidra.turn_halves(v, torch.tensor([3]), 4, 100.0)[0, 0]
    assert torch.allclose(turned, torch.tensor([math.cos(3.0), 0.0, math.sin(3.0), 0.0, 7.0, 9.0], dtype=torch.float64))
    slow = plain_vofidra.turn_halves(torch.tensor([[[0.0, 1.0, 0.0, 0.0]]], dtype=torch.float64), torch.tensor([5]), 4, 100.0)[0, 0]
    assert torch.allclose(slow, torch.tensor([0.0, math.cos(0.5), 0.0, math.sin(0.5)], dtype=torch.float64))
    # distance rows: one each below half the table, logarithmic steps beyond, the last from the last distance on
    assert [plain_vofidra.distance_bucket(n, 8, 64) for n in (0, 3, 4, 7, 8, 15, 16, 31, 32, 63, 64, 1000)] == [0, 3, 4, 4, 5, 5, 6, 6, 7, 7, 7, 7]
    # the temperature steps every `every` positions, counted from position every - 1
    temps = plain_vofidra.query_temperature(torch.arange(9), 0.5, 4)
    assert torch.allclose(temps, torch.tensor([1.0] * 3 + [1 + 0.5 * math.log(2)] * 4 + [1 + 0.5 * math.log(3)] * 2, dtype=torch.float64))
    # routing: a dropped group's outputs cannot be chosen even when every corrected score that is kept is negative; weights are made
    # from the scores without the correction; outputs past the experts hand the input through
    router = {"experts": 2, "identity": 2, "top": 2, "groups": {"count": 2, "keep": 1}}
    w = {"r.router": torch.tensor([[1.0], [0.0], [3.0], [-9.0]], dtype=torch.float64),
         "r.correction": torch.tensor([-5.0, -5.0, -9.0, -9.0], dtype=torch.float64)}
    ids, weights = plain_vofidra.route(torch.ones(1, 1, dtype=torch.float64), w, "r.", router)
    scores = torch.softmax(torch.tensor([1.0, 0.0, 3.0, -9.0], dtype=torch.float64), dim=0)
    assert ids.tolist() == [[0, 1]] and torch.allclose(weights[0], scores[:2] / scores[:2].sum())
    w["r.correction"] = torch.tensor([0.0, 0.0, 0.0, 0.8], dtype=torch.float64)       # the correction moves the choice, not the weight
    ids, weights = plain_vofidra.route(torch.ones(1, 1, dtype=torch.float64), w, "r.", dict(router, groups={"count": 1, "keep": 1}))
    assert ids.tolist() == [[2, 3]] and torch.allclose(weights[0], scores[2:] / scores[2:].sum())
    h = torch.randn(1, 1, generator=g, dtype=torch.float64)
    w.update({"r.router": torch.zeros(4, 1, dtype=torch.float64), "r.correction": torch.tensor([0.0, 0.0, 1.0, 1.0], dtype=torch.float64)})
    out = plain_vofidra.routed_units(h, w, "r.", {"router": dict(router, groups={"count": 1, "keep": 1})})
    assert torch.allclose(out, h)                                                     # two identity outputs of weight 1/2 each
