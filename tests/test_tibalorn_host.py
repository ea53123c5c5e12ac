"""Host-side tests of the Tibalorn design: its configuration, its description made of parts, the tensors it expects,
the cache manager's strided groups, the frequency law, and properties of the plain implementation the GPU tests
compare with."""
import copy
import math

import pytest
import torch

import plain_tibalorn
from tibalorn_configs import CONFIGS, TA, TB, TC, TD, TE, write_model


def test_the_registry_resolves_the_design():
    from torchinferno_b200.config.registry import registered_architectures, resolve_architecture
    assert "Tibalorn" in registered_architectures()
    assert resolve_architecture({"architecture": "Tibalorn"}).name == "Tibalorn"
    with pytest.raises(ValueError):
        resolve_architecture({"architecture": "Tibalorn", "architectures": ["LlamaForCausalLM"]})


def test_config_errors_name_what_is_missing_or_wrong():
    from torchinferno_b200.config.model_config import ConfigError
    from torchinferno_b200.config.tibalorn_config import TibalornConfig
    for config in (TA, TB, TC, TD, TE):
        TibalornConfig.from_dict(config)
    for path, value in ((("width",), None), (("embedding",), None), (("norm", "eps"), 0.0), (("layers", 0, "type"), "conv"),
                        (("logit_softcap",), None), (("logit_softcap",), -1.0),
                        (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mixer", "rot", "dims"), 18),
                        (("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "mask"), None),
                        (("layers", 0, "mixer", "mask", "pool"), 0), (("layers", 0, "mixer", "mask", "size"), None),
                        (("layers", 0, "mixer", "vdim"), 7), (("layers", 0, "mixer", "scale"), None),
                        (("layers", 0, "mixer", "rot", "scaling", "factor"), None),
                        (("layers", 0, "mlp", "kind"), "moe"), (("layers", 0, "mlp", "ff"), None),
                        (("layers", 1, "mixer", "groups"), 3), (("layers", 1, "mixer", "norm_groups"), 5),
                        (("layers", 1, "mixer", "state"), 0), (("layers", 1, "mixer", "conv"), None)):
        bad = copy.deepcopy(TA)
        node = bad
        for key in path[:-1]:
            node = node[key]
        if value is None:
            del node[path[-1]]
        else:
            node[path[-1]] = value
        with pytest.raises(ConfigError):
            TibalornConfig.from_dict(bad)
    assert TibalornConfig.from_dict(TD).logit_softcap is None       # (present and null: no cap)


def test_the_schedule_gives_attentions_two_caches_and_recurrences_state():
    from torchinferno_b200.config.tibalorn_config import TibalornConfig
    from torchinferno_b200.models.tibalorn import build_tibalorn
    spec = build_tibalorn(TibalornConfig.from_dict(TA))
    assert [(c.layer, c.cache, c.side_cache) for c in spec.schedule] == [(0, 0, 1), (1, None, None), (2, 2, 3), (3, None, None)]
    assert spec.cache_layers == 4 and spec.embedding_scale == 4.0 and spec.logit_softcap == 8.0 and spec.tie_head_to_embedding
    assert build_tibalorn(TibalornConfig.from_dict(TC)).cache_layers == 0
    assert build_tibalorn(TibalornConfig.from_dict(TD)).logit_softcap is None


def test_expected_tensors_and_requirements():
    from torchinferno_b200.weights.random_init import build_model
    model = build_model(TA, dtype=torch.float32, device="cpu")
    names = model.expected_tensors()
    assert names["l0.mix.q"].shape == (64, 64) and names["l0.mix.k"].shape == (32, 64) and names["l0.mix.v"].shape == (48, 64)
    assert names["l0.mix.g"].shape == (96, 64) and names["l0.mix.o"].shape == (64, 96) and names["l0.mix.v.b"].shape == (48,)
    assert names["l0.mix.temp"].shape == (4,) and names["l0.mix.sink"].shape == (4,)
    assert names["l1.mix.in"].shape == (2 * 32 + 2 * 2 * 12 + 4, 64) and names["l1.mix.conv"].shape == (32 + 48, 3)
    assert names["l1.mix.conv.b"].shape == (80,) and names["l1.mix.norm"].shape == (32,) and names["l1.mix.o"].shape == (64, 32)
    assert names["l1.mix.A_log"].shape == names["l1.mix.D"].shape == names["l1.mix.dt_bias"].shape == (4,)
    assert names["l1.mlp.up"].shape == (24, 64) and names["l1.mlp.down"].shape == (64, 24)
    assert "l2.norm2" not in names and "l2.mlp.up" not in names and "l3.norm2.b" not in names and "head" not in names
    assert {"embed", "final.norm", "final.norm.b", "l0.norm2.b", "l3.norm1"} <= set(names)
    caches, states = model.cache_requirements(), model.state_requirements()
    assert [(c.kv_heads, c.head_dim, c.value_width, c.window, c.stride) for c in caches] == \
        [(2, 16, 24, 20, 1), (2, 16, 24, None, 6), (2, 8, 8, 7, 1), (2, 8, 8, None, 3)]
    assert [None if s is None else s.shape for s in states] == [None, (4 * 12 * 8 + 2 * 80,), None, (2 * 5 * 20 + 3 * 50,)]
    assert model.capturable()
    # a block longer than the window keeps its own tokens until it is complete
    model = build_model(TB, dtype=torch.float32, device="cpu")
    assert [(c.window, c.stride) for c in model.cache_requirements()] == [(16, 1), (None, 1), (4, 1), (None, 4), (33, 1), (None, 33)]


def test_a_random_model_folder_holds_exactly_the_expected_tensors(tmp_path):
    from torchinferno_b200.weights.random_init import build_model
    write_model(TB, tmp_path, seed=3)
    config, weights = plain_tibalorn.read_model_folder(tmp_path)
    assert set(weights) == set(build_model(TB, dtype=torch.float32, device="cpu").expected_tensors())
    assert config["layers"] == TB["layers"]
    assert float((weights["l1.norm1"] - 1).abs().max()) > 0.01 and float(weights["l1.norm1.b"].abs().max()) > 0.01
    assert float((weights["l1.mix.temp"] - 1).abs().max()) > 0.01 and float(weights["l1.mix.sink"].abs().max()) > 0.01


def test_a_strided_group_takes_its_pages_as_blocks_complete():
    from torchinferno_b200.cache.manager import CacheManager, OutOfPages
    from torchinferno_b200.parts.base import CacheSpec
    specs = [CacheSpec(2, 8, 10, 12), CacheSpec(2, 8, None, 12, stride=6)]
    cache = CacheManager(specs, [None], page_size=4, num_pages=12, max_requests=2, max_request_tokens=48, dtype=torch.float32,
                         device="cpu")
    assert len(cache.groups) == 2 and cache.groups[1].allocator.num_pages == 12 // 6 + 2
    assert cache.kv_binding(1).keys.shape == (4, 2, 4, 8) and cache.kv_binding(1).values.shape == (4, 2, 4, 12)
    cache.open("a")
    assert cache.pages_needed("a", 5) == [2, 0] and cache.pages_needed("a", 6) == [2, 1] and cache.pages_needed("a", 30) == [8, 2]
    cache.extend("a", 5)
    assert [sum(p >= 0 for p in cache.block_table("a", g)) for g in (0, 1)] == [2, 0]
    cache.extend("a", 1)                        # the sixth token completes block 0
    assert [sum(p >= 0 for p in cache.block_table("a", g)) for g in (0, 1)] == [2, 1]
    cache.extend("a", 23)                       # 29 tokens: 4 whole blocks still fit the first page of the strided group
    assert sum(p >= 0 for p in cache.block_table("a", 1)) == 1
    cache.extend("a", 1)                        # 30 tokens: the fifth block opens the second page
    assert sum(p >= 0 for p in cache.block_table("a", 1)) == 2
    assert cache.release_behind_window("a") == 5        # the next query reads keys 21 ..: pages 0 to 4 of the windowed group go
    assert sum(p >= 0 for p in cache.block_table("a", 0)) == 3 and sum(p >= 0 for p in cache.block_table("a", 1)) == 2
    cache.audit()
    cache.open("b")
    with pytest.raises(OutOfPages):
        cache.extend("b", 40)                   # ten pages of tokens are not free: nothing changes
    assert cache.length("b") == 0
    cache.audit()
    cache.close("a"), cache.close("b")
    assert cache.free_pages() == [12, 4]
    cache.audit()


def test_the_frequency_law_of_the_rotary_part():
    from torchinferno_b200.parts.rope import rotary_amplitude, rotary_frequencies
    for dims, base, law in ((16, 1e6, (2.0, 2048, 32.0, 1.0)), (8, 1000.0, (4.0, 64, 8.0, 1.0)), (6, 100.0, (8.0, 32, 2.0, 1.0)),
                            (2, 10000.0, (3.0, 40, 4.0, 2.0)), (40, 10000.0, (2.0, 128, 32.0, 1.0))):
        factor, original, fast, slow = law
        mine = rotary_frequencies(dims, base, {"rope_type": "yarn", "factor": factor, "original": original, "fast": fast, "slow": slow})
        plain, amplitude = plain_tibalorn.yarn_frequencies(dims, base, {"factor": factor, "original": original, "fast": fast, "slow": slow})
        assert torch.allclose(mine.double(), plain, rtol=1e-6, atol=0)
        assert rotary_amplitude({"rope_type": "yarn", "factor": factor}) == pytest.approx(amplitude) == pytest.approx(0.1 * math.log(factor) + 1)
        # by hand: pairs that turn more than `fast` times over `original` positions keep their frequency, those that
        # turn less than `slow` times are divided by the factor
        plain_f = base ** (-2 * torch.arange(dims // 2, dtype=torch.float64) / dims)
        turns = original * plain_f / (2 * math.pi)
        for i in range(dims // 2):
            d = dims * math.log(original / (2 * math.pi * float(turns[i]))) / (2 * math.log(base))
            assert abs(d - i) < 1e-9
            if i <= max(math.floor(dims * math.log(original / (2 * math.pi * fast)) / (2 * math.log(base))), 0):
                assert float(plain[i]) == pytest.approx(float(plain_f[i]))
            if i >= min(math.ceil(dims * math.log(original / (2 * math.pi * slow)) / (2 * math.log(base))), dims - 1) and \
                    i > max(math.floor(dims * math.log(original / (2 * math.pi * fast)) / (2 * math.log(base))), 0):
                assert float(plain[i]) == pytest.approx(float(plain_f[i]) / factor)
    assert rotary_amplitude(None) == 1.0
    assert torch.allclose(rotary_frequencies(8, 100.0, None).double(), 100.0 ** (-torch.arange(4, dtype=torch.float64) / 4), rtol=1e-6)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_the_plain_implementation_is_causal(name, tmp_path):
    config, seed = CONFIGS[name]
    write_model(config, tmp_path, seed=seed)
    cfg, w = plain_tibalorn.read_model_folder(tmp_path)
    tokens = torch.randint(0, cfg["vocab"], (53,)).tolist()
    whole = plain_tibalorn.forward(cfg, w, tokens)
    assert torch.isfinite(whole).all() and whole.abs().max() > 1.0
    cap = cfg["logit_softcap"]
    assert cap is None or whole.abs().max() < cap
    assert torch.allclose(plain_tibalorn.forward(cfg, w, tokens[:19]), whole[:19], atol=1e-12, rtol=1e-10)


def test_plain_mechanisms_against_closed_forms():
    g = torch.Generator().manual_seed(5)
    # what a query sees: with a window of 4 and blocks of 3, query 9 sees tokens 6 .. 9 and the blocks that end at or
    # before position 5, i.e. blocks 0 and 1; query 8 sees tokens 5 .. 8 and block 0 only (block 1 ends at 5 > 8 - 4)
    pos = torch.arange(12)
    zeros, none = torch.zeros(1, 12, 12, dtype=torch.float64), torch.tensor([-math.inf], dtype=torch.float64)
    wt, wb = plain_tibalorn.pooled_window_weights(zeros, zeros[..., :4], pos, 4, 3, none)
    assert (wt[0, 9] > 0).tolist() == [False] * 6 + [True] * 4 + [False] * 2 and (wb[0, 9] > 0).tolist() == [True, True, False, False]
    assert (wt[0, 8] > 0).tolist() == [False] * 5 + [True] * 4 + [False] * 3 and (wb[0, 8] > 0).tolist() == [True, False, False, False]
    assert (wt[0, 2] > 0).tolist() == [True] * 3 + [False] * 9 and not (wb[0, 5] > 0).any() and (wb[0, 6] > 0).tolist() == [True, False, False, False]
    assert float(wt[0, 9].sum() + wb[0, 9].sum()) == pytest.approx(1.0) and float(wt[0, 9, 9]) == pytest.approx(1 / 6)
    # a sink equal to the scores counts as one more key that gives nothing
    wt, wb = plain_tibalorn.pooled_window_weights(zeros, zeros[..., :4], pos, 4, 3, torch.zeros(1, dtype=torch.float64))
    assert float(wt[0, 9, 9]) == pytest.approx(1 / 7) and float(wt[0, 0, 0]) == pytest.approx(1 / 2)
    # a value turned by its position and the sum turned back: the weight of key j then multiplies the value turned by j - i
    v = torch.randn(5, 1, 6, generator=g).double()
    turn = plain_tibalorn.value_angles(torch.arange(5), 6, 100.0)
    kept = plain_tibalorn.turn_halves(v, turn, 6)
    back = plain_tibalorn.turn_halves(kept[1:2].expand(5, 1, 6).contiguous(), -turn, 6)
    rel = plain_tibalorn.value_angles(1 - torch.arange(5), 6, 100.0)
    assert torch.allclose(back, plain_tibalorn.turn_halves(v[1:2].expand(5, 1, 6).contiguous(), rel, 6), atol=1e-12)
    assert float(turn[3, 1]) == pytest.approx(3 * 100.0 ** (-2 / 6))
    # the recurrence against its closed sum: S_t = sum_s dt_s B_s x_s^T prod_(s < r <= t) a_r
    T, H, P, N = 7, 2, 3, 4
    x, B, C = torch.randn(T, H, P, generator=g).double(), torch.randn(T, 2, N, generator=g).double(), torch.randn(T, 2, N, generator=g).double()
    dt, a_log, skip = torch.rand(T, H, generator=g).double(), torch.randn(H, generator=g).double(), torch.randn(H, generator=g).double()
    y, S = plain_tibalorn.state_space_scan(x, B, C, dt, a_log, skip)
    a = torch.exp(-torch.exp(a_log) * dt)
    for h in range(H):
        for t in (0, 3, 6):
            closed = sum(dt[s, h] * torch.prod(a[s + 1:t + 1, h]) * B[s, h][:, None] * x[s, h][None, :] for s in range(t + 1))
            assert torch.allclose(y[t, h], closed.T @ C[t, h] + skip[h] * x[t, h], atol=1e-12)
        assert torch.allclose(S[h], closed, atol=1e-12)
    # the convolution's last column is the current token's, and there are zeros before the start
    u, wgt, b = torch.randn(6, 2, generator=g).double(), torch.randn(2, 3, generator=g).double(), torch.randn(2, generator=g).double()
    out = plain_tibalorn.short_convolution(u, wgt, b)
    assert torch.allclose(out[0], b + wgt[:, 2] * u[0]) and torch.allclose(out[4], b + wgt[:, 0] * u[2] + wgt[:, 1] * u[3] + wgt[:, 2] * u[4])
    # the norm in parts: each part by its own root mean square
    row = torch.tensor([[3.0, 4.0, 0.0, 10.0]], dtype=torch.float64)
    assert torch.allclose(plain_tibalorn.group_rms(row, 2, 0.0), torch.tensor([[3 / math.sqrt(12.5), 4 / math.sqrt(12.5), 0.0, math.sqrt(2.0)]],
                                                                                dtype=torch.float64))
    assert torch.allclose(plain_tibalorn.feed_forward(torch.tensor([[1.0, -2.0]], dtype=torch.float64),
                                                      {"up": torch.eye(2, dtype=torch.float64) * 3, "down": torch.ones(1, 2, dtype=torch.float64)}, ""),
                          torch.tensor([[9.0]], dtype=torch.float64))
