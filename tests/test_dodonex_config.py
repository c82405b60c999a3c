"""The Dodonex configuration and what the framework makes of it, without a GPU: registry,
model description, tensor names, sizes taken from tensor shapes, cache groups; and the plain
implementation against itself (a recurrence in portions, a window of visible keys)."""
import copy
import json

import pytest
import torch

import dodonex_cases as cases
import plain_dodonex as plain


def test_registry_takes_the_architecture_name_as_a_plain_string(tmp_path):
    from torchlet_b200.config import DodonexConfig, architecture_name, config_from_dict, load_config

    raw = cases.CASES["P"]
    assert architecture_name(raw) == "Dodonex"
    assert architecture_name({"architectures": ["Qwen2ForCausalLM"], "architecture": "Dodonex"}) == "Qwen2ForCausalLM"
    with pytest.raises(ValueError):
        architecture_name({"vocab": 3})
    config = config_from_dict(raw)
    assert isinstance(config, DodonexConfig)
    (tmp_path / "config.json").write_text(json.dumps(config.to_dict()))
    assert load_config(tmp_path) == config


def test_model_description_follows_the_layer_list():
    config = cases.config_for("P")
    spec = config.model_spec()
    assert [l.mixer.kind for l in spec.layers] == ["general_delta", "latent_attention", "latent_attention",
                                                    "general_delta", "latent_attention"]
    assert [e.cache_from for e in spec.schedule] == [None, None, 1, None, 1]
    assert spec.layers[2].feed_forward is None and spec.layers[1].feed_forward.kind == "clamped_glu"
    assert all(l.block == "parallel_scaled" and l.block_params == {"residual_mult": 0.6} for l in spec.layers)
    assert [l.token_input.params["offset"] for l in spec.layers] == [0, 8, 16, 24, 32]
    assert spec.embedding_scale == 5.0 and spec.logit_scale == 1.5 and spec.tie_word_embeddings
    assert spec.final_norm.params["groups"] == 3
    assert spec.layers[1].mixer.params["rot_dims"] == 4 and not spec.layers[4].mixer.params["own_kv"]
    assert cases.config_for("Q").model_spec().layers[0].token_input is None


def test_tensor_names_and_shapes():
    from torchlet_b200.parts import expected_tensors

    names = {t.name: tuple(t.shape) for t in expected_tensors(cases.config_for("P").model_spec()) if not t.optional}
    assert names["embed"] == (97, 96) and names["side.embed"] == (97, 40) and names["final.norm"] == (96,)
    assert names["l0.mix.w1"] == (6, 96) and names["l0.mix.w2"] == (48, 6) and names["l0.mix.a.b"] == (48,)
    assert names["l1.mix.dkv"] == (48, 96) and names["l1.mix.uq"] == (72, 24) and names["l1.mix.uv"] == (72, 40)
    assert "l2.mix.dkv" not in names and "l2.mix.dkv.norm" not in names and "l2.mlp.gate" not in names
    assert names["l4.mix.o"] == (96, 16) and names["l3.side.proj"] == (96, 8) and names["l0.norm1"] == (96,)
    assert len(names) == len(set(names))


def test_decay_rank_comes_from_the_tensor_shape():
    from torchlet_b200.config import DodonexConfig

    raw = copy.deepcopy(cases.CASES["Q"])
    del raw["layers"][1]["mixer"]["decay_rank"]
    config = DodonexConfig.from_dict(raw)
    with pytest.raises(ValueError, match="decay rank"):
        config.model_spec()
    config = config.with_tensor_shapes({"l1.mix.w1": (3, 64), "l0.mix.uk": (12, 22)})
    assert config.model_spec().layers[1].mixer.params["decay_rank"] == 3


@pytest.mark.parametrize("change,message", [
    (lambda r: r["layers"][2]["mixer"].update(kv_from=2), "earlier layer"),
    (lambda r: r["layers"][2]["mixer"].update(kv_from=0), "cache of its own"),
    (lambda r: r["layers"][4]["mixer"].update(kv_rank=48), "differs from layer"),
    (lambda r: r["layers"][0].update(type="other"), "unknown type"),
    (lambda r: r["norm"].update(groups=5), "divisible"),
    (lambda r: r["layers"][1]["mlp"].pop("limit"), "lacks"),
])
def test_configurations_that_are_refused(change, message):
    from torchlet_b200.config import DodonexConfig

    raw = copy.deepcopy(cases.CASES["P"])
    change(raw)
    with pytest.raises(ValueError, match=message):
        DodonexConfig.from_dict(raw)


def test_cache_groups_of_one_plane_and_states():
    from torchlet_b200.cache.storage import plan_groups
    from torchlet_b200.parts import LayeredModel

    model = LayeredModel(cases.config_for("Q").model_spec())
    needs = model.cache_needs()
    assert [n.kv.head_dim if n.kv else None for n in needs] == [28, None, 20]
    assert needs[1].state.shape == (1, 20, 20) and needs[1].state.dtype == "float32"
    groups, where = plan_groups(needs, 10)
    assert [(g.num_kv_heads, g.head_dim, g.planes) for g in groups] == [(1, 28, 1), (1, 20, 1)]
    needs = LayeredModel(cases.config_for("P").model_spec()).cache_needs()
    assert [n.owner for n in needs] == [0, 1, 1, 3, 1]
    groups, where = plan_groups(needs, 10)
    assert len(groups) == 1 and groups[0].entries == (1,)


def test_plain_delta_rule_in_portions_equals_the_whole():
    H, D, W = 2, 12, 20
    g = torch.Generator().manual_seed(0)
    shapes = {"r": (H * D, W), "k": (H * D, W), "v": (H * D, W), "g": (H * D, W), "a": (H * D, W), "a.b": (H * D,),
              "w1": (4, W), "w2": (H * D, 4), "w0": (H * D,), "norm": (H * D,), "o": (W, H * D)}
    w = {"m." + n: torch.randn(*s, generator=g, dtype=torch.float64) * 0.4 for n, s in shapes.items()}
    h = torch.randn(30, W, generator=g, dtype=torch.float64)
    mixer = {"heads": H, "dim": D}
    whole, final = plain.general_delta(h, w, "m.", mixer, 1e-5)
    a, state = plain.general_delta(h[:11], w, "m.", mixer, 1e-5)
    b, state = plain.general_delta(h[11:13], w, "m.", mixer, 1e-5, state)
    c, state = plain.general_delta(h[13:], w, "m.", mixer, 1e-5, state)
    assert torch.allclose(torch.cat([a, b, c]), whole, atol=1e-12) and torch.allclose(state, final, atol=1e-12)
    # the removal term reads the OLD state: with a = 1 and w = 1 a repeated key overwrites its value
    S = torch.zeros(1, 3, 3, dtype=torch.float64)
    u = torch.tensor([[0.0, 1.0, 0.0]], dtype=torch.float64)
    for value in (torch.tensor([[1.0, 2.0, 3.0]]), torch.tensor([[-4.0, 0.5, 9.0]])):
        seen = torch.einsum("hi,hij->hj", u, S)
        S = S - u[:, :, None] * seen[:, None, :] + u[:, :, None] * value.double()[:, None, :]
    assert torch.allclose(torch.einsum("hij,hi->hj", S, u), torch.tensor([[-4.0, 0.5, 9.0]], dtype=torch.float64))


def test_plain_rotation_and_group_norm():
    x = torch.arange(12, dtype=torch.float64).reshape(1, 12) + 1
    y = plain.group_rms_norm(x, torch.ones(12, dtype=torch.float64), 0.0, 3)
    assert torch.allclose(y.reshape(3, 4).pow(2).mean(-1), torch.ones(3, dtype=torch.float64))
    v = torch.tensor([[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]], dtype=torch.float64)
    r = plain.rotate_half_pairs(v, torch.tensor([3]), 100.0, 4)  # entries 0,1 pair with 2,3; 4,5 pass
    assert torch.equal(r[0, 4:], v[0, 4:])
    a0, a1 = 3.0, 3.0 * 100.0 ** (-0.5)
    import math
    assert abs(r[0, 0] - (1 * math.cos(a0) - 3 * math.sin(a0))) < 1e-12
    assert abs(r[0, 3] - (4 * math.cos(a1) + 2 * math.sin(a1))) < 1e-12
    assert torch.allclose(plain.rotate_half_pairs(v, torch.tensor([0]), 100.0, 4), v)
