"""The Numuzen configuration on the CPU: registry, the model's description and tensor names, the rank
from a tensor's shape, refused configurations, cache groups and state, the frequency table, and the
plain implementation's own consistency (a recurrence in portions, a window query by query)."""
import copy
import math

import pytest
import torch

import numuzen_cases as cases
import plain_numuzen as plain
from torchlet_b200.config import NumuzenConfig, config_from_dict, known_architectures
from torchlet_b200.parts import LayeredModel, expected_tensors


def test_registered_and_chosen_by_name():
    assert "Numuzen" in known_architectures()
    config = config_from_dict(cases.CASES["P"])
    assert isinstance(config, NumuzenConfig)
    assert NumuzenConfig.from_dict(config.to_dict()) == config


def test_description_and_tensor_names():
    spec = cases.config_for("P").model_spec()
    assert [layer.block for layer in spec.layers] == ["sandwich"] * 4
    assert [layer.mixer.kind for layer in spec.layers] == ["gated_attention", "gated_linear_attention"] * 2
    assert spec.layers[2].feed_forward is None and len(spec.layers[2].norms) == 2
    names = {t.name: t.shape for t in expected_tensors(spec)}
    for name, shape in {"embed": (101, 96), "final.norm": (96,), "l0.norm1": (96,), "l0.norm1b": (96,), "l0.norm2b": (96,),
                        "l0.mix.q": (96, 96), "l0.mix.k": (48, 96), "l0.mix.q.norm": (96,), "l0.mix.k.norm": (48,),
                        "l0.mix.g": (96, 96), "l0.mix.o": (96, 96), "l0.mlp.router": (5, 96), "l0.mlp.e4.gate": (40, 96),
                        "l0.mlp.e0.down": (96, 40), "l1.mix.q": (36, 96), "l1.mix.v": (60, 96), "l1.mix.g": (60, 96),
                        "l1.mix.o": (96, 60), "l1.mix.norm": (20,), "l1.mix.a1": (6, 96), "l1.mix.a2": (36, 6),
                        "l1.mix.a2.b": (36,)}.items():
        assert names[name] == shape, name
    assert "l0.mix.v" not in names and "l2.norm2" not in names and "l2.mlp.router" not in names
    assert spec.tie_word_embeddings and spec.embedding_name == "embed"


def test_the_decay_rank_comes_from_the_shape():
    raw = copy.deepcopy(cases.CASES["P"])
    for layer in raw["layers"]:
        layer["mixer"].pop("decay_rank", None)
    config = NumuzenConfig.from_dict(raw)
    with pytest.raises(ValueError, match="decay rank"):
        config.model_spec()
    config = config.with_tensor_shapes({"l1.mix.a1": (6, 96), "l3.mix.a1": (5, 96), "l0.mix.q": (96, 96)})
    assert config.model_spec().layers[3].mixer.params["decay_rank"] == 5


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="conv"), "unknown type"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda c: c["layers"][0]["mixer"].update(vdim=8), "values are the keys"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unknown mlp kind"),
    (lambda c: c["layers"][1]["mixer"].pop("tau"), "lacks tau"),
    (lambda c: c.pop("width"), "lacks required keys"),
])
def test_refused_configurations(change, message):
    raw = copy.deepcopy(cases.CASES["P"])
    change(raw)
    with pytest.raises(ValueError, match=message):
        NumuzenConfig.from_dict(raw)


def test_cache_groups_and_state():
    model = LayeredModel(cases.config_for("P").model_spec())
    needs = model.cache_needs()
    assert [(n.kv.num_kv_heads, n.kv.head_dim, n.kv.window) if n.kv else None for n in needs] == \
        [(2, 24, 13), None, (2, 24, 37), None]
    assert [n.state.shape if n.state else None for n in needs] == [None, (3, 12, 20), None, (2, 24, 8)]
    from torchlet_b200.cache.storage import plan_groups

    groups, where = plan_groups(needs, 10)
    assert len(groups) == 2 and where == {0: (0, 0), 2: (1, 0)}  # two windows: two pools that free their pages apart


def test_frequency_table():
    from torchlet_b200.parts.rotary import scaled_frequencies

    for rot in ({"dims": 8, "base": 500.0, "scaling": cases.YARN}, {"dims": 16, "base": 100.0},
                {"dims": 64, "base": 1e6, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}):
        got, magnitude = scaled_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        want, want_magnitude = plain.rotation_frequencies(rot)
        assert torch.allclose(got, want, rtol=1e-12) and abs(magnitude - want_magnitude) < 1e-12
    f, m = plain.rotation_frequencies({"dims": 64, "base": 1e6, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}})
    plain_f = torch.tensor([1e6 ** (-2.0 * i / 64) for i in range(32)], dtype=torch.float64)
    assert torch.allclose(f[:5], plain_f[:5]) and torch.allclose(f[-5:], plain_f[-5:] / 8.0) and m == pytest.approx(0.1 * math.log(8) + 1)


def test_plain_recurrence_in_portions_and_plain_window():
    g = torch.Generator().manual_seed(3)
    q, k, a = (torch.rand(30, 6, generator=g, dtype=torch.float64) for _ in range(3))
    v = torch.rand(30, 4, generator=g, dtype=torch.float64)
    whole, _ = plain.linear_recurrence(q, k, v, a)
    first, state = plain.linear_recurrence(q[:11], k[:11], v[:11], a[:11])
    rest, _ = plain.linear_recurrence(q[11:], k[11:], v[11:], a[11:], state)
    assert torch.allclose(torch.cat([first, rest]), whole, rtol=1e-12)
    # closed form of one output: o_t = sum_s (prod_{s < r <= t} a_r * k_s) . q_t  v_s
    t = 7
    want = sum(((a[s + 1:t + 1].prod(dim=0) * k[s]) @ q[t]) * v[s] for s in range(t + 1))
    assert torch.allclose(whole[t], want, rtol=1e-12)
    # the window: query i sees exactly ``window`` keys, itself included, and the sink takes its share
    out = plain.sink_softmax_attention(torch.zeros(9, 2, dtype=torch.float64), torch.zeros(9, 2, dtype=torch.float64),
                                       torch.eye(9, dtype=torch.float64), 1.0, None, 3)
    assert torch.allclose(out[8], torch.tensor([0, 0, 0, 0, 0, 0, .25, .25, .25], dtype=torch.float64))
    assert torch.allclose(out[0], torch.tensor([.5, 0, 0, 0, 0, 0, 0, 0, 0], dtype=torch.float64))
