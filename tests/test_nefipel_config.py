"""Nefipel on the CPU: its config.json reader, the tensors it asks for, and properties of the plain
implementation's own mechanisms that the tests on the GPU lean on."""
import copy

import pytest
import torch

import plain_nefipel as plain
import tiny_nefipel as tiny
from vosti_b200.config import ConfigError, model_spec_from_config, model_spec_from_dir
from vosti_b200.models import expected_weights
from vosti_b200.weights import check_tensors
from vosti_b200.weights.loader import WeightError


def test_spec_kinds_sizes_and_names():
    spec = model_spec_from_config(tiny.A)
    assert spec.architecture == "Nefipel" and spec.hidden_size == 72 and spec.vocab_size == 211
    assert spec.tie_word_embeddings and spec.embedding["scale"] == 3.3 and spec.embedding["out_dtype"] == "float32"
    assert all(layer.arrangement == "post_norm_stream" and layer.mixer.kind == "sink_attention" and layer.norm["alpha"] == 1.7
               for layer in spec.layers)
    assert [layer.mixer.get("maps", 1) for layer in spec.layers] == [2, 1, 1, 2]
    first, second = spec.layers[0].mixer, spec.layers[1].mixer
    assert first["diff"] == 0.2 and first["position"]["interleaved"] and not first.get("qkv_bias") and not first.get("out_gate")
    assert second["qkv_bias"] and second["out_gate"] and not second["position"]["interleaved"]
    assert first["position"]["scaling"] == ("yarn", 3.0, 48.0, 4.0, 1.0) and spec.layers[2].mixer["position"]["scaling"] is None
    assert second["position"]["rotary_dim"] == 8 and second["head_norm_eps"] == 2e-6
    ff = spec.layers[0].feed_forward
    assert (ff.kind, ff["experts"], ff["identity"], ff["groups"], ff["keep"], ff["top"], ff["shared"], ff["activation"]) == \
        ("moe", 6, 3, 3, 2, 3, 36, "relu2")
    last = spec.layers[3].feed_forward
    assert (last["identity"], last["groups"], last["keep"], last["shared"]) == (0, 1, 1, 0)
    assert spec.layers[1].feed_forward.kind == "swiglu" and spec.layers[1].feed_forward["activation"] == "relu"
    assert spec.layers[2].feed_forward is None
    assert model_spec_from_config(tiny.B).embedding["scale"] == 1.0
    names = expected_weights(spec)
    for name, shape in {"embed": (211, 72), "final.norm": (72,), "l0.norm1": (72,), "l0.norm2": (72,),
                        "l0.mix.q": (3 * 2 * 10, 72), "l0.mix.k": (1 * 2 * 10, 72), "l0.mix.v": (14, 72), "l0.mix.o": (72, 42),
                        "l0.mix.q.norm": (10,), "l0.mix.lk2": (10,), "l0.mlp.router": (9, 72), "l0.mlp.correction": (9,),
                        "l0.mlp.e5.up": (20, 72), "l0.mlp.e5.down": (72, 20), "l0.mlp.shared.up": (36, 72),
                        "l0.mlp.shared.down": (72, 36), "l0.mlp.shared.sg": (1, 72),
                        "l1.mix.q": (96, 72), "l1.mix.q.b": (96,), "l1.mix.k.b": (48,), "l1.mix.v.b": (32,), "l1.mix.k.norm": (24,),
                        "l1.mix.g": (64, 72), "l1.mix.o": (72, 64), "l1.mlp.gate": (100, 72), "l1.mlp.down": (72, 100),
                        "l3.mlp.router": (5, 72)}.items():
        assert tuple(names[name].shape) == shape, name
    for absent in ("head", "l0.mix.q.b", "l0.mix.g", "l1.mix.lq1", "l0.mlp.e6.up", "l3.mlp.shared.up", "l2.mlp.gate", "l0.mlp.e0.gate"):
        assert absent not in names, absent
    assert sorted(n for n, w in names.items() if w.optional) == ["l2.norm2"]


def test_checkpoints_with_and_without_unused_tensors_load():
    for unused in (True, False):
        spec, tensors = tiny.tensors_for(tiny.A, 5, unused)
        check_tensors(tensors, expected_weights(spec))
    spec, tensors = tiny.tensors_for(tiny.A, 5)
    del tensors["l0.mlp.correction"]
    with pytest.raises(WeightError) as error:
        check_tensors(tensors, expected_weights(spec))
    assert error.value.missing == ["l0.mlp.correction"]


def test_config_errors_name_the_key():
    for path, message in ((("layers", 0, "mixer", "diff"), "diff"), (("norm",), "norm"), (("postln_alpha",), "postln_alpha"),
                          (("layers", 1, "mixer", "rot", "base"), "base"), (("layers", 0, "mixer", "rot", "scaling", "slow"), "slow"),
                          (("layers", 0, "mlp", "router", "top"), "top"), (("layers", 0, "mlp", "expert"), "expert"),
                          (("layers", 1, "mixer", "kv_heads"), "kv_heads"), (("layers", 0, "mlp", "router", "groups", "keep"), "keep")):
        config = copy.deepcopy(tiny.A)
        block = config
        for key in path[:-1]:
            block = block[key]
        del block[path[-1]]
        with pytest.raises(ConfigError, match=message):
            model_spec_from_config(config)
    config = copy.deepcopy(tiny.A)
    config["layers"][2]["type"] = "attention_3"
    with pytest.raises(ConfigError, match="attention_3"):
        model_spec_from_config(config)
    config = copy.deepcopy(tiny.A)
    config["layers"][1]["mlp"] = dict(kind="sparse", ff=8)
    with pytest.raises(ConfigError, match="sparse"):
        model_spec_from_config(config)


def test_a_router_that_cannot_choose_is_refused():
    from vosti_b200.models.decoder import DecoderModel
    config = copy.deepcopy(tiny.A)
    config["layers"][0]["mlp"]["router"]["groups"] = dict(count=3, keep=1)     # three rows are kept, three are to be chosen: fine
    DecoderModel(model_spec_from_config(config))
    config["layers"][0]["mlp"]["router"]["top"] = 4                            # four of three
    with pytest.raises(ConfigError, match="top"):
        DecoderModel(model_spec_from_config(config))
    config = copy.deepcopy(tiny.A)
    config["layers"][0]["mlp"]["router"]["groups"] = dict(count=2, keep=1)     # nine rows in two groups
    with pytest.raises(ConfigError, match="groups"):
        DecoderModel(model_spec_from_config(config))


def test_random_model_folder_round_trip(tmp_path):
    from vosti_b200.weights import write_random_model
    write_random_model(tmp_path, tiny.B, seed=3)
    spec = model_spec_from_dir(tmp_path)
    assert spec.architecture == "Nefipel" and len(spec.layers) == 3


def test_plain_routing_keeps_to_the_best_groups_and_weights_sum_to_one():
    gen = torch.Generator().manual_seed(1)
    h = torch.randn(50, 16, generator=gen, dtype=torch.float64)
    w = {"router": torch.randn(12, 16, generator=gen, dtype=torch.float64), "correction": torch.randn(12, generator=gen, dtype=torch.float64)}
    r = dict(experts=9, identity=3, top=3, groups=dict(count=4, keep=2))
    chosen, weights = plain.route(h, w, r)
    assert torch.allclose(weights.sum(-1), torch.ones(50, dtype=torch.float64))
    assert all(len({e // 3 for e in row}) <= 2 and len(set(row)) == 3 for row in chosen.tolist())
    # a large correction decides the choice, not the weight: the weights are shares of the uncorrected scores
    w["correction"] = torch.zeros(12, dtype=torch.float64)
    w["correction"][7] = 10.0
    chosen, weights = plain.route(h, w, dict(experts=9, identity=3, top=3))
    s = torch.softmax(h @ w["router"].T, dim=-1)
    assert all(7 in row for row in chosen.tolist())
    picked = s.gather(1, chosen)
    assert torch.allclose(weights, picked / picked.sum(-1, keepdim=True))


def test_plain_identity_expert_returns_its_input():
    gen = torch.Generator().manual_seed(2)
    h = torch.randn(7, 8, generator=gen, dtype=torch.float64)
    w = {"router": torch.zeros(2, 8, dtype=torch.float64), "correction": torch.tensor([0.0, 1.0], dtype=torch.float64),
         "e0.up": torch.randn(4, 8, generator=gen, dtype=torch.float64), "e0.down": torch.randn(8, 4, generator=gen, dtype=torch.float64)}
    out = plain.expert_feed_forward(h, w, dict(router=dict(experts=1, identity=1, top=1)))
    assert torch.allclose(out, h)          # the identity expert is chosen alone, so its weight is one


def test_plain_differential_attention_with_equal_maps_cancels_by_lambda():
    """With both maps equal a head's output is (1 - lambda) a before the unit norm, so the norm makes the
    result independent of lambda's size and dependent on its side of one only."""
    gen = torch.Generator().manual_seed(3)
    m = dict(heads=2, kv_heads=1, dim=4, vdim=6, scale=0.5, diff=0.3, rot=dict(base=100.0, dims=4))
    width, T = 12, 9
    w = {"q": torch.randn(2, 1, 4, width, generator=gen, dtype=torch.float64).expand(2, 2, 4, width).reshape(16, width),
         "k": torch.randn(1, 1, 4, width, generator=gen, dtype=torch.float64).expand(1, 2, 4, width).reshape(8, width),
         "v": torch.randn(6, width, generator=gen, dtype=torch.float64), "o": torch.eye(12, dtype=torch.float64),
         "q.norm": torch.ones(4, dtype=torch.float64), "k.norm": torch.ones(4, dtype=torch.float64)}
    h = torch.randn(T, width, generator=gen, dtype=torch.float64)
    outs = []
    for size in (0.0, 0.2):                           # lambda = diff and lambda = e^(4 * 0.04) - 1 + diff, both below one
        w.update(lq1=torch.full((4,), size, dtype=torch.float64), lk1=torch.full((4,), size, dtype=torch.float64),
                 lq2=torch.zeros(4, dtype=torch.float64), lk2=torch.zeros(4, dtype=torch.float64))
        assert plain.differential_lambda(w, 0.3) < 1
        outs.append(plain.differential_attention(h, w, m, 1e-12))
    assert torch.allclose(outs[0], outs[1], atol=1e-9)
    assert torch.allclose((outs[0].view(T, 2, 6) ** 2).mean(-1), torch.full((T, 2), 0.49, dtype=torch.float64), atol=1e-6)
