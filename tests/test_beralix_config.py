"""Beralix on the CPU: its config.json reader, the tensors it asks for, the rescaled rotation
frequencies against the plain implementation, and the identities the latent attention's kernels
rest on, shown with the plain implementation's own functions."""
import copy
import math

import pytest
import torch

import plain_beralix as plain
import tiny_beralix as tiny
from vosti_b200.config import ConfigError, PartSpec, model_spec_from_config, model_spec_from_dir
from vosti_b200.models import expected_weights
from vosti_b200.parts import build_position
from vosti_b200.weights import check_tensors
from vosti_b200.weights.loader import WeightError


def test_spec_kinds_sizes_and_names():
    spec = model_spec_from_config(tiny.A)
    assert spec.architecture == "Beralix" and spec.hidden_size == 72 and spec.vocab_size == 211
    assert [layer.mixer.kind for layer in spec.layers] == ["latent_attention", "sink_attention", "selective_scan",
                                                           "sink_attention", "latent_attention", "sink_attention"]
    assert all(layer.arrangement == "sandwich_stream" and layer.layer_scale and layer.out_norm.kind == "layer_norm_stream"
               for layer in spec.layers)
    assert [layer.mixer.get("value_mix") for layer in spec.layers if layer.mixer.kind == "sink_attention"] == ["source", "mix", "mix"]
    assert spec.layers[1].mixer["window"] == 7 and spec.layers[1].mixer["position"]["rotary_dim"] == 8
    assert spec.layers[0].mixer["position"]["scaling"] == ("yarn", 3.0, 48.0, 4.0, 1.0)
    assert spec.layers[3].mixer["position"]["scaling"] is None
    assert spec.head.get("softcap") == 0.0 and model_spec_from_config(tiny.B).head.get("softcap") == 8.0
    names = expected_weights(spec)
    for name, shape in {"embed": (211, 72), "head": (211, 72), "final.norm": (72,), "final.norm.b": (72,), "l0.norm1b.b": (72,),
                        "l0.ls2": (72,), "l0.mix.q": (3 * 26, 72), "l0.mix.dkv": (46, 72), "l0.mix.dkv.norm": (40,),
                        "l0.mix.uk": (60, 40), "l0.mix.uv": (30, 40), "l0.mix.g": (3, 72), "l0.mix.o": (72, 30),
                        "l1.mix.k": (48, 72), "l1.mix.v": (32, 72), "l1.mix.vmix": (), "l2.mix.in": (100, 72),
                        "l2.mix.conv": (50, 4), "l2.mix.x": (13, 50), "l2.mix.dt": (50, 3), "l2.mix.A_log": (50, 5),
                        "l2.mix.D": (50,), "l0.mlp.gate": (40, 72), "l0.mlp.down": (72, 40)}.items():
        assert tuple(names[name].shape) == shape, name
    # what a model never reads may be there or not: the giver's mixing weight, an absent feed-forward's norms and scale
    optional = sorted(n for n, w in names.items() if w.optional)
    assert optional == sorted(["l1.mix.vmix"] + [f"l{i}.{t}" for i in (2, 4) for t in ("norm2", "norm2.b", "norm2b", "norm2b.b", "ls2")])
    assert "l2.mlp.gate" not in names


def test_checkpoints_with_and_without_unused_tensors_load():
    for unused in (True, False):
        spec, tensors = tiny.tensors_for(tiny.A, 5, unused)
        check_tensors(tensors, expected_weights(spec))
    spec, tensors = tiny.tensors_for(tiny.A, 5)
    del tensors["l3.mix.vmix"]          # a layer that mixes needs its weight
    with pytest.raises(WeightError) as error:
        check_tensors(tensors, expected_weights(spec))
    assert error.value.missing == ["l3.mix.vmix"]


def test_config_errors_name_the_key():
    for path, message in ((("layers", 0, "mixer", "kv_rank"), "kv_rank"), (("norm",), "norm"), (("layers", 2, "mixer", "dt_rank"), "dt_rank"),
                          (("layers", 1, "mixer", "rot", "base"), "base"), (("layers", 0, "mixer", "rot", "scaling", "slow"), "slow")):
        config = copy.deepcopy(tiny.A)
        block = config
        for key in path[:-1]:
            block = block[key]
        del block[path[-1]]
        with pytest.raises(ConfigError, match=message):
            model_spec_from_config(config)
    config = copy.deepcopy(tiny.A)
    config["layers"][2]["type"] = "mamba9"
    with pytest.raises(ConfigError, match="mamba9"):
        model_spec_from_config(config)
    config = copy.deepcopy(tiny.A)
    config["layers"][3]["mixer"]["vdim"] = 8          # the values it is to mix in have another width
    with pytest.raises(ConfigError, match="v_mix"):
        model_spec_from_config(config)
    config = copy.deepcopy(tiny.A)
    config["layers"][0]["mlp"] = dict(kind="sparse", ff=8)
    with pytest.raises(ConfigError, match="sparse"):
        model_spec_from_config(config)


def test_random_model_folder_round_trip(tmp_path):
    from vosti_b200.weights import write_random_model
    write_random_model(tmp_path, tiny.B, seed=3)
    spec = model_spec_from_dir(tmp_path)
    assert spec.architecture == "Beralix" and len(spec.layers) == 4


@pytest.mark.parametrize("base,dims,scaling", [(100.0, 6, (3.0, 48, 4.0, 1.0)), (300.0, 8, (2.0, 24, 3.0, 0.5)), (1000.0, 2, (4.0, 16, 2.0, 1.0)),
                                               (10000.0, 32, (8.0, 64, 8.0, 1.0)), (500000.0, 64, (16.0, 4096, 32.0, 1.0)), (50.0, 12, None)])
def test_rescaled_frequencies_against_plain(base, dims, scaling):
    rot = dict(base=base, dims=dims, scaling=None if scaling is None else dict(zip(("factor", "original", "fast", "slow"), scaling)))
    want, magnitude = plain.rotation_frequencies(rot)
    part = build_position(PartSpec.make("rope", theta=base, rotary_dim=dims, max_positions=0,
                                        scaling=None if scaling is None else ("yarn",) + tuple(float(v) for v in scaling)), 64, dims)
    assert torch.allclose(part.frequencies().double(), torch.tensor(want, dtype=torch.float64), rtol=1e-6, atol=0)
    assert part.magnitude() == pytest.approx(magnitude)
    if scaling is not None:
        assert magnitude == pytest.approx(0.1 * math.log(scaling[0]) + 1)
        # the fastest frequencies stay, the slowest are divided by the factor, none leaves that range
        plain_f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        assert all(f / scaling[0] * (1 - 1e-12) <= w <= f * (1 + 1e-12) for f, w in zip(plain_f, want))


def test_attention_in_the_latent_space_equals_attention_over_expanded_heads():
    """What the latent attention's kernels compute, written out here: scores from (W_uk[h]^T q_h) . c
    and values as W_uv[h] applied to the weighted latent, against the plain mixer."""
    gen = torch.Generator().manual_seed(1)
    m = tiny.A["layers"][0]["mixer"]
    H, D, R, Dv, rank, width, T, eps = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], 72, 33, 1e-5
    p = {"q": torch.randn(H * (D + R), width, generator=gen) / 8, "dkv": torch.randn(rank + R, width, generator=gen) / 8,
         "dkv.norm": 1 + 0.2 * torch.randn(rank, generator=gen), "uk": torch.randn(H * D, rank, generator=gen) / 6,
         "uv": torch.randn(H * Dv, rank, generator=gen) / 6, "g": torch.randn(H, width, generator=gen) / 4,
         "o": torch.randn(width, H * Dv, generator=gen) / 5}
    p = {k: v.double() for k, v in p.items()}
    h = torch.randn(T, width, generator=gen).double()
    want = plain.latent_attention(h, p, m, eps)
    rot = dict(m["rot"], dims=R)
    pos = torch.arange(T)
    q = (h @ p["q"].T).view(T, H, D + R)
    down = h @ p["dkv"].T
    c = plain.rms_norm(down[:, :rank], p["dkv.norm"], eps)
    r = plain.rotate(down[:, None, rank:], pos, rot)[:, 0]
    q_latent = torch.einsum("thd,hdr->thr", q[..., :D], p["uk"].view(H, D, rank))
    scores = (torch.einsum("ihr,jr->hij", q_latent, c) + torch.einsum("ihr,jr->hij", plain.rotate(q[..., D:], pos, rot), r)) * m["scale"]
    scores = scores.masked_fill(~(pos[None, :] <= pos[:, None])[None], float("-inf"))
    weighted = torch.einsum("hij,jr->ihr", torch.softmax(scores, -1), c)
    heads = torch.einsum("thr,hvr->thv", weighted, p["uv"].view(H, Dv, rank)) * torch.sigmoid(h @ p["g"].T)[:, :, None]
    assert torch.allclose(heads.reshape(T, H * Dv) @ p["o"].T, want, atol=1e-10)


def test_plain_scan_carries_its_state_token_by_token():
    """The recurrence of the plain implementation, run once over a sequence and once token by token
    with the state and the convolution's last inputs carried by hand."""
    gen = torch.Generator().manual_seed(2)
    m = dict(inner=10, state=3, conv=3, dt_rank=2)
    width, T = 12, 9
    p = {"in": torch.randn(20, width, generator=gen) / 3, "conv": torch.randn(10, 3, generator=gen) / 2, "conv.b": torch.randn(10, generator=gen) / 4,
         "x": torch.randn(8, 10, generator=gen) / 3, "dt": torch.randn(10, 2, generator=gen), "dt.b": torch.randn(10, generator=gen),
         "A_log": torch.randn(10, 3, generator=gen) / 2, "D": torch.randn(10, generator=gen), "o": torch.randn(width, 10, generator=gen) / 3}
    p = {k: v.double() for k, v in p.items()}
    h = torch.randn(T, width, generator=gen).double()
    want = plain.selective_scan(h, p, m)
    S, tail, rows = torch.zeros(10, 3, dtype=torch.float64), torch.zeros(2, 10, dtype=torch.float64), []
    for t in range(T):
        xz = h[t] @ p["in"].T
        u, z = xz[:10], xz[10:]
        window = torch.cat([tail, u[None]])
        x = plain.silu((window * p["conv"].T).sum(0) + p["conv.b"])
        tail = window[1:]
        proj = p["x"] @ x
        dt = plain.softplus(p["dt"] @ proj[:2] + p["dt.b"])
        S = torch.exp(dt[:, None] * -torch.exp(p["A_log"])) * S + (dt * x)[:, None] * proj[2:5][None]
        rows.append(((S @ proj[5:] + p["D"] * x) * plain.silu(z)) @ p["o"].T)
    assert torch.allclose(torch.stack(rows), want, atol=1e-10)
