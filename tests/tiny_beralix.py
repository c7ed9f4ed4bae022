"""Small Beralix configurations for the tests, with weights of a size that makes every mechanism
matter (unit-variance activations, scores of several units so that single keys dominate rows,
biases and layer scales of order one), written as a model folder.

A: odd sizes everywhere; all three kinds of layer, a latent layer first; head counts that differ
   from layer to layer; fewer key/value heads than heads; key and value widths that differ; a
   rotation of part of the head with rescaled frequencies in one attention layer and of the whole
   head without rescaling in the other; windows of 7 and 20; three layers that mix values (the
   first one gives them); a layer without a feed-forward; feed-forwards narrower and wider than
   the model; 5 states and a convolution of 4 taps; no soft cap on the logits.
B: values of one: one head, one state, a step-size rank of one, a convolution of one tap (no tail
   in the state), a window of one (a query sees itself only), a rotated part of two elements; an
   attention layer without a window and without value mixing; a scan layer first; no attention
   layer gives values, so none mixes.
C: attention heads of 64 with equal key and value widths and pages of 16 tokens (the sizes the
   tensor-core attention kernels take in bfloat16), latent widths in whole 16-byte words, 40
   states (eight lanes a channel), two scan layers in a row.
D: latent layers of the sizes the tensor-core latent kernels take in bfloat16 (latents of 128 and
   256, rotated parts of 32 and 64), one whose projection rows are whole 16-byte words (its
   per-head products run on the tensor cores both ways) and one whose are not; 12 states.
"""
import json
from pathlib import Path

import torch

from vosti_b200.config import model_spec_from_config
from vosti_b200.models import expected_weights
from vosti_b200.weights import write_safetensors


def _scaling(factor, original, fast, slow):
    return dict(factor=factor, original=original, fast=fast, slow=slow)


def _latent(heads, dim, rot_dim, vdim, rank, scale, base, scaling, mlp):
    return dict(type="latent_attention", mlp=mlp, mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=rank,
                                                             scale=scale, rot=dict(base=base, dims=rot_dim, scaling=scaling)))


def _window(heads, kv, dim, vdim, scale, size, base, dims, scaling, v_mix, mlp):
    mixer = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, rot=dict(base=base, dims=dims, scaling=scaling))
    if size:
        mixer["mask"] = dict(size=size)
    if v_mix:
        mixer["v_mix"] = True
    return dict(type="attention", mixer=mixer, mlp=mlp)


def _scan(inner, state, conv, dt_rank, mlp):
    return dict(type="mamba1", mixer=dict(inner=inner, state=state, conv=conv, dt_rank=dt_rank), mlp=mlp)


def _dense(ff):
    return dict(kind="dense", ff=ff)


A = dict(architecture="Beralix", vocab=211, width=72, norm=dict(eps=2e-6), layers=[
    _latent(3, 20, 6, 10, 40, 0.9, 100.0, _scaling(3.0, 48, 4.0, 1.0), _dense(40)),
    _window(4, 2, 24, 16, 0.8, 7, 300.0, 8, _scaling(2.0, 24, 3.0, 0.5), True, _dense(100)),
    _scan(50, 5, 4, 3, None),
    _window(6, 2, 12, 16, 1.1, 20, 10000.0, 12, None, True, _dense(72)),
    _latent(5, 12, 10, 24, 24, 1.0, 5000.0, None, None),
    _window(2, 2, 20, 16, 1.0, 7, 300.0, 20, _scaling(5.0, 64, 16.0, 2.0), True, _dense(24)),
])
B = dict(architecture="Beralix", vocab=128, width=64, norm=dict(eps=1e-5), logit_softcap=8.0, layers=[
    _scan(40, 1, 1, 1, _dense(48)),
    _window(1, 1, 32, 40, 0.7, 1, 1000.0, 2, _scaling(4.0, 16, 2.0, 1.0), False, _dense(80)),
    _latent(1, 8, 2, 8, 8, 1.2, 50.0, _scaling(2.0, 8, 2.0, 1.0), _dense(32)),
    _window(2, 1, 16, 24, 0.9, 0, 1000.0, 16, None, False, None),
])
C = dict(architecture="Beralix", vocab=160, width=128, norm=dict(eps=1e-6), logit_softcap=25.0, layers=[
    _window(4, 2, 64, 64, 0.5, 48, 10000.0, 32, _scaling(8.0, 64, 8.0, 1.0), True, _dense(192)),
    _latent(4, 40, 16, 56, 64, 0.6, 20000.0, _scaling(4.0, 128, 16.0, 1.0), _dense(64)),
    _scan(96, 40, 3, 8, _dense(64)),
    _scan(64, 16, 2, 16, None),
    _window(2, 2, 64, 64, 0.5, 33, 50000.0, 64, None, True, _dense(128)),
])
D = dict(architecture="Beralix", vocab=192, width=96, norm=dict(eps=1e-5), logit_softcap=15.0, layers=[
    _latent(8, 24, 32, 40, 128, 0.5, 8000.0, _scaling(4.0, 64, 8.0, 1.0), _dense(96)),
    _scan(128, 12, 3, 6, _dense(48)),
    _window(8, 2, 64, 64, 0.4, 19, 100000.0, 32, None, True, None),
    _latent(4, 32, 64, 16, 256, 0.45, 1000.0, None, _dense(64)),
    _window(8, 2, 64, 64, 0.4, 50, 100000.0, 64, _scaling(2.0, 32, 4.0, 1.0), True, _dense(96)),
])
ALL = {"a": (A, 31), "b": (B, 32), "c": (C, 33), "d": (D, 34)}      # config, seed
PAGE = {"a": 8, "b": 4, "c": 16, "d": 16}


def draw(name, shape, gen):
    """One tensor by its role, float32 (the caller rounds to bfloat16)."""
    n = lambda std, mean=0.0: mean + std * torch.randn(shape, generator=gen)
    last = name.split(".")[-1]
    if name == "embed":
        return n(1.0)
    if last == "conv":
        return n(0.6)
    if last == "A_log":
        return n(0.7, -0.5)
    if name.endswith("dt.b"):
        return n(1.0, -1.0)
    if last == "vmix":
        return n(0.1, 0.45)
    if last in ("ls1", "ls2"):
        return n(0.3, 0.8)
    if last == "b":                          # biases of norms and of the convolution
        return n(0.3)
    if len(shape) == 1:                      # weights of norms, D
        return n(0.2, 1.0)
    if last in ("g", "dt"):
        return n(2.0 / shape[1] ** 0.5)
    return n(1.0 / shape[1] ** 0.5)


def tensors_for(config, seed, unused=True):
    """`unused` false leaves out the tensors the model never reads (norms and scale of an absent
    feed-forward, the mixing weight of the layer that gives the values); a checkpoint may have them or not."""
    spec = model_spec_from_config(config)
    gen = torch.Generator().manual_seed(seed)
    return spec, {name: draw(name, tuple(w.shape), gen).to(torch.bfloat16) for name, w in expected_weights(spec).items()
                  if unused or not w.optional}


def write_model(folder, config, seed, unused=True):
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    _, tensors = tensors_for(config, seed, unused)
    (folder / "config.json").write_text(json.dumps(config))
    write_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt"})
    return str(folder)
