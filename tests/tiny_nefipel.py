"""Small Nefipel configurations for the tests, with weights of a size that makes every mechanism
matter (scores of several units, biases and corrections of a size that changes choices, gates
away from one half), written as a model folder.

A: odd sizes everywhere; both kinds of layer, a differential layer first; head counts that differ
   from layer to layer; fewer key/value heads than heads; key and value widths that differ; a
   rotation of part of the head with rescaled frequencies and one of the whole head without; a
   mixture with identity experts, groups and a shared expert and one with none of them; a layer
   without a feed-forward; feed-forwards narrower and wider than the model.
B: values of one: one head, one kv head, a rotated part of two elements, one expert beside one
   identity expert, one chosen, every expert a group of its own, alpha 1, no embedding scale.
C: heads of 64 and 128 with equal key and value widths and pages of 16 tokens (the sizes the
   tensor-core attention kernels take in bfloat16 for layers with one score map), widths in
   whole 16-byte words, sixteen experts in four groups with four identity experts.
"""
import json
from pathlib import Path

import torch

from vosti_b200.config import model_spec_from_config
from vosti_b200.models import expected_weights
from vosti_b200.weights import write_safetensors


def _scaling(factor, original, fast, slow):
    return dict(factor=factor, original=original, fast=fast, slow=slow)


def _mixer(heads, kv, dim, vdim, scale, base, dims, scaling=None, diff=None):
    rot = dict(base=base, dims=dims)
    if scaling is not None:
        rot["scaling"] = scaling
    mixer = dict(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=scale, rot=rot)
    if diff is not None:
        mixer["diff"] = diff
    return mixer


def gated(heads, kv, dim, vdim, scale, base, dims, scaling, mlp):
    return dict(type="attention", mixer=_mixer(heads, kv, dim, vdim, scale, base, dims, scaling), mlp=mlp)


def differential(heads, kv, dim, vdim, scale, base, dims, scaling, diff, mlp):
    return dict(type="attention_2", mixer=_mixer(heads, kv, dim, vdim, scale, base, dims, scaling, diff), mlp=mlp)


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(experts, top, ff, identity=None, groups=None, shared=None):
    router = dict(experts=experts, top=top)
    if identity is not None:
        router["identity"] = identity
    if groups is not None:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    block = dict(kind="moe", expert=dict(ff=ff), router=router)
    if shared is not None:
        block["shared"] = dict(ff=shared)
    return block


A = dict(architecture="Nefipel", vocab=211, width=72, norm=dict(eps=2e-6), postln_alpha=1.7, embedding=dict(scale=3.3), layers=[
    differential(3, 1, 10, 14, 0.95, 100.0, 6, _scaling(3.0, 48, 4.0, 1.0), 0.2, moe(6, 3, 20, identity=3, groups=(3, 2), shared=36)),
    gated(4, 2, 24, 16, 0.6, 300.0, 8, _scaling(2.0, 24, 3.0, 0.5), dense(100)),
    gated(6, 3, 12, 20, 0.85, 10000.0, 12, None, None),
    differential(2, 2, 20, 8, 0.7, 5000.0, 20, None, 0.45, moe(5, 2, 24)),
])
B = dict(architecture="Nefipel", vocab=128, width=64, norm=dict(eps=1e-5), postln_alpha=1.0, layers=[
    gated(1, 1, 32, 40, 0.5, 1000.0, 2, _scaling(4.0, 16, 2.0, 1.0), moe(1, 1, 48, identity=1, groups=(2, 1))),
    differential(1, 1, 2, 3, 1.5, 50.0, 2, _scaling(2.0, 8, 2.0, 1.0), 0.1, dense(80)),
    differential(2, 1, 16, 24, 0.7, 1000.0, 16, None, 0.6, moe(3, 1, 16, shared=8)),
])
C = dict(architecture="Nefipel", vocab=160, width=128, norm=dict(eps=1e-6), postln_alpha=3.0, embedding=dict(scale=11.3), layers=[
    gated(4, 2, 64, 64, 0.35, 10000.0, 32, _scaling(8.0, 64, 8.0, 1.0), dense(192)),
    differential(4, 2, 64, 64, 0.35, 20000.0, 64, _scaling(4.0, 128, 16.0, 1.0), 0.3, moe(12, 4, 32, identity=4, groups=(4, 2), shared=64)),
    gated(2, 1, 128, 128, 0.25, 50000.0, 64, None, moe(8, 2, 48, identity=0, groups=(2, 1))),
    differential(2, 1, 32, 96, 0.5, 8000.0, 16, None, 0.25, dense(64)),
])
ALL = {"a": (A, 41), "b": (B, 42), "c": (C, 43)}      # config, seed
PAGE = {"a": 8, "b": 4, "c": 16}


def draw(name, shape, gen):
    """One tensor by its role, float32 (the caller rounds to bfloat16)."""
    n = lambda std, mean=0.0: mean + std * torch.randn(shape, generator=gen)
    last = name.split(".")[-1]
    if name == "embed":
        return n(1.0)
    if last == "correction":
        return n(0.1)
    if last in ("lq1", "lk1", "lq2", "lk2"):
        return n(0.3)
    if last == "b":                          # projection biases
        return n(0.4)
    if len(shape) == 1:                      # weights of norms
        return n(0.2, 1.0)
    if last in ("g", "sg", "router"):
        return n(2.0 / shape[1] ** 0.5)
    return n(1.0 / shape[1] ** 0.5)


def tensors_for(config, seed, unused=True):
    """`unused` false leaves out the tensors the model never reads (the second norm of a layer
    without a feed-forward); a checkpoint may have them or not."""
    spec = model_spec_from_config(config)
    gen = torch.Generator().manual_seed(seed)
    expected = expected_weights(spec)
    drawn = {name: draw(name, tuple(w.shape), gen).to(torch.bfloat16) for name, w in expected.items()}
    return spec, {name: t for name, t in drawn.items() if unused or not expected[name].optional}


def write_model(folder, config, seed, unused=True):
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    _, tensors = tensors_for(config, seed, unused)
    (folder / "config.json").write_text(json.dumps(config))
    write_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt"})
    return str(folder)
