"""The Beralix design, read from its own config.json.

A decoder over a float32 residual stream whose every sublayer is normed before and after
(layer norms with weight and bias) and scaled by a learned vector as it joins the stream:

    x <- x + ls1 * norm1b(mixer(norm1(x)));   x <- x + ls2 * norm2b(ff(norm2(x)))

Three kinds of layer, in any order:

  "latent_attention"  causal attention whose keys and values are made from one cached latent per
                      token, a rotated key part shared by the heads, a sigmoid gate per head;
  "attention"         grouped-query attention over a sliding window with a partial rotation;
                      layers marked `v_mix` blend their values with those of the first such layer;
  "mamba1"            a selective scan with a short convolution.

Rotations pair element i with i + dims / 2 and may be rescaled ("scaling": factor, original,
fast, slow; see parts/rope.py, "yarn"). Feed-forwards are SiLU-gated and dense, or absent; the
logits pass a soft cap.

Keys (a missing one is an error unless marked optional; optional blocks may be absent or null):

    architecture  "Beralix"
    vocab, width
    norm.eps
    logit_softcap                          optional
    layers[i].type                         "latent_attention" | "attention" | "mamba1"
    layers[i].mixer (latent_attention)     heads, dim, rot_dim, vdim, kv_rank, scale, rot.base, rot.scaling (optional)
    layers[i].mixer (attention)            heads, kv_heads, dim, vdim, scale, rot.base, rot.dims, rot.scaling (optional),
                                           mask.size (optional), v_mix (optional)
    layers[i].mixer (mamba1)               inner, state, conv, dt_rank
    layers[i].mlp                          optional: {kind: "dense", ff}
"""
from __future__ import annotations

from typing import Any, Mapping, Optional

from .schema import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

ARCHITECTURE = "Beralix"
MAX_POSITIONS = 1 << 30        # the design sets no limit (angles are formed from the position); the cache pool does


def _need(block: Mapping[str, Any], key: str, where: str):
    if not isinstance(block, Mapping) or key not in block:
        raise ConfigError(f"Beralix config: {where} lacks '{key}'")
    return block[key]


def _positive_int(block, key, where) -> int:
    value = _need(block, key, where)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"Beralix config: {where}.{key} must be a positive integer, got {value!r}")
    return value


def _number(block, key, where) -> float:
    value = _need(block, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or value != value:
        raise ConfigError(f"Beralix config: {where}.{key} must be a number, got {value!r}")
    return float(value)


def _rotation(rot: Mapping[str, Any], dims: int, where: str) -> PartSpec:
    scaling = rot.get("scaling") if isinstance(rot, Mapping) else None
    if scaling is not None:
        sw = where + ".scaling"
        scaling = ("yarn", _number(scaling, "factor", sw), _number(scaling, "original", sw), _number(scaling, "fast", sw),
                   _number(scaling, "slow", sw))
    return PartSpec.make("rope", theta=_number(rot, "base", where), rotary_dim=dims, scaling=scaling, max_positions=0)


def _latent(i: int, block: Mapping[str, Any], eps: float) -> PartSpec:
    where = f"layers[{i}].mixer"
    rot_dim = _positive_int(block, "rot_dim", where)
    return PartSpec.make(
        "latent_attention", num_heads=_positive_int(block, "heads", where), head_dim=_positive_int(block, "dim", where),
        rot_dim=rot_dim, v_head_dim=_positive_int(block, "vdim", where), kv_rank=_positive_int(block, "kv_rank", where),
        scale=_number(block, "scale", where), eps=eps, gate=True,
        position=_rotation(_need(block, "rot", where), rot_dim, where + ".rot"))


def _window(i: int, block: Mapping[str, Any], value_mix: Optional[str]) -> PartSpec:
    where = f"layers[{i}].mixer"
    rot = _need(block, "rot", where)
    mask = block.get("mask")
    return PartSpec.make(
        "sink_attention", num_heads=_positive_int(block, "heads", where), num_kv_heads=_positive_int(block, "kv_heads", where),
        head_dim=_positive_int(block, "dim", where), v_head_dim=_positive_int(block, "vdim", where),
        scale=_number(block, "scale", where), window=0 if mask is None else _positive_int(mask, "size", where + ".mask"),
        chunk=0, sink=False, value_mix=value_mix,
        position=_rotation(rot, _positive_int(rot, "dims", where + ".rot"), where + ".rot"))


def _scan(i: int, block: Mapping[str, Any]) -> PartSpec:
    where = f"layers[{i}].mixer"
    return PartSpec.make("selective_scan", inner=_positive_int(block, "inner", where), state=_positive_int(block, "state", where),
                         conv_taps=_positive_int(block, "conv", where), dt_rank=_positive_int(block, "dt_rank", where))


def _feed_forward(i: int, block: Optional[Mapping[str, Any]]) -> Optional[PartSpec]:
    if block is None:
        return None
    where = f"layers[{i}].mlp"
    kind = _need(block, "kind", where)
    if kind != "dense":
        raise ConfigError(f"Beralix config: {where}.kind is {kind!r}; 'dense' is known")
    return PartSpec.make("swiglu", intermediate_size=_positive_int(block, "ff", where), tensor_names=("gate", "up", "down"),
                         float32_out=True)


def spec_from_config(raw: Mapping[str, Any]) -> ModelSpec:
    if not isinstance(raw, Mapping) or raw.get("architecture") != ARCHITECTURE:
        raise ConfigError("Beralix config: 'architecture' must be 'Beralix'")
    width, vocab = _positive_int(raw, "width", "config"), _positive_int(raw, "vocab", "config")
    eps = _number(_need(raw, "norm", "config"), "eps", "norm")
    norm = PartSpec.make("layer_norm_stream", eps=eps, bias=True, bias_name="b")
    layers = _need(raw, "layers", "config")
    if not isinstance(layers, list) or not layers:
        raise ConfigError("Beralix config: 'layers' must be a nonempty list")
    names = (("input_norm", "norm1"), ("mixer_out_norm", "norm1b"), ("post_norm", "norm2"), ("ff_out_norm", "norm2b"),
             ("mixer", "mix"), ("feed_forward", "mlp"), ("mixer_scale", "ls1"), ("ff_scale", "ls2"))
    specs, mixing = [], None
    for i, layer in enumerate(layers):
        kind = _need(layer, "type", f"layers[{i}]")
        block = _need(layer, "mixer", f"layers[{i}]")
        if kind == "latent_attention":
            mixer = _latent(i, block, eps)
        elif kind == "attention":
            role = None
            if block.get("v_mix"):
                sizes = (block.get("kv_heads"), block.get("vdim"))
                if mixing is None:
                    role, mixing = "source", sizes
                elif sizes != mixing:
                    raise ConfigError(f"Beralix config: layers[{i}] mixes in the values of the first v_mix layer, which have "
                                      f"other sizes (kv_heads, vdim) = {mixing}")
                else:
                    role = "mix"
            mixer = _window(i, block, role)
        elif kind == "mamba1":
            mixer = _scan(i, block)
        else:
            raise ConfigError(f"Beralix config: layers[{i}].type is {kind!r}; 'latent_attention', 'attention' and 'mamba1' are known")
        specs.append(LayerSpec(mixer=mixer, feed_forward=_feed_forward(i, layer.get("mlp")), norm=norm, position=None,
                               arrangement="sandwich_stream", names=names, out_norm=norm, layer_scale=True))
    cap = raw.get("logit_softcap")
    if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or cap < 0):
        raise ConfigError("Beralix config: logit_softcap must be a number >= 0")
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=width, vocab_size=vocab, max_positions=MAX_POSITIONS,
        layers=tuple(specs), run_order=tuple(RunEntry(i) for i in range(len(specs))), final_norm=norm,
        tie_word_embeddings=False, embed_name="embed", final_norm_name="final.norm", lm_head_name="head",
        layer_prefix="l{i}.", head=PartSpec.make("linear", softcap=float(cap or 0.0)))
