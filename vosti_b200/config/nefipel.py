"""The Nefipel design, read from its own config.json.

A decoder over a float32 residual stream that norms after the sum,

    x <- norm1(alpha x + mixer(x));   x <- norm2(alpha x + ff(x))

with root-mean-square norms, one alpha for the model, and the sublayers reading x itself. The
embedding rows are multiplied by a constant; the output head is the embedding table (unscaled).
Two kinds of layer, in any order:

  "attention"    grouped-query softmax attention: projections with biases, an RMS norm of every
                 query and key head (weight shared by the heads), a rotation of the first
                 elements of each head in pairs (i, i + dims / 2), and a sigmoid gate from the
                 layer's input on the concatenated heads;
  "attention_2"  differential attention: two score maps a head over the same values, no biases,
                 the same head norm, a rotation in neighbouring pairs (2i, 2i + 1), the second
                 map subtracted with one learned factor a layer, the difference brought to unit
                 root mean square and multiplied by 1 - diff.

Either rotation may be rescaled by index ("scaling": factor, original, fast, slow; see
parts/rope.py, "yarn"). Feed-forwards: dense relu(gate) * up; or a mixture of squared-relu experts
chosen by corrected softmax scores inside the best groups of neighbouring experts, the last
`identity` of which return their input, with an optional shared expert behind a per-token sigmoid
gate; or none.

Keys (a missing one is an error unless marked optional; optional blocks may be absent or null):

    architecture  "Nefipel"
    vocab, width, postln_alpha
    norm.eps
    embedding.scale                        optional (1)
    layers[i].type                         "attention" | "attention_2"
    layers[i].mixer                        heads, kv_heads, dim, vdim, scale, rot.base, rot.dims,
                                           rot.scaling (optional); attention_2 also: diff
    layers[i].mlp                          optional: {kind: "dense", ff} or {kind: "moe", expert.ff,
                                           router: {experts, top, identity (optional), groups: {count, keep}
                                           (optional)}, shared: {ff} (optional)}
"""
from __future__ import annotations

from typing import Any, Mapping, Optional

from .schema import ConfigError, LayerSpec, ModelSpec, PartSpec, RunEntry

ARCHITECTURE = "Nefipel"
MAX_POSITIONS = 1 << 30        # the design sets no limit (angles are formed from the position); the cache pool does


def _need(block: Mapping[str, Any], key: str, where: str):
    if not isinstance(block, Mapping) or key not in block:
        raise ConfigError(f"Nefipel config: {where} lacks '{key}'")
    return block[key]


def _positive_int(block, key, where) -> int:
    value = _need(block, key, where)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"Nefipel config: {where}.{key} must be a positive integer, got {value!r}")
    return value


def _count(block, key, where) -> int:
    """An optional count: absent, null or a non-negative integer."""
    value = block.get(key) if isinstance(block, Mapping) else None
    if value is None:
        return 0
    if isinstance(value, bool) or not isinstance(value, int) or value < 0:
        raise ConfigError(f"Nefipel config: {where}.{key} must be a non-negative integer, got {value!r}")
    return value


def _number(block, key, where) -> float:
    value = _need(block, key, where)
    if isinstance(value, bool) or not isinstance(value, (int, float)) or value != value:
        raise ConfigError(f"Nefipel config: {where}.{key} must be a number, got {value!r}")
    return float(value)


def _rotation(rot: Mapping[str, Any], where: str, interleaved: bool) -> PartSpec:
    scaling = rot.get("scaling") if isinstance(rot, Mapping) else None
    if scaling is not None:
        sw = where + ".scaling"
        scaling = ("yarn", _number(scaling, "factor", sw), _number(scaling, "original", sw), _number(scaling, "fast", sw),
                   _number(scaling, "slow", sw))
    return PartSpec.make("rope", theta=_number(rot, "base", where), rotary_dim=_positive_int(rot, "dims", where),
                         scaling=scaling, max_positions=0, interleaved=interleaved)


def _attention(i: int, block: Mapping[str, Any], eps: float, differential: bool) -> PartSpec:
    where = f"layers[{i}].mixer"
    common = dict(
        num_heads=_positive_int(block, "heads", where), num_kv_heads=_positive_int(block, "kv_heads", where),
        head_dim=_positive_int(block, "dim", where), v_head_dim=_positive_int(block, "vdim", where),
        scale=_number(block, "scale", where), window=0, chunk=0, sink=False, head_norm_eps=eps, partial_out=True,
        position=_rotation(_need(block, "rot", where), where + ".rot", interleaved=differential))
    if differential:
        return PartSpec.make("sink_attention", maps=2, diff=_number(block, "diff", where), out_norm_eps=eps, **common)
    return PartSpec.make("sink_attention", qkv_bias=True, out_gate=True, **common)


def _feed_forward(i: int, block: Optional[Mapping[str, Any]]) -> Optional[PartSpec]:
    if block is None:
        return None
    where = f"layers[{i}].mlp"
    kind = _need(block, "kind", where)
    if kind == "dense":
        return PartSpec.make("swiglu", intermediate_size=_positive_int(block, "ff", where), tensor_names=("gate", "up", "down"),
                             float32_out=True, activation="relu", partial_out=True)
    if kind == "moe":
        router = _need(block, "router", where)
        rw = where + ".router"
        groups = router.get("groups") if isinstance(router, Mapping) else None
        shared = block.get("shared")
        return PartSpec.make(
            "moe", experts=_positive_int(router, "experts", rw), top=_positive_int(router, "top", rw),
            intermediate_size=_positive_int(_need(block, "expert", where), "ff", where + ".expert"), gated=False,
            activation="relu2", route="scored", correction=True, identity=_count(router, "identity", rw),
            groups=1 if groups is None else _positive_int(groups, "count", rw + ".groups"),
            keep=1 if groups is None else _positive_int(groups, "keep", rw + ".groups"),
            shared=0 if shared is None else _positive_int(shared, "ff", where + ".shared"), float32_out=True, partial_out=True)
    raise ConfigError(f"Nefipel config: {where}.kind is {kind!r}; 'dense' and 'moe' are known")


def spec_from_config(raw: Mapping[str, Any]) -> ModelSpec:
    if not isinstance(raw, Mapping) or raw.get("architecture") != ARCHITECTURE:
        raise ConfigError("Nefipel config: 'architecture' must be 'Nefipel'")
    width, vocab = _positive_int(raw, "width", "config"), _positive_int(raw, "vocab", "config")
    eps = _number(_need(raw, "norm", "config"), "eps", "norm")
    alpha = _number(raw, "postln_alpha", "config")
    embedding = raw.get("embedding")
    scale = 1.0 if embedding is None else _number(embedding, "scale", "embedding")
    layers = _need(raw, "layers", "config")
    if not isinstance(layers, list) or not layers:
        raise ConfigError("Nefipel config: 'layers' must be a nonempty list")
    names = (("input_norm", "norm1"), ("post_norm", "norm2"), ("mixer", "mix"), ("feed_forward", "mlp"))
    specs = []
    for i, layer in enumerate(layers):
        kind = _need(layer, "type", f"layers[{i}]")
        if kind not in ("attention", "attention_2"):
            raise ConfigError(f"Nefipel config: layers[{i}].type is {kind!r}; 'attention' and 'attention_2' are known")
        mixer = _attention(i, _need(layer, "mixer", f"layers[{i}]"), eps, kind == "attention_2")
        specs.append(LayerSpec(mixer=mixer, feed_forward=_feed_forward(i, layer.get("mlp")),
                               norm=PartSpec.make("rms_stream", eps=eps, alpha=alpha), position=None,
                               arrangement="post_norm_stream", names=names))
    return ModelSpec(
        architecture=ARCHITECTURE, hidden_size=width, vocab_size=vocab, max_positions=MAX_POSITIONS,
        layers=tuple(specs), run_order=tuple(RunEntry(i) for i in range(len(specs))),
        final_norm=PartSpec.make("rms_stream", eps=eps), tie_word_embeddings=True, embed_name="embed",
        final_norm_name="final.norm", lm_head_name="head", layer_prefix="l{i}.",
        embedding=PartSpec.make("table", scale=scale, out_dtype="float32"))
