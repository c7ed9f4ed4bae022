"""A block: mixer, feed-forward and their norms around the residual stream.

'pre_norm' is the reference's wiring with a deferred add
(src/exec/dense_swiglu_decoder.rs:556-615, 740-813, 370-383): a block receives
(hidden, residual), norms hidden + residual (the first block norms the embedding and
adds nothing), runs the mixer, norms mixer_out + residual, runs the feed-forward and
returns (feed_forward_out, residual); the model's final norm does the last add.
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..config.schema import ConfigError, LayerSpec
from ..weights.loader import WeightSpec
from .base import Norm, build_feed_forward, build_mixer, build_norm, build_token_input, part_factory, register_part


class PreNormBlock:
    def __init__(self, spec: LayerSpec, hidden_size: int):
        self.spec = spec
        self.mixer = build_mixer(spec.mixer, hidden_size, spec.position)
        self.feed_forward = build_feed_forward(spec.feed_forward, hidden_size)
        self.input_norm = build_norm(spec.norm, hidden_size)
        self.post_norm = build_norm(spec.norm, hidden_size) if self.feed_forward is not None else None

    def _children(self):
        n = self.spec.name_of
        yield n("input_norm"), self.input_norm
        yield n("mixer"), self.mixer
        if self.feed_forward is not None:
            yield n("post_norm"), self.post_norm
            yield n("feed_forward"), self.feed_forward

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {f"{name}.{key}": spec for name, part in self._children()
                for key, spec in part.weight_specs().items()}

    def load(self, tensors, dtype):
        for name, part in self._children():
            prefix = name + "."
            part.load({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, dtype)

    def setup(self, device, dtype):
        for _, part in self._children():
            part.setup(device, dtype)

    def forward(self, ctx, hidden, residual, cache, writes_cache=True):
        # In a step of few tokens a norm leaves HBM idle: it is told which weight the product
        # after it will stream, so that it can ask for it ahead of time (ops.hint_prefetch).
        few = ctx.num_tokens <= ops.PREFETCH_MAX_TOKENS
        if residual is None:
            residual = hidden = ops.materialize(hidden)
            normed = self.input_norm.forward(ctx, hidden)
        else:
            hinted = few and ops.hint_prefetch(self.mixer.first_weight())
            normed, residual = self.input_norm.forward_add(ctx, hidden, residual)
            if hinted:
                ops.hint_prefetch(None)
        out = self.mixer.forward(ctx, normed, cache, writes_cache)
        # (a mixer or feed-forward may return its last product as unsummed K splits; the
        # norm that follows adds them, see ops.PartialSum)
        if self.feed_forward is not None:
            hinted = few and ops.hint_prefetch(self.feed_forward.first_weight())
            normed, residual = self.post_norm.forward_add(ctx, out, residual)
            if hinted:
                ops.hint_prefetch(None)
            out = self.feed_forward.forward(ctx, normed)
        return out, residual


register_part("arrangement", "pre_norm", PreNormBlock, replace=True)


def build_block(spec: LayerSpec, hidden_size: int):
    return part_factory("arrangement", spec.arrangement)(spec, hidden_size)


class ParallelBlock:
    """'parallel': one norm whose output both sublayers read, x <- x + (mixer(h) + ff(h)) with
    h = norm(x), over a float32 residual stream (the norm is one that keeps the stream, like
    `DynamicTanh`). The add is deferred like the pre-norm block's: a block receives the stream
    and what the block before left to be added (`ops.DeferredSum`), its norm adds while it
    reads, and it returns its own sublayers' outputs unadded. A block without a feed-forward
    returns the mixer's output alone.

    Checkpoint names: `LayerSpec.names` maps the roles "norm", "mixer", "feed_forward" to name
    fragments; the norm's `weight` tensor is called by the fragment itself and its other tensors
    `<fragment>.<key>`."""

    def __init__(self, spec: LayerSpec, hidden_size: int):
        self.spec = spec
        if spec.position is not None:
            raise ConfigError("parallel block: position encodings belong to the mixers that apply them")
        self.mixer = build_mixer(spec.mixer, hidden_size, None)
        self.feed_forward = build_feed_forward(spec.feed_forward, hidden_size)
        self.norm = build_norm(spec.norm, hidden_size)
        self.capture_safe = True

    def _children(self):
        n = self.spec.name_of
        yield n("norm"), self.norm
        yield n("mixer"), self.mixer
        if self.feed_forward is not None:
            yield n("feed_forward"), self.feed_forward

    def _names(self):
        """(checkpoint name relative to the layer, part, the part's key) for every tensor."""
        n = self.spec.name_of
        for key in self.norm.weight_specs():
            yield (n("norm") if key == "weight" else f"{n('norm')}.{key}"), self.norm, key
        for key in self.mixer.weight_specs():
            yield f"{n('mixer')}.{key}", self.mixer, key
        if self.feed_forward is not None:
            for key in self.feed_forward.weight_specs():
                yield f"{n('feed_forward')}.{key}", self.feed_forward, key

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {name: part.weight_specs()[key] for name, part, key in self._names()}

    def load(self, tensors, dtype):
        per_part = {}
        for name, part, key in self._names():
            if name in tensors:
                per_part.setdefault(id(part), (part, {}))[1][key] = tensors[name]
        for part, own in per_part.values():
            part.load(own, dtype)

    def setup(self, device, dtype):
        for _, part in self._children():
            part.setup(device, dtype)

    def forward(self, ctx, hidden, residual, cache, writes_cache=True):
        normed, residual = self.norm.forward_add(ctx, hidden, residual)
        mixed = self.mixer.forward(ctx, normed, cache, writes_cache)
        fed = self.feed_forward.forward(ctx, normed) if self.feed_forward is not None else None
        return ops.DeferredSum(mixed, fed), residual


register_part("arrangement", "parallel", ParallelBlock, replace=True)


class StreamPreNormBlock:
    """'pre_norm_stream': the pre-norm wiring over a float32 residual stream,

        x <- x + mixer(norm1(x));   x <- x + ff(norm2(x));   x <- x + token_input(x)

    with norms that keep the stream (`StreamRMSNorm`, `DynamicTanh`); the feed-forward and the token
    input (`LayerSpec.token_input`, a part of role "token_input" that reads the stream itself, not
    a normed copy) are optional. Adds are deferred like the other blocks': a block receives the
    stream and what the block before left to be added, its first norm adds while it reads, and
    it returns its last sublayer's output unadded.

    Checkpoint names: `LayerSpec.names` maps the roles "input_norm", "post_norm", "mixer",
    "feed_forward", "token_input" to name fragments; a norm's `weight` tensor is called by the
    fragment itself, every other tensor `<fragment>.<key>`."""

    def __init__(self, spec: LayerSpec, hidden_size: int):
        self.spec = spec
        if spec.position is not None:
            raise ConfigError("pre_norm_stream block: position encodings belong to the mixers that apply them")
        self.mixer = build_mixer(spec.mixer, hidden_size, None)
        self.feed_forward = build_feed_forward(spec.feed_forward, hidden_size)
        self.input_norm = build_norm(spec.norm, hidden_size)
        self.post_norm = build_norm(spec.norm, hidden_size) if self.feed_forward is not None else None
        self.token_input = build_token_input(spec.token_input, hidden_size)
        self.capture_safe = True

    def _children(self):
        n = self.spec.name_of
        yield n("input_norm"), self.input_norm
        yield n("mixer"), self.mixer
        if self.feed_forward is not None:
            yield n("post_norm"), self.post_norm
            yield n("feed_forward"), self.feed_forward
        if self.token_input is not None:
            yield n("token_input"), self.token_input

    def _names(self):
        """(checkpoint name relative to the layer, part, the part's key) for every tensor."""
        for fragment, part in self._children():
            for key in part.weight_specs():
                bare = isinstance(part, Norm) and key == "weight"
                yield (fragment if bare else f"{fragment}.{key}"), part, key

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {name: part.weight_specs()[key] for name, part, key in self._names()}

    def load(self, tensors, dtype):
        per_part = {}
        for name, part, key in self._names():
            if name in tensors:
                per_part.setdefault(id(part), (part, {}))[1][key] = tensors[name]
        for part, own in per_part.values():
            part.load(own, dtype)

    def setup(self, device, dtype):
        for _, part in self._children():
            part.setup(device, dtype)

    def forward(self, ctx, hidden, residual, cache, writes_cache=True):
        if residual is None and isinstance(hidden, torch.Tensor) and hidden.dtype == torch.float32:
            residual, normed = hidden, self.input_norm.forward(ctx, hidden)      # float32 embedding rows are the stream
        else:
            normed, residual = self.input_norm.forward_add(ctx, hidden, residual)
        out = self.mixer.forward(ctx, normed, cache, writes_cache)
        if self.feed_forward is not None:
            normed, residual = self.post_norm.forward_add(ctx, out, residual)
            out = self.feed_forward.forward(ctx, normed)
        if self.token_input is not None:
            # this sublayer reads the stream itself: the pending output is added now
            x = ops.rms_stream(out, None, 0.0, ctx.dtype, stream=residual, stream_out=residual)
            out = self.token_input.forward(ctx, x)
        return ops.DeferredSum(out), residual


register_part("arrangement", "pre_norm_stream", StreamPreNormBlock, replace=True)


class SandwichStreamBlock(StreamPreNormBlock):
    """'sandwich_stream': norms before and after every sublayer over a float32 residual stream, and
    an optional learned scale on what joins the stream,

        x <- x + s1 * out_norm1(mixer(norm1(x)));   x <- x + s2 * out_norm2(ff(norm2(x)))

    `LayerSpec.norm` names the norms before the sublayers, `LayerSpec.out_norm` those after them (a
    norm with `defer`, such as `LayerNormStream`); with `LayerSpec.layer_scale` the vectors s1, s2
    exist. Adds are deferred like the other blocks': a sublayer's output travels as an
    `ops.DeferredNormed` and the kernel of the next norm that reads the stream norms it, scales
    it, adds it and norms the sum, one launch per sublayer boundary.

    Checkpoint names: `LayerSpec.names` maps the roles "input_norm", "mixer_out_norm", "post_norm",
    "ff_out_norm", "mixer", "feed_forward", "mixer_scale", "ff_scale" to name fragments; a norm's
    `weight` tensor and a scale are called by the fragment itself, every other tensor
    `<fragment>.<key>`. A layer without a feed-forward has neither its norms nor its scale; a
    checkpoint may carry them all the same."""

    def __init__(self, spec: LayerSpec, hidden_size: int):
        super().__init__(spec, hidden_size)
        if spec.out_norm is None or spec.token_input is not None:
            raise ConfigError("sandwich_stream block: it needs an out_norm and takes no token input")
        self.mixer_out_norm = build_norm(spec.out_norm, hidden_size)
        self.ff_out_norm = build_norm(spec.out_norm, hidden_size)          # built also without a feed-forward: its tensors may be present
        if self.post_norm is None:
            self.unused_post_norm = build_norm(spec.norm, hidden_size)
        if not hasattr(self.mixer_out_norm, "defer"):
            raise ConfigError("sandwich_stream block: the out_norm must be one that can be deferred into the stream's kernel")
        self.scaled = bool(spec.layer_scale)
        self.mixer_scale = self.ff_scale = None

    def _children(self):
        n = self.spec.name_of
        yield n("input_norm"), self.input_norm
        yield n("mixer"), self.mixer
        yield n("mixer_out_norm"), self.mixer_out_norm
        if self.feed_forward is not None:
            yield n("post_norm"), self.post_norm
            yield n("feed_forward"), self.feed_forward
            yield n("ff_out_norm"), self.ff_out_norm

    def _scales(self):
        n = self.spec.name_of
        if self.scaled:
            yield n("mixer_scale"), "mixer_scale", False
            yield n("ff_scale"), "ff_scale", self.feed_forward is None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        import dataclasses
        specs = super().weight_specs()
        for name, _, unused in self._scales():
            specs[name] = WeightSpec((self.mixer.hidden_size,), init="norm", std=0.1, optional=unused)
        if self.feed_forward is None:
            # tensors of the absent sublayer: taken if the checkpoint has them, never read
            n = self.spec.name_of
            for fragment, part in ((n("post_norm"), self.unused_post_norm), (n("ff_out_norm"), self.ff_out_norm)):
                for key, w in part.weight_specs().items():
                    specs[fragment if key == "weight" else f"{fragment}.{key}"] = dataclasses.replace(w, optional=True)
        return specs

    def load(self, tensors, dtype):
        super().load(tensors, dtype)
        for name, attribute, unused in self._scales():
            setattr(self, attribute, None if unused else tensors[name])

    def forward(self, ctx, hidden, residual, cache, writes_cache=True):
        normed, residual = self.input_norm.forward_add(ctx, hidden, residual)
        out = self.mixer_out_norm.defer(self.mixer.forward(ctx, normed, cache, writes_cache), self.mixer_scale)
        if self.feed_forward is not None:
            normed, residual = self.post_norm.forward_add(ctx, out, residual)
            out = self.ff_out_norm.defer(self.feed_forward.forward(ctx, normed), self.ff_scale)
        return out, residual


register_part("arrangement", "sandwich_stream", SandwichStreamBlock, replace=True)


class PostNormStreamBlock(StreamPreNormBlock):
    """'post_norm_stream': the norm comes after the sum, over a float32 residual stream,

        x <- norm1(alpha * x + mixer(x));   x <- norm2(alpha * x + ff(x))

    with one constant alpha for the model (`LayerSpec.norm` parameter `alpha`, default 1; the other
    parameters are those of a root-mean-square norm: `eps`, `unit_offset`). The sublayers read x
    itself, rounded to the serving type. One kernel per sublayer boundary scales the stream, adds
    the sublayer's float32 output, norms, and writes the new stream and its rounding
    (`ops.post_norm_stream`); a block hands the next one both (`ops.StreamPair`) and no residual,
    so the model's final norm reads the stream alone. A layer without a feed-forward has no
    second step; a checkpoint may carry its norm all the same.

    Checkpoint names: `LayerSpec.names` maps the roles "input_norm" (norm1), "post_norm" (norm2),
    "mixer", "feed_forward" to name fragments; a norm's `weight` tensor is called by the fragment
    itself, every other tensor `<fragment>.<key>`."""

    def __init__(self, spec: LayerSpec, hidden_size: int):
        super().__init__(spec, hidden_size)
        if spec.token_input is not None or spec.out_norm is not None or spec.layer_scale:
            raise ConfigError("post_norm_stream block: it takes no token input, output norm or layer scale")
        self.alpha = float(spec.norm.get("alpha", 1.0))
        if self.post_norm is None:
            self.unused_post_norm = build_norm(spec.norm, hidden_size)
        for norm in (self.input_norm, self.post_norm):
            if norm is not None and not hasattr(norm, "offset"):
                raise ConfigError("post_norm_stream block: the norm must be a root-mean-square norm over the stream (rms_stream)")

    def weight_specs(self) -> Dict[str, WeightSpec]:
        import dataclasses
        specs = super().weight_specs()
        if self.feed_forward is None:
            fragment = self.spec.name_of("post_norm")
            for key, w in self.unused_post_norm.weight_specs().items():
                specs[fragment if key == "weight" else f"{fragment}.{key}"] = dataclasses.replace(w, optional=True)
        return specs

    def _after(self, ctx, norm, pair, y):
        return ops.post_norm_stream(pair.stream, y, norm.weight, self.alpha, norm.eps, ctx.dtype, offset=norm.offset)

    def forward(self, ctx, hidden, residual, cache, writes_cache=True):
        if residual is not None:
            raise ConfigError("post_norm_stream block: the block before it left a residual; it follows blocks of its own kind")
        if isinstance(hidden, ops.StreamPair):
            pair = hidden
        else:
            # the embedding's rows start the stream: float32 rows as they are, others widened
            hidden = ops.materialize(hidden)
            stream = hidden if hidden.dtype == torch.float32 else ops.stream_sum(None, hidden)
            rounded = stream if ctx.dtype == torch.float32 else (
                hidden if hidden.dtype == ctx.dtype else ops.stream_sum(stream, None, out_dtype=ctx.dtype))
            pair = ops.StreamPair(rounded, stream)
        pair = self._after(ctx, self.input_norm, pair, self.mixer.forward(ctx, pair.rounded, cache, writes_cache))
        if self.feed_forward is not None:
            pair = self._after(ctx, self.post_norm, pair, self.feed_forward.forward(ctx, pair.rounded))
        return pair, None


register_part("arrangement", "post_norm_stream", PostNormStreamBlock, replace=True)
