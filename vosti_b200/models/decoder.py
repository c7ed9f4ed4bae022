"""A decoder-only model put together from a `ModelSpec`: embedding, blocks in run
order, final norm, output head, each of them a part chosen by the spec.

The loop is the reference's (src/exec/dense_swiglu_model.rs:131-1041): embed; each
block maps (hidden, residual) to (hidden, residual); a last add-and-norm; rows that are
wanted are gathered and multiplied with the head, which is the embedding table when the
embeddings are tied. Logits are float32.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from ..config.schema import ModelSpec
from ..parts import Part, build_block, build_embedding, build_head, build_norm, build_reentry
from ..weights.loader import WeightSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.blocks = [build_block(layer, spec.hidden_size) for layer in spec.layers]
        self.final_norm = build_norm(spec.final_norm, spec.hidden_size)
        self.embedding = build_embedding(spec.embedding, spec.hidden_size, spec.vocab_size)
        self.head = build_head(spec.head, spec.hidden_size, spec.vocab_size, spec.tie_word_embeddings)
        self.reentry = build_reentry(spec.reentry, spec.hidden_size)
        # One cache (pages and state slot storage) per (layer, instance) that owns one. Cache i
        # belongs to layer i's first run; further runs of a layer get caches after those.
        self.cache_index = {(i, 0): i for i in range(len(self.blocks))}
        self.cache_layers = list(range(len(self.blocks)))
        for entry in spec.run_order:
            if entry.cache_from is None and (entry.layer, entry.instance) not in self.cache_index:
                self.cache_index[(entry.layer, entry.instance)] = len(self.cache_layers)
                self.cache_layers.append(entry.layer)
        # an embedding that keeps something per request gets state slots of its own, after the blocks' caches
        self.embedding_cache = len(self.cache_layers) if self.embedding.state_spec() is not None else None
        self.device = None
        self.dtype = None

    def parts(self):
        """Every part of the model."""
        yield self.embedding
        for block in self.blocks:
            for _, part in block._children():
                yield part
            position = getattr(block.mixer, "position", None)
            if position is not None:
                yield position
        yield self.final_norm
        yield self.head
        if self.reentry is not None:
            yield self.reentry

    def cache_specs(self):
        """(paged cache spec, state spec) of every cache in `cache_layers` order."""
        own = self.embedding_cache is not None
        return ([self.blocks[i].mixer.cache_spec() for i in self.cache_layers] + ([None] if own else []),
                [self.blocks[i].mixer.state_spec() for i in self.cache_layers] + ([self.embedding.state_spec()] if own else []))

    @property
    def capture_safe(self) -> bool:
        """Whether a decode step of this model may be recorded as a CUDA graph and replayed:
        every part must launch the same kernels with the same arguments for every step of a
        shape (see parts.base.Part.capture_safe)."""
        return all(getattr(part, "capture_safe", True) for part in self.parts()) and \
            all(getattr(block, "capture_safe", True) for block in self.blocks)

    # ------------------------------------------------------------ weights
    @staticmethod
    def _prefix_of(name: str) -> str:
        """'model.norm.weight' -> 'model.norm.': the names in a spec are those of a part's
        `weight` tensor; its other tensors (a bias) stand beside it."""
        return name[: -len("weight")] if name.endswith("weight") else name + "."

    @classmethod
    def _tensor_name(cls, name: str, key: str) -> str:
        """Checkpoint name of a model-level part's tensor `key`, given the name of its `weight`."""
        return name if key == "weight" else cls._prefix_of(name) + key

    @classmethod
    def _part_tensor_name(cls, name: str, part, key: str) -> str:
        """The same, unless the part's spec names the tensor outright (parameter `names`: pairs of
        (key, checkpoint name))."""
        named = dict(part.spec.get("names") or ())
        return named[key] if key in named else cls._tensor_name(name, key)

    @classmethod
    def _own(cls, tensors, name: str, part):
        """The tensors of a model-level part, by the part's own keys."""
        return {key: tensors[cls._part_tensor_name(name, part, key)] for key in part.weight_specs()
                if cls._part_tensor_name(name, part, key) in tensors}

    def expected_weights(self) -> Dict[str, WeightSpec]:
        spec = self.spec
        out = {self._part_tensor_name(spec.embed_name, self.embedding, key): w
               for key, w in self.embedding.weight_specs().items()}
        for i, block in enumerate(self.blocks):
            prefix = spec.layer_prefix.format(i=i)
            for key, w in block.weight_specs().items():
                out[prefix + key] = w
        for key, w in self.final_norm.weight_specs().items():
            out[self._tensor_name(spec.final_norm_name, key)] = w
        for key, w in self.head.weight_specs().items():
            out[self._tensor_name(spec.lm_head_name, key)] = w
        if self.reentry is not None:
            for key, w in self.reentry.weight_specs().items():
                out[self._tensor_name(spec.reentry_name, key)] = w
        return out

    def ignorable_weights(self):
        """Tensors a checkpoint may carry that this model does not read."""
        return (self.spec.lm_head_name,) if self.spec.tie_word_embeddings else ()

    def tied_weights(self) -> Dict[str, str]:
        """Tensors a checkpoint may carry although this model reads another in their place,
        mapped to that other tensor: if present they must hold the same values."""
        spec = self.spec
        return {spec.lm_head_name: spec.embed_name} if spec.tie_word_embeddings else {}

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype) -> None:
        spec = self.spec
        under = lambda prefix: {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}
        self.embedding.load(self._own(tensors, spec.embed_name, self.embedding), dtype)
        for i, block in enumerate(self.blocks):
            block.load(under(spec.layer_prefix.format(i=i)), dtype)
        self.final_norm.load(self._own(tensors, spec.final_norm_name, self.final_norm), dtype)
        self.head.load(self._own(tensors, spec.lm_head_name, self.head), dtype,
                       tied=self.embedding.table() if spec.tie_word_embeddings else None)
        if self.reentry is not None:
            self.reentry.load(self._own(tensors, spec.reentry_name, self.reentry), dtype)
        self.device = next(iter(tensors.values())).device
        self.dtype = dtype
        for part in (self.embedding, self.final_norm, self.head) + ((self.reentry,) if self.reentry is not None else ()):
            part.setup(self.device, dtype)
        for block in self.blocks:
            block.setup(self.device, dtype)

    def weight_bytes(self) -> int:
        """Bytes of every distinct weight tensor one step reads whole: the blocks, the final
        norm and the head. The embedding table is not among them (a step reads one row per
        token) unless the head is tied to it."""
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            for value in vars(obj).values():
                if isinstance(value, ops.PackedWeight):
                    value = value.data
                if isinstance(value, torch.Tensor) and value.is_cuda:
                    base = value.untyped_storage().data_ptr()
                    if base not in seen:
                        seen.add(base)
                        total += value.untyped_storage().nbytes()
                elif isinstance(value, (list, tuple)):
                    # parts inside a part (the branches of a mixer) and lists of tensors
                    for item in value:
                        for inner in (item if isinstance(item, tuple) else (item,)):
                            if isinstance(inner, Part):
                                visit(inner)
                            elif isinstance(inner, torch.Tensor) and inner.is_cuda:
                                base = inner.untyped_storage().data_ptr()
                                if base not in seen:
                                    seen.add(base)
                                    total += inner.untyped_storage().nbytes()
        for block in self.blocks:
            for _, part in block._children():
                visit(part)
        visit(self.final_norm)
        if self.reentry is not None:
            visit(self.reentry)
        visit(self.head)          # a tied head is the embedding table, read whole by the head's product
        return total

    # ------------------------------------------------------------ forward
    def forward(self, ctx, layer_caches: List):
        """Run every entry of the run order over the batch in `ctx`; returns the last
        block's (hidden, residual), both [T, hidden] (residual None without blocks)."""
        source = ctx.extras.get("feedback") if ctx.extras else None
        feedback = None if source is None else (source, ctx.feedback_values)
        if self.embedding_cache is not None:
            hidden = self.embedding.forward(ctx, ctx.tokens, feedback=feedback, cache=layer_caches[self.embedding_cache])
        else:
            hidden = self.embedding.forward(ctx, ctx.tokens, feedback=feedback)
        first = hidden                      # the embedding output, which a re-entry reads again
        residual: Optional[torch.Tensor] = None
        for entry in self.spec.run_order:
            owner = entry.layer if entry.cache_from is None else entry.cache_from
            if entry.reenter:
                hidden, residual = self.reentry.forward(ctx, hidden, residual, first)
            hidden, residual = self.blocks[entry.layer].forward(
                ctx, hidden, residual, layer_caches[self.cache_index[(owner, entry.instance)]],
                writes_cache=entry.cache_from is None)
        return hidden, residual

    def logits(self, ctx, hidden: torch.Tensor, residual: Optional[torch.Tensor], rows: torch.Tensor) -> torch.Tensor:
        """float32 logits [len(rows), vocab] of the rows (flat token indices) asked for:
        only those rows are gathered, added, normed and multiplied with the head."""
        if isinstance(hidden, ops.DeferredNormed):
            # a sublayer output still to be normed, scaled and added: only the wanted rows are
            hidden = hidden.rows(rows, ctx.status)
            return self.head.forward(ctx, self.final_norm.forward_add(ctx, hidden, ops.gather_rows(residual, rows, ctx.status))[0])
        if isinstance(hidden, ops.DeferredSum):
            # a float32 stream with sublayer outputs still to be added: add, then gather
            hidden, residual = ops.stream_sum(residual, hidden), None
        hidden = ops.gather_rows(ops.materialize(hidden), rows, ctx.status)
        if residual is None:
            final = self.final_norm.forward(ctx, hidden)
        else:
            final = self.final_norm.forward_add(ctx, hidden, ops.gather_rows(residual, rows, ctx.status))[0]
        return self.head.forward(ctx, final)
