"""The decoder put together from parts: embedding (and the spec's hook after it), the layer calls of
`ModelSpec.order`, final norm on the wanted rows only, LM head in 32-bit logits (and the spec's hook on
them).  How one layer arranges its parts is a registered block kind named by the layer's spec
("pre_norm": x += mixer(norm1(x)); x += ffn(norm2(x))), and the run order is a list of the spec; the
reference hard-codes both in its parser (tiny_llm/parser/llama_parser.cpp:181-271)."""
from __future__ import annotations

from typing import Dict, List

import torch

from .. import ops
from ..config.spec import LayerSpec, ModelSpec
from ..weights import COMPUTE, WeightSpec
from .registry import build_block, build_part, register_block


class Block:
    """The pre-norm residual block: x += s * mixer(norm1(x)); x += s * ffn(norm2(x)), with s the layer's
    `residual_scale` (the parts take it as `out_scale` and fold it into their output matrices).  A layer without
    a feed-forward names neither `ffn` nor `norm2` and ends after the first line."""

    def __init__(self, spec: LayerSpec, shares_cache: bool = False):
        for role in ("norm1", "mixer"):
            if getattr(spec, role) is None:
                raise ValueError(f"layer {spec.prefix!r}: a pre_norm block needs a {role}")
        if (spec.ffn is None) != (spec.norm2 is None):
            raise ValueError(f"layer {spec.prefix!r}: a pre_norm block has a norm2 exactly when it has a feed-forward")
        self.spec = spec
        scale = {} if spec.residual_scale == 1.0 else {"out_scale": spec.residual_scale}
        self.norm1 = build_part("norm", spec.norm1)
        self.mixer = build_part("mixer", spec.mixer, **scale, **({"shares_cache": True} if shares_cache else {}))
        self.norm2 = None if spec.ffn is None else build_part("norm", spec.norm2)
        self.ffn = None if spec.ffn is None else build_part("ffn", spec.ffn, **scale)

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None]

    def _prefixes(self):
        p = self.spec.prefix
        return p + self.spec.norm1_name, p + self.spec.mixer_prefix, p + self.spec.norm2_name, p + self.spec.ffn_prefix

    def weight_specs(self) -> List[WeightSpec]:
        n1, mx, n2, ff = self._prefixes()
        specs = self.norm1.weight_specs(n1) + self.mixer.weight_specs(mx)
        if self.ffn is not None:
            specs += self.norm2.weight_specs(n2) + self.ffn.weight_specs(ff)
        return specs

    def load(self, weights) -> None:
        n1, mx, n2, ff = self._prefixes()
        self.norm1.load(n1, weights)
        self.mixer.load(mx, weights)
        if self.ffn is not None:
            self.norm2.load(n2, weights)
            self.ffn.load(ff, weights)

    def forward(self, ctx, resid, cache) -> None:
        h = self.norm1.forward(ctx, resid)
        self.mixer.forward(ctx, h, resid, cache)
        if self.ffn is not None:
            h = self.norm2.forward(ctx, resid)
            self.ffn.forward(ctx, h, resid)


register_block("pre_norm", Block)


class SandwichBlock:
    """Norms on both sides of each branch: x += norm1_out(mixer(norm1(x))); x += norm2_out(ffn(norm2(x))).  The two
    norms behind the branches are named in `LayerSpec.more` under the roles "norm1_out" and "norm2_out" (the second
    only when the layer has a feed-forward).  A branch adds its output into a zeroed float32 buffer, whose norm is
    then added into the stream by one kernel that also hands the buffer back zeroed."""

    def __init__(self, spec: LayerSpec, shares_cache: bool = False):
        more = {role: (family, part, name) for role, family, part, name in spec.more}
        for role in ("norm1", "mixer"):
            if getattr(spec, role) is None:
                raise ValueError(f"layer {spec.prefix!r}: a sandwich block needs a {role}")
        if "norm1_out" not in more or (spec.ffn is not None) != ("norm2_out" in more) or \
                (spec.ffn is None) != (spec.norm2 is None):
            raise ValueError(f"layer {spec.prefix!r}: a sandwich block has a norm behind each of its branches "
                             f"(roles norm1_out, norm2_out) and one ahead of it")
        if spec.residual_scale != 1.0:
            raise ValueError(f"layer {spec.prefix!r}: a normed branch has no use for a residual scale")
        self.spec = spec
        self.norm1 = build_part("norm", spec.norm1)
        self.mixer = build_part("mixer", spec.mixer, **({"shares_cache": True} if shares_cache else {}))
        self.norm1_out = build_part("norm", more["norm1_out"][1])
        self.norm2 = self.ffn = self.norm2_out = None
        if spec.ffn is not None:
            self.norm2 = build_part("norm", spec.norm2)
            self.ffn = build_part("ffn", spec.ffn)
            self.norm2_out = build_part("norm", more["norm2_out"][1])
        self._out_names = {role: more[role][2] for role in ("norm1_out", "norm2_out") if role in more}
        self.hidden_size = None

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm1_out, self.norm2, self.ffn, self.norm2_out) if p is not None]

    def _named(self):
        p, s = self.spec.prefix, self.spec
        named = [(self.norm1, p + s.norm1_name), (self.mixer, p + s.mixer_prefix), (self.norm1_out, p + self._out_names["norm1_out"])]
        if self.ffn is not None:
            named += [(self.norm2, p + s.norm2_name), (self.ffn, p + s.ffn_prefix), (self.norm2_out, p + self._out_names["norm2_out"])]
        return named

    def weight_specs(self) -> List[WeightSpec]:
        return [w for part, name in self._named() for w in part.weight_specs(name)]

    def load(self, weights) -> None:
        for part, name in self._named():
            part.load(name, weights)

    def forward(self, ctx, resid, cache) -> None:
        h = self.norm1.forward(ctx, resid)
        branch = ctx.workspace.get_zeroed("branch_out", tuple(resid.shape))
        self.mixer.forward(ctx, h, branch, cache)
        self.norm1_out.add_into(ctx, branch, resid)
        if self.ffn is not None:
            h = self.norm2.forward(ctx, resid)
            self.ffn.forward(ctx, h, branch)
            self.norm2_out.add_into(ctx, branch, resid)


register_block("sandwich_norm", SandwichBlock)


class BranchNormBlock:
    """A norm BEHIND each branch only: x += norm1(mixer(x)); x += norm2(ffn(x)).  The branches read the stream itself
    (rounded to the engine's dtype where that is not float32; the float32 engine hands them the stream as it is); a
    branch adds its output into a zeroed float32 buffer, whose norm one kernel adds into the stream, handing the
    buffer back zeroed.  That kernel also leaves the new stream rounded to bfloat16 for the next branch to read
    (`ctx.stream_copy`, which names the stream it is a copy of; whoever else changes the stream drops it), so only a
    layer behind something else pays a copy kernel.  `norm1` and `norm2` of the layer's spec are these norms."""

    leaves_stream_copy = True    # the model keeps `ctx.stream_copy` across this block (any other block drops it)

    def __init__(self, spec: LayerSpec, shares_cache: bool = False):
        for role in ("norm1", "mixer"):
            if getattr(spec, role) is None:
                raise ValueError(f"layer {spec.prefix!r}: a branch_norm block needs a {role}")
        if (spec.ffn is None) != (spec.norm2 is None):
            raise ValueError(f"layer {spec.prefix!r}: a branch_norm block has a norm2 exactly when it has a feed-forward")
        if spec.residual_scale != 1.0:
            raise ValueError(f"layer {spec.prefix!r}: a normed branch has no use for a residual scale")
        self.spec = spec
        self.norm1 = build_part("norm", spec.norm1)
        self.mixer = build_part("mixer", spec.mixer, **({"shares_cache": True} if shares_cache else {}))
        self.norm2 = None if spec.ffn is None else build_part("norm", spec.norm2)
        self.ffn = None if spec.ffn is None else build_part("ffn", spec.ffn)

    def parts(self):
        return [p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None]

    def _named(self):
        p, s = self.spec.prefix, self.spec
        named = [(self.norm1, p + s.norm1_name), (self.mixer, p + s.mixer_prefix)]
        if self.ffn is not None:
            named += [(self.norm2, p + s.norm2_name), (self.ffn, p + s.ffn_prefix)]
        return named

    def weight_specs(self) -> List[WeightSpec]:
        return [w for part, name in self._named() for w in part.weight_specs(name)]

    def load(self, weights) -> None:
        for part, name in self._named():
            part.load(name, weights)

    @staticmethod
    def _input(ctx, resid):
        if ctx.dtype == torch.float32:
            return resid
        held = getattr(ctx, "stream_copy", None)
        if held is not None and held[0] == resid.data_ptr() and tuple(held[1].shape) == tuple(resid.shape):
            return held[1]
        h = ctx.workspace.get("stream_copy", tuple(resid.shape), ctx.dtype)
        ops.unary(resid, h)
        return h

    @staticmethod
    def _join(ctx, norm, branch, resid):
        copy = None if ctx.dtype != torch.bfloat16 else ctx.workspace.get("stream_copy", tuple(resid.shape), ctx.dtype)
        norm.add_into(ctx, branch, resid, copy=copy)
        ctx.stream_copy = None if copy is None else (resid.data_ptr(), copy)

    def forward(self, ctx, resid, cache) -> None:
        branch = ctx.workspace.get_zeroed("branch_out", tuple(resid.shape))
        self.mixer.forward(ctx, self._input(ctx, resid), branch, cache)
        self._join(ctx, self.norm1, branch, resid)
        if self.ffn is not None:
            self.ffn.forward(ctx, self._input(ctx, resid), branch)
            self._join(ctx, self.norm2, branch, resid)


register_block("branch_norm", BranchNormBlock)


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        for pos, call in enumerate(spec.order):
            if not 0 <= call.layer < len(spec.layers):
                raise ValueError(f"run order entry {pos} names layer {call.layer}, the model has {len(spec.layers)}")
            if call.reads_cache_of is not None and not 0 <= call.reads_cache_of < pos:
                raise ValueError(f"run order entry {pos} reads the cache of entry {call.reads_cache_of}, "
                                 f"which does not run before it")
        if spec.embedding_scale != 1.0 and any(c.add_embedding for c in spec.order):
            raise ValueError("a run order that adds the embedding output again takes the table's rows as they are")
        if spec.after_embedding is not None and any(c.add_embedding for c in spec.order):
            raise ValueError("a run order that adds the embedding output again cannot be combined with a hook that "
                             "rewrites the stream after the embedding")
        shared = {c.layer for c in spec.order if c.reads_cache_of is not None}
        owning = {c.layer for c in spec.order if c.reads_cache_of is None}
        if shared & owning:
            raise ValueError(f"layers {sorted(shared & owning)} are run both with a cache of their own and with another's")
        self.blocks = [build_block(ls, shares_cache=(i in shared)) for i, ls in enumerate(spec.layers)]
        self.final_norm = build_part("norm", spec.final_norm)
        self.after_embedding = None if spec.after_embedding is None else build_part("hook", spec.after_embedding)
        self.on_logits = None if spec.on_logits is None else build_part("hook", spec.on_logits)
        self._hook_keeps = self.after_embedding is not None and hasattr(self.after_embedding, "cache_need")
        self.embed = None
        self.lm_head = None
        self.loaded = False
        # a callable(position in the run order, float32 stream [T, H]) called after every layer call: for tests and
        # debugging only (a runner built around a model with a probe must not capture or tape its steps)
        self.probe = None
        # a part that synchronises or computes on the host must not be captured; parts say so themselves
        parts = [self.final_norm] + [x for b in self.blocks for x in b.parts()] + \
            [h for h in (self.after_embedding, self.on_logits) if h is not None]
        self.graph_safe = all(getattr(x, "graph_safe", False) for x in parts)

    # ---- what the model wants from the weights and the cache
    def weight_specs(self) -> Dict[str, WeightSpec]:
        s = self.spec
        specs = [WeightSpec(s.embed_name, (s.vocab_size, s.hidden_size), COMPUTE)]
        for b in self.blocks:
            specs += b.weight_specs()
        specs += self.final_norm.weight_specs(s.final_norm_name)
        if self.after_embedding is not None:
            specs += self.after_embedding.weight_specs(s.after_embedding_name)
        if self.on_logits is not None:
            specs += self.on_logits.weight_specs(s.on_logits_name)
        if not s.tie_word_embeddings:
            # a checkpoint without an output matrix uses the embedding table for it
            specs.append(WeightSpec(s.lm_head_name, (s.vocab_size, s.hidden_size), COMPUTE, alias_of=s.embed_name))
        out = {}
        for w in specs:
            if w.name in out and out[w.name] != w:
                raise ValueError(f"two parts want tensor {w.name!r} with different shapes")
            out[w.name] = w
        return out

    def cache_needs(self):
        """One need per run-order entry; None for an entry that reads another entry's cache or needs none.  A hook
        after the embedding that keeps something per request adds one more entry at the end."""
        def need(block):
            return None if block.mixer is None else block.mixer.cache_need()
        needs = [None if c.reads_cache_of is not None else need(self.blocks[c.layer]) for c in self.spec.order]
        if self._hook_keeps:   # what the hook after the embedding keeps per request comes behind the layer calls' entries
            needs.append(self.after_embedding.cache_need())
        return needs

    def load(self, weights: Dict[str, torch.Tensor]) -> None:
        s = self.spec
        self.embed = weights[s.embed_name]
        for b in self.blocks:
            b.load(weights)
        self.final_norm.load(s.final_norm_name, weights)
        if self.after_embedding is not None:
            self.after_embedding.load(s.after_embedding_name, weights)
        if self.on_logits is not None:
            self.on_logits.load(s.on_logits_name, weights)
        self.lm_head = self.embed if s.tie_word_embeddings else weights[s.lm_head_name]
        self.loaded = True

    # ---- one step
    def forward(self, ctx) -> torch.Tensor:
        """Runs the step's tokens through every layer call; returns float32 logits at
        `ctx.batch.logit_rows` ([n_out, vocab]), or None when no row is wanted."""
        s = self.spec
        b = ctx.batch
        resid = ctx.workspace.get("resid", (b.num_tokens, s.hidden_size), torch.float32)
        ops.embedding(b.tokens, self.embed, resid, scale=s.embedding_scale)
        ctx.stream_copy = None     # a rounded copy of the stream that a block may leave for the next one
        if self._hook_keeps:
            self.after_embedding.forward(ctx, resid, ctx.cache_view(len(s.order)))
        elif self.after_embedding is not None:
            self.after_embedding.forward(ctx, resid)
        for pos, call in enumerate(s.order):
            owner = pos if call.reads_cache_of is None else call.reads_cache_of
            if call.add_embedding:   # the embedding output is the table's rows again: gathered and added in one kernel
                ops.embedding(b.tokens, self.embed, resid, accumulate=True)
                ctx.stream_copy = None
            self.blocks[call.layer].forward(ctx, resid, ctx.cache_view(owner))
            if not getattr(self.blocks[call.layer], "leaves_stream_copy", False):
                ctx.stream_copy = None
            if self.probe is not None:
                self.probe(pos, resid)
        if b.num_logits == 0:
            return None
        h = self.final_norm.forward(ctx, resid, rows=b.logit_rows)
        logits = ctx.workspace.get("logits", (b.num_logits, s.vocab_size), torch.float32)
        ops.linear(h, self.lm_head, logits)
        if self.on_logits is not None:
            self.on_logits.forward(ctx, logits)
        return logits
