"""Typed configuration of Gevovik, a small decoder that adds a hashed bigram row to every token's embedding, norms what
a branch gives instead of what it reads (x += n(mixer(x)); x += n(ff(x)), every norm with ONE learned number), and mixes
tokens in one of three ways per layer: a state-space recurrence with a scalar decay per head (`mamba2`); latent
attention with a sink in the softmax, whose layers may read the latents that an earlier layer cached
(`latent_attention`); or two mixers side by side on the same input, summed with fixed factors (`parallel`): a windowed
grouped-query attention with normed and rotated queries and keys, scores mixed across the heads before the softmax and
a gate per head, beside a gated delta rule with a decay per key channel.  Feed-forwards are two matrices around
relu(.)^2.

config.json keys (every size and every constant that differs between models of the design comes from here):

  architecture      "Gevovik"
  vocab, width      vocabulary and width of the residual stream
  embedding.scale   what the embedding rows are multiplied by
  embedding.bigram  {"buckets", "mul_prev", "mul_cur"} | absent: row (prev * mul_prev + cur * mul_cur) mod buckets of
                    the tensor `bigram` is added; a sequence's first token takes row `buckets`
  norm.eps          eps of every RMS norm (the layers', the per-head ones, the latent's, the parts' of mamba2)
  layers[i]         {"type": "mamba2" | "latent_attention" | "parallel", "mixer": {...}, "mlp": {...} | null}
    mamba2            {"heads", "vdim", "state", "groups", "norm_groups", "conv"}
    latent_attention  {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot": {"dims", "base", "scaling"?},
                       "kv_from": j | absent}   (with kv_from the layer has no `dkv` and reads layer j's cache)
    parallel          {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"} | absent,
                                "rot": {"dims", "base", "scaling": {"factor", "original", "fast", "slow"}?} | absent},
                       "right": {"heads", "kv_heads", "dim", "vdim", "conv"}, "left_scale", "right_scale"}
    mlp               {"kind": "dense", "ff"}

Tensor names: `embed`, `bigram`, `head`, `final.norm`, and per layer `l<i>.norm1`, `l<i>.norm2` (one number each),
`l<i>.mix.*` (`l<i>.mix.left.*` and `l<i>.mix.right.*` for a parallel mixer), `l<i>.mlp.up|down`."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .dunelix import DEFAULT_MAX_POSITIONS, _need, _number, _pos_int
from .errors import ConfigError
from .registry import register_architecture
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec

MIXERS = ("mamba2", "latent_attention", "parallel")


def _check_rot(rot: dict, limit: int, where: str) -> None:
    dims = _pos_int(rot, "dims", where)
    if dims % 2 or dims > limit:
        raise ConfigError(f'config.json: {where}: "dims" ({dims}) must be even and at most {limit}')
    if _number(rot, "base", where) <= 0:
        raise ConfigError(f'config.json: {where}: "base" must be positive')
    sc = rot.get("scaling")
    if sc is not None:
        for k in ("factor", "original", "fast", "slow"):
            if _number(sc, k, where + ".scaling") <= 0:
                raise ConfigError(f'config.json: {where}.scaling: "{k}" must be positive')
        if rot["base"] == 1:
            raise ConfigError(f'config.json: {where}: a scaled rotation needs a "base" other than 1')


def _check_mamba2(m: dict, where: str) -> None:
    heads, groups = _pos_int(m, "heads", where), _pos_int(m, "groups", where)
    if heads % groups:
        raise ConfigError(f'config.json: {where}: "heads" ({heads}) must be a multiple of "groups" ({groups})')
    vdim, parts = _pos_int(m, "vdim", where), _pos_int(m, "norm_groups", where)
    if (heads * vdim) % parts:
        raise ConfigError(f'config.json: {where}: "norm_groups" ({parts}) must divide heads * vdim ({heads * vdim})')
    _pos_int(m, "state", where)
    _pos_int(m, "conv", where)


def _check_latent(m: dict, where: str, index: int, layers: list) -> None:
    for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
        _pos_int(m, k, where)
    _number(m, "scale", where)
    if m.get("rot") is not None:
        _check_rot(m["rot"], m["rot_dim"], where + ".rot")
    src = m.get("kv_from")
    if src is not None:
        if not isinstance(src, int) or isinstance(src, bool) or not 0 <= src < index:
            raise ConfigError(f'config.json: {where}: "kv_from" must name an earlier layer, found {src!r}')
        other = layers[src]
        if other.get("type") != "latent_attention" or other["mixer"].get("kv_from") is not None:
            raise ConfigError(f'config.json: {where}: "kv_from" names layer {src}, which keeps no latents of its own')
        for k in ("kv_rank", "rot_dim", "rot"):
            if other["mixer"].get(k) != m.get(k):
                raise ConfigError(f'config.json: {where}: "{k}" differs from layer {src}, whose cache this layer reads')


def _check_parallel(m: dict, where: str) -> None:
    left, right = _need(m, "left", where), _need(m, "right", where)
    for side, d in (("left", left), ("right", right)):
        heads, kv = _pos_int(d, "heads", f"{where}.{side}"), _pos_int(d, "kv_heads", f"{where}.{side}")
        if heads % kv:
            raise ConfigError(f'config.json: {where}.{side}: "heads" ({heads}) must be a multiple of "kv_heads" ({kv})')
        _pos_int(d, "dim", f"{where}.{side}")
        _pos_int(d, "vdim", f"{where}.{side}")
    _number(left, "scale", where + ".left")
    if left.get("mask") is not None:
        _pos_int(left["mask"], "size", where + ".left.mask")
    if left.get("rot") is not None:
        _check_rot(left["rot"], left["dim"], where + ".left.rot")
    _pos_int(right, "conv", where + ".right")
    _number(m, "left_scale", where)
    _number(m, "right_scale", where)


@dataclass(frozen=True)
class GevovikConfig:
    vocab: int
    width: int
    embedding_scale: float
    bigram: Optional[Tuple[int, int, int]]      # (buckets, mul_prev, mul_cur)
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]
    eos_token_ids: Tuple[int, ...] = ()
    initializer_range: float = 0.06

    architecture = "Gevovik"

    @classmethod
    def from_dict(cls, d: dict) -> "GevovikConfig":
        vocab, width = _pos_int(d, "vocab", "top level"), _pos_int(d, "width", "top level")
        layers_in = _need(d, "layers", "top level")
        if not isinstance(layers_in, list) or not layers_in:
            raise ConfigError('config.json: "layers" must be a non-empty list')
        layers = []
        for i, l in enumerate(layers_in):
            where = f"layers[{i}]"
            kind, mixer = _need(l, "type", where), _need(l, "mixer", where)
            if kind == "mamba2":
                _check_mamba2(mixer, where + ".mixer")
            elif kind == "latent_attention":
                _check_latent(mixer, where + ".mixer", i, layers_in)
            elif kind == "parallel":
                _check_parallel(mixer, where + ".mixer")
            else:
                raise ConfigError(f'config.json: {where}: unknown mixer type {kind!r} (known: {", ".join(MIXERS)})')
            mlp = l.get("mlp")
            if mlp is not None:
                if _need(mlp, "kind", where + ".mlp") != "dense":
                    raise ConfigError(f'config.json: {where}.mlp: unknown kind {mlp["kind"]!r} (known: dense)')
                _pos_int(mlp, "ff", where + ".mlp")
            layers.append(copy.deepcopy({"type": kind, "mixer": mixer, "mlp": mlp}))
        emb = d.get("embedding") or {}
        big = emb.get("bigram")
        bigram = None
        if big is not None:
            bigram = (_pos_int(big, "buckets", "embedding.bigram"), int(_number(big, "mul_prev", "embedding.bigram")),
                      int(_number(big, "mul_cur", "embedding.bigram")))
            if bigram[1] < 0 or bigram[2] < 0:
                raise ConfigError('config.json: embedding.bigram: "mul_prev" and "mul_cur" must not be negative')
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab=vocab, width=width,
                   embedding_scale=_number(emb, "scale", "embedding") if emb.get("scale") is not None else 1.0,
                   bigram=bigram, norm_eps=_number(_need(d, "norm", "top level"), "eps", "norm"), layers=tuple(layers),
                   eos_token_ids=eos_ids, initializer_range=float(d.get("initializer_range", 0.06)))

    def to_dict(self) -> dict:
        emb: Dict[str, Any] = {"scale": self.embedding_scale}
        if self.bigram is not None:
            emb["bigram"] = {"buckets": self.bigram[0], "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]}
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "embedding": emb,
             "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(list(self.layers)),
             "initializer_range": self.initializer_range}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def _mixer(self, l: dict) -> PartSpec:
        m, w, eps = l["mixer"], self.width, self.norm_eps
        if l["type"] == "mamba2":
            return PartSpec("mamba2", {"hidden_size": w, "num_heads": m["heads"], "value_dim": m["vdim"],
                                       "state_dim": m["state"], "groups": m["groups"], "taps": m["conv"],
                                       "norm_parts": m["norm_groups"], "eps": eps})
        if l["type"] == "latent_attention":
            rot = m.get("rot") or {}
            return PartSpec("latent_attention", {
                "hidden_size": w, "num_heads": m["heads"], "plain_dim": m["dim"], "rot_part": m["rot_dim"],
                "value_dim": m["vdim"], "rank": m["kv_rank"], "scale": float(m["scale"]), "eps": eps,
                "rot_dims": rot.get("dims", 0), "rot_base": float(rot.get("base", 10000.0)),
                "rot_scaling": rot.get("scaling"), "window": None, "sink": True, "gate": False})
        left, right = m["left"], m["right"]
        rot = left.get("rot") or {}
        left_spec = PartSpec("sink_attention", {
            "hidden_size": w, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"], "key_dim": left["dim"],
            "value_dim": left["vdim"], "scale": float(left["scale"]), "eps": eps, "bias": False, "qk_norm": True,
            "sink": False, "gate": "head", "window": (left.get("mask") or {}).get("size"),
            "rot_dims": rot.get("dims", 0), "rot_base": float(rot.get("base", 10000.0)),
            "rot_scaling": rot.get("scaling"), "rot_layout": "halves", "head_temp": True, "talk": True})
        right_spec = PartSpec("gated_delta_rule", {
            "hidden_size": w, "num_heads": right["heads"], "num_kv_heads": right["kv_heads"], "key_dim": right["dim"],
            "value_dim": right["vdim"], "taps": right["conv"], "eps": eps, "decay": "channel", "gate_act": "sigmoid",
            "gate_low_rank": True})
        return PartSpec("side_by_side", {
            "hidden_size": w, "norm": False, "branches": (("left.", left_spec), ("right.", right_spec)),
            "weights": (float(m["left_scale"]), float(m["right_scale"]))})

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rms_norm", {"size": self.width, "eps": self.norm_eps, "weight_suffix": "", "scalar": True})
        layers: List[LayerSpec] = []
        order: List[LayerCall] = []
        for i, l in enumerate(self.layers):
            ffn = None
            if l["mlp"] is not None:
                ffn = PartSpec("dense_mlp", {"hidden_size": self.width, "intermediate_size": l["mlp"]["ff"],
                                             "names": ("up", "down"), "act": "relu2"})
            layers.append(LayerSpec(prefix=f"l{i}.", norm1=norm, mixer=self._mixer(l), norm2=norm if ffn else None,
                                    ffn=ffn, mixer_prefix="mix.", ffn_prefix="mlp.", norm1_name="norm1",
                                    norm2_name="norm2", block="branch_norm"))
            order.append(LayerCall(i, reads_cache_of=l["mixer"].get("kv_from") if l["type"] == "latent_attention" else None))
        hook = None
        if self.bigram is not None:
            hook = PartSpec("bigram_embedding", {"size": self.width, "buckets": self.bigram[0],
                                                 "mul_prev": self.bigram[1], "mul_cur": self.bigram[2]})
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=DEFAULT_MAX_POSITIONS, layers=layers, order=order, final_norm=norm, embed_name="embed",
            final_norm_name="final.norm", lm_head_name="head", tie_word_embeddings=False,
            eos_token_ids=self.eos_token_ids, initializer_range=self.initializer_range,
            embedding_scale=self.embedding_scale, after_embedding=hook, after_embedding_name="bigram")


register_architecture(GevovikConfig.architecture, GevovikConfig)
