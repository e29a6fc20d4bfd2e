"""Typed configuration of Fiponex, a small decoder whose layers norm both sides of every branch and mix tokens in
one of three ways: grouped-query attention with normed queries and keys, a sink in the softmax and a gated output;
latent attention (keys and values projected from one small cached vector per token, a rotated key part shared by the
heads, a sliding window, the same sink and a gate per head); or the gated delta rule (a matrix state per head behind
short convolutions).  Feed-forwards are dense gated layers or mixtures of small gated experts behind a softmax router.
The embedding is multiplied by a constant.

config.json keys (every size and every constant that differs between models of the design comes from here):

  architecture      "Fiponex"
  vocab, width      vocabulary and width of the residual stream
  embedding.scale   what the embedding rows are multiplied by
  norm.eps          eps of every RMS norm (the layers', the per-head ones and the latent's)
  layers[i]         {"type": "attention" | "latent_attention" | "delta", "mixer": {...}, "mlp": {...} | null}
    attention         {"heads", "kv_heads", "dim", "vdim", "scale", "q_temp": {"coef", "every"} | absent}
    latent_attention  {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "mask": {"size"} | absent,
                       "rot": {"dims", "base"} | absent}
    delta             {"heads", "kv_heads", "dim", "vdim", "conv"}
    mlp               {"kind": "dense", "ff"}  or  {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}}

Tensor names: `embed`, `head`, `final.norm`, and per layer `l<i>.norm1`, `l<i>.norm1b`, `l<i>.norm2`, `l<i>.norm2b`,
`l<i>.mix.*`, `l<i>.mlp.gate|up|down` or `l<i>.mlp.router`, `l<i>.mlp.e<j>.gate|up|down`."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Tuple

from .dunelix import DEFAULT_MAX_POSITIONS, _need, _number, _pos_int
from .errors import ConfigError
from .registry import register_architecture
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec

MIXERS = ("attention", "latent_attention", "delta")


def _check_attention(m: dict, where: str) -> None:
    heads, kv = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f'config.json: {where}: "heads" ({heads}) must be a multiple of "kv_heads" ({kv})')
    _pos_int(m, "dim", where)
    _pos_int(m, "vdim", where)
    _number(m, "scale", where)
    qt = m.get("q_temp")
    if qt is not None:
        _number(qt, "coef", where + ".q_temp")
        every = _number(qt, "every", where + ".q_temp")
        if every < 1 or every != int(every):
            raise ConfigError(f'config.json: {where}.q_temp: "every" must be a whole number of positions, found {qt["every"]!r}')


def _check_latent(m: dict, where: str) -> None:
    for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
        _pos_int(m, k, where)
    _number(m, "scale", where)
    if m.get("mask") is not None:
        _pos_int(m["mask"], "size", where + ".mask")
    rot = m.get("rot")
    if rot is not None:
        dims = _pos_int(rot, "dims", where + ".rot")
        if dims % 2 or dims > m["rot_dim"]:
            raise ConfigError(f'config.json: {where}.rot: "dims" ({dims}) must be even and at most "rot_dim" ({m["rot_dim"]})')
        if _number(rot, "base", where + ".rot") <= 0:
            raise ConfigError(f'config.json: {where}.rot: "base" must be positive')


def _check_delta(m: dict, where: str) -> None:
    heads, kv = _pos_int(m, "heads", where), _pos_int(m, "kv_heads", where)
    if heads % kv:
        raise ConfigError(f'config.json: {where}: "heads" ({heads}) must be a multiple of "kv_heads" ({kv})')
    for k in ("dim", "vdim", "conv"):
        _pos_int(m, k, where)


def _check_mlp(mlp: dict, where: str) -> None:
    kind = _need(mlp, "kind", where)
    if kind == "dense":
        _pos_int(mlp, "ff", where)
    elif kind == "moe":
        _pos_int(_need(mlp, "expert", where), "ff", where + ".expert")
        r = _need(mlp, "router", where)
        n, top = _pos_int(r, "experts", where + ".router"), _pos_int(r, "top", where + ".router")
        if top > n:
            raise ConfigError(f'config.json: {where}.router: "top" ({top}) exceeds "experts" ({n})')
    else:
        raise ConfigError(f'config.json: {where}: unknown kind {kind!r} (known: dense, moe)')


@dataclass(frozen=True)
class FiponexConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[Dict[str, Any], ...]
    eos_token_ids: Tuple[int, ...] = ()
    initializer_range: float = 0.06

    architecture = "Fiponex"

    @classmethod
    def from_dict(cls, d: dict) -> "FiponexConfig":
        vocab, width = _pos_int(d, "vocab", "top level"), _pos_int(d, "width", "top level")
        layers_in = _need(d, "layers", "top level")
        if not isinstance(layers_in, list) or not layers_in:
            raise ConfigError('config.json: "layers" must be a non-empty list')
        layers = []
        for i, l in enumerate(layers_in):
            where = f"layers[{i}]"
            kind, mixer = _need(l, "type", where), _need(l, "mixer", where)
            if kind == "attention":
                _check_attention(mixer, where + ".mixer")
            elif kind == "latent_attention":
                _check_latent(mixer, where + ".mixer")
            elif kind == "delta":
                _check_delta(mixer, where + ".mixer")
            else:
                raise ConfigError(f'config.json: {where}: unknown mixer type {kind!r} (known: {", ".join(MIXERS)})')
            mlp = l.get("mlp")
            if mlp is not None:
                _check_mlp(mlp, where + ".mlp")
            layers.append(copy.deepcopy({"type": kind, "mixer": mixer, "mlp": mlp}))
        emb = d.get("embedding") or {}
        eos = d.get("eos_token_id")
        eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab=vocab, width=width,
                   embedding_scale=_number(emb, "scale", "embedding") if emb.get("scale") is not None else 1.0,
                   norm_eps=_number(_need(d, "norm", "top level"), "eps", "norm"), layers=tuple(layers),
                   eos_token_ids=eos_ids, initializer_range=float(d.get("initializer_range", 0.06)))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
             "layers": copy.deepcopy(list(self.layers)), "initializer_range": self.initializer_range}
        if self.eos_token_ids:
            d["eos_token_id"] = list(self.eos_token_ids)
        return d

    def _mixer(self, l: dict) -> PartSpec:
        m, w, eps = l["mixer"], self.width, self.norm_eps
        if l["type"] == "attention":
            qt = m.get("q_temp") or {}
            return PartSpec("sink_attention", {
                "hidden_size": w, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "key_dim": m["dim"],
                "value_dim": m["vdim"], "scale": float(m["scale"]), "eps": eps,
                "stretch_coef": float(qt.get("coef", 0.0)), "stretch_every": int(qt.get("every", 0))})
        if l["type"] == "latent_attention":
            rot, mask = m.get("rot") or {}, m.get("mask") or {}
            return PartSpec("latent_attention", {
                "hidden_size": w, "num_heads": m["heads"], "plain_dim": m["dim"], "rot_part": m["rot_dim"],
                "value_dim": m["vdim"], "rank": m["kv_rank"], "scale": float(m["scale"]), "eps": eps,
                "rot_dims": rot.get("dims", 0), "rot_base": float(rot.get("base", 10000.0)), "window": mask.get("size")})
        return PartSpec("gated_delta_rule", {
            "hidden_size": w, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "key_dim": m["dim"],
            "value_dim": m["vdim"], "taps": m["conv"], "eps": eps})

    def _ffn(self, mlp: dict) -> PartSpec:
        if mlp["kind"] == "dense":
            return PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": mlp["ff"],
                                       "names": ("gate", "up", "down"), "act": "relu"})
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "num_experts": mlp["router"]["experts"], "top": mlp["router"]["top"],
            "expert_size": mlp["expert"]["ff"], "router": "softmax", "correction": False, "glu": "silu"})

    def model_spec(self) -> ModelSpec:
        norm = PartSpec("rms_norm", {"size": self.width, "eps": self.norm_eps, "weight_suffix": "", "one_plus": True})
        layers: List[LayerSpec] = []
        for i, l in enumerate(self.layers):
            ffn = None if l["mlp"] is None else self._ffn(l["mlp"])
            more = (("norm1_out", "norm", norm, "norm1b"),) + ((("norm2_out", "norm", norm, "norm2b"),) if ffn else ())
            layers.append(LayerSpec(prefix=f"l{i}.", norm1=norm, mixer=self._mixer(l), norm2=norm if ffn else None,
                                    ffn=ffn, mixer_prefix="mix.", ffn_prefix="mlp.", norm1_name="norm1",
                                    norm2_name="norm2", block="sandwich_norm", more=more))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=self.width,
            max_positions=DEFAULT_MAX_POSITIONS, layers=layers, order=[LayerCall(i) for i in range(len(layers))],
            final_norm=norm, embed_name="embed", final_norm_name="final.norm", lm_head_name="head",
            tie_word_embeddings=False, eos_token_ids=self.eos_token_ids, initializer_range=self.initializer_range,
            embedding_scale=self.embedding_scale)


register_architecture(FiponexConfig.architecture, FiponexConfig)
