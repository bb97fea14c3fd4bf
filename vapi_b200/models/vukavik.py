"""Vukavik (``"architecture": "Vukavik"``) as a plan of parts.

A decoder-only model whose ``layers`` list names each layer's mixer: grouped-query attention
with per-head q/k norms, interleaved rotary pairs with YaRN-scaled frequencies, a chunked
causal mask, a sink per head and a gate per head (``attention``); the gated delta rule
(``delta``); or Mamba-2 (``mamba2``).  A layer norms each sublayer on both sides and scales what
it adds by ``residual_mult``; its feed-forward is a dense SwiGLU or absent.  The logits are
scaled by ``logit_scale``.  Everything here is data handed to parameterised parts.

config.json keys: ``vocab``, ``width``, ``residual_mult``, ``logit_scale``, ``norm.eps`` and
``layers[i] = {type, mixer: {...}, mlp: {kind, ff} | null}`` with, per mixer type,
attention: ``heads kv_heads dim vdim scale rot{base dims scaling{factor original fast slow}} mask{size}``;
delta: ``heads kv_heads dim vdim conv``; mamba2: ``heads vdim state groups conv norm_groups``.
Tensors: ``embed``, ``l<i>.norm1 norm1b norm2 norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.{gate,up,down}``,
``final.norm``, ``head``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from ..config.model import Architecture, ConfigError, register_architecture, require_int
from ..parts import (GQAttention, GatedDeltaMixer, Mamba2Mixer, OutputHead, RMSNorm, SandwichBlock,
                     ScaledRotaryEncoding, SwiGLU, TokenEmbedding)
from .plan import LayerCall, ModelPlan

#: positions are counted in float32, which holds integers exactly up to here
MAX_POSITIONS = 1 << 24


def _num(v: Dict[str, Any], key: str, where: str) -> float:
    x = v.get(key)
    if isinstance(x, bool) or not isinstance(x, (int, float)):
        raise ConfigError(f"config.json: {where} needs the number `{key}`")
    return float(x)


def _int(v: Dict[str, Any], key: str, where: str) -> int:
    x = v.get(key)
    if isinstance(x, bool) or not isinstance(x, int) or x <= 0:
        raise ConfigError(f"config.json: {where} needs the positive integer `{key}`")
    return int(x)


@dataclass(frozen=True)
class VukavikLayer:
    kind: str                               # attention | delta | mamba2
    mixer: Tuple[Tuple[str, Any], ...]      # the mixer's sizes and constants, as sorted items
    ff: Optional[int]                       # feed-forward width, None: no feed-forward

    def m(self) -> Dict[str, Any]:
        return dict(self.mixer)


@dataclass(frozen=True)
class VukavikConfig:
    vocab: int
    width: int
    residual_mult: float
    logit_scale: float
    norm_eps: float
    layers: Tuple[VukavikLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()
    raw: Any = None

    KINDS = ("attention", "delta", "mamba2")

    @classmethod
    def from_json(cls, v: Dict[str, Any]) -> "VukavikConfig":
        norm = v.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: missing `norm`")
        raw_layers = v.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: `layers` must be a non-empty list")
        layers = []
        for i, e in enumerate(raw_layers):
            where = f"layer {i}"
            if not isinstance(e, dict) or e.get("type") not in cls.KINDS:
                raise ConfigError(f"config.json: {where}: type must be one of {list(cls.KINDS)}")
            mx = e.get("mixer")
            if not isinstance(mx, dict):
                raise ConfigError(f"config.json: {where} has no `mixer`")
            kind = e["type"]
            m: Dict[str, Any] = {}
            if kind == "attention":
                for k in ("heads", "kv_heads", "dim", "vdim"):
                    m[k] = _int(mx, k, where)
                m["scale"] = _num(mx, "scale", where)
                rot = mx.get("rot")
                if isinstance(rot, dict):
                    m["rot_dims"], m["rot_base"] = _int(rot, "dims", where + " rot"), _num(rot, "base", where + " rot")
                    sc = rot.get("scaling")
                    if isinstance(sc, dict):
                        m["rot_scaling"] = tuple(sorted((k, _num(sc, k, where + " rot.scaling"))
                                                        for k in ("factor", "original", "fast", "slow")))
                mask = mx.get("mask")
                m["chunk"] = _int(mask, "size", where + " mask") if isinstance(mask, dict) else 0
            elif kind == "delta":
                for k in ("heads", "kv_heads", "dim", "vdim", "conv"):
                    m[k] = _int(mx, k, where)
            else:
                for k in ("heads", "vdim", "state", "groups", "conv", "norm_groups"):
                    m[k] = _int(mx, k, where)
            mlp = e.get("mlp")
            ff = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}: the feed-forward kind must be `dense`")
                ff = _int(mlp, "ff", where + " mlp")
            layers.append(VukavikLayer(kind, tuple(sorted(m.items())), ff))
        eos = v.get("eos_token_id")
        eos_ids = (int(eos),) if isinstance(eos, int) and not isinstance(eos, bool) else \
            tuple(int(x) for x in eos if isinstance(x, int)) if isinstance(eos, list) else ()
        return cls(vocab=require_int(v, "vocab"), width=require_int(v, "width"),
                   residual_mult=_num(v, "residual_mult", "the model"), logit_scale=_num(v, "logit_scale", "the model"),
                   norm_eps=_num(norm, "eps", "norm"), layers=tuple(layers), eos_token_ids=tuple(sorted(set(eos_ids))),
                   raw=None)


def vukavik_plan(cfg: VukavikConfig) -> ModelPlan:
    W, eps = cfg.width, cfg.norm_eps
    emb = TokenEmbedding(cfg.vocab, W, "embed")
    encodings: Dict[Any, ScaledRotaryEncoding] = {}
    layers, prefixes = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.m()
        if layer.kind == "attention":
            pos = None
            if "rot_dims" in m:
                enc = ScaledRotaryEncoding(m["rot_dims"], m["rot_base"], dict(m["rot_scaling"]) if "rot_scaling" in m else None)
                enc = encodings.setdefault(enc.key(), enc)
                if enc.name == "rope":
                    enc.name = f"rope{len(encodings) - 1}"
                pos = enc.name
            mixer = GQAttention(W, m["heads"], m["kv_heads"], m["dim"], qk_norm_eps=eps, pos=pos,
                                rot_dim=m.get("rot_dims"), scale=m["scale"], v_head_dim=m["vdim"], chunk=m["chunk"],
                                sink=True, head_gate=True, rope_layout="interleaved", weight_suffix="",
                                names={"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm",
                                       "sink": "sink", "gate": "g"})
        elif layer.kind == "delta":
            mixer = GatedDeltaMixer(W, m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"], eps, weight_suffix="",
                                    names={"q": "q", "k": "k", "v": "v", "a": "a", "b": "b", "g": "g", "o": "o",
                                           "conv": ".conv", "A_log": "A_log", "dt_bias": "dt_bias", "norm": "norm"})
        else:
            mixer = Mamba2Mixer(W, m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"], eps,
                                weight_suffix="",
                                names={"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias",
                                       "A_log": "A_log", "D": "D", "norm": "norm", "o": "o"})
        ffn = ffn_norm = ffn_post = None
        if layer.ff is not None:
            ffn = SwiGLU(W, layer.ff, {"gate": "gate", "up": "up", "down": "down"}, weight_suffix="")
            ffn_norm, ffn_post = RMSNorm(W, eps, "norm2"), RMSNorm(W, eps, "norm2b")
        layers.append(SandwichBlock(RMSNorm(W, eps, "norm1"), mixer, RMSNorm(W, eps, "norm1b"), ffn_norm, ffn, ffn_post,
                                    {"mixer": "mix.", "ffn": "mlp."}, mult=cfg.residual_mult))
        prefixes.append(f"l{i}.")
    return ModelPlan(
        architecture="Vukavik", vocab_size=cfg.vocab, hidden_size=W, max_positions=MAX_POSITIONS, embedding=emb,
        layers=layers, layer_prefixes=prefixes, order=[LayerCall(i) for i in range(len(layers))],
        final_norm=RMSNorm(W, eps, "norm"), final_norm_prefix="final.",
        head=OutputHead(cfg.vocab, W, False, emb, "head", scale=cfg.logit_scale),
        position_encodings=list(encodings.values()), eos_token_ids=cfg.eos_token_ids, config=cfg)


register_architecture(Architecture(name="Vukavik", model_types=("vukavik",), parse=VukavikConfig.from_json, plan=vukavik_plan))
