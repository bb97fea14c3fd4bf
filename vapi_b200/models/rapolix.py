"""Rapolix (``"architecture": "Rapolix"``) as a plan of parts.

A decoder-only model.  The embedding adds a sinusoidal position vector.  The residual stream runs as
``streams`` copies joined by hyper-connections (without that key: one ordinary stream).  Every layer is
pre-normed by layer norms with a weight and no bias; its mixer (``type`` ``parallel``) is two mixers side by
side on the same input, each RMS-normed and the two averaged: grouped-query attention without rotation over a
sliding window that keeps the first tokens, with an output gate (``left``), and a recurrent block around the
real-gated linear recurrent unit (``right``).  Its feed-forward is a dense SwiGLU with biases, a mixture of
squared-ReLU experts (grouped routing with a correction, identity experts, a shared expert), or absent.  The
logits pass ``cap * tanh(logits / cap)``.  Everything here is data handed to parameterised parts.

config.json keys: ``vocab``, ``width``, ``norm.eps``, ``streams``, ``logit_softcap`` and
``layers[i] = {type, mixer: {left: {heads kv_heads dim vdim scale mask{size keep_first}}, right: {width blocks
conv}}, mlp: null | {kind: dense, ff} | {kind: moe, expert{ff}, router{experts identity top groups{count keep}},
shared{ff}}}``.
Tensors: ``embed``, ``l<i>.norm1 norm2``, ``l<i>.hc1.{in,out,mix}`` ``hc2.*``, ``l<i>.mix.left.{q,k,v,g,o,out}``,
``l<i>.mix.right.{y,y.b,x,x.b,conv,conv.b,ra,ra.b,ri,ri.b,lam,o,out}``, ``l<i>.mlp.{gate,up,down}(.b)`` or
``l<i>.mlp.{e<j>.up, e<j>.down, router, correction, shared.up, shared.down}``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from ..config.model import Architecture, ConfigError, register_architecture, require_int
from ..parts import (GQAttention, HyperBlock, LayerNorm, OutputHead, ParallelMixer, RGLRUMixer, SparseMoE, SwiGLU,
                     TokenEmbedding)
from .plan import LayerCall, ModelPlan

#: positions are counted in float32, which holds integers exactly up to here
MAX_POSITIONS = 1 << 24
#: the position vector's wavelengths grow geometrically from 2 pi to 2 pi times this
SINUSOID_BASE = 10000.0
#: log a = -DECAY_C * r * softplus(lam)
DECAY_C = 8.0


def _num(v: Any, key: str, where: str) -> float:
    x = v.get(key) if isinstance(v, dict) else None
    if isinstance(x, bool) or not isinstance(x, (int, float)):
        raise ConfigError(f"config.json: {where} needs the number `{key}`")
    return float(x)


def _int(v: Any, key: str, where: str, least: int = 1) -> int:
    x = v.get(key) if isinstance(v, dict) else None
    if isinstance(x, bool) or not isinstance(x, int) or x < least:
        raise ConfigError(f"config.json: {where} needs the integer `{key}` >= {least}")
    return int(x)


def _opt_int(v: Any, key: str, where: str, default: int, least: int = 0) -> int:
    if not isinstance(v, dict) or v.get(key) is None:
        return default
    return _int(v, key, where, least)


@dataclass(frozen=True)
class RapolixLayer:
    left: Tuple[Tuple[str, Any], ...]        # the attention's sizes and constants, as sorted items
    right: Tuple[Tuple[str, Any], ...]       # the recurrent block's
    mlp: Optional[Tuple[Tuple[str, Any], ...]]   # None: no feed-forward


@dataclass(frozen=True)
class RapolixConfig:
    vocab: int
    width: int
    norm_eps: float
    streams: Optional[int]                   # None: one ordinary residual stream
    logit_softcap: Optional[float]
    layers: Tuple[RapolixLayer, ...]
    eos_token_ids: Tuple[int, ...] = ()

    @classmethod
    def from_json(cls, v: Dict[str, Any]) -> "RapolixConfig":
        norm = v.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: missing `norm`")
        raw = v.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: `layers` must be a non-empty list")
        width = require_int(v, "width")
        layers = []
        for i, e in enumerate(raw):
            where = f"layer {i}"
            if not isinstance(e, dict) or e.get("type") != "parallel":
                raise ConfigError(f"config.json: {where}: type must be `parallel`")
            mx = e.get("mixer")
            if not isinstance(mx, dict) or not isinstance(mx.get("left"), dict) or not isinstance(mx.get("right"), dict):
                raise ConfigError(f"config.json: {where} needs `mixer.left` and `mixer.right`")
            le, ri = mx["left"], mx["right"]
            left: Dict[str, Any] = {k: _int(le, k, where + " left") for k in ("heads", "kv_heads", "dim", "vdim")}
            if left["heads"] % left["kv_heads"]:
                raise ConfigError(f"config.json: {where}: {left['heads']} heads over {left['kv_heads']} kv heads")
            left["scale"] = _num(le, "scale", where + " left")
            mask = le.get("mask")
            left["window"] = _opt_int(mask, "size", where + " mask", 0, 1)
            left["keep_first"] = _opt_int(mask, "keep_first", where + " mask", 0, 0)
            right = {k: _int(ri, k, where + " right") for k in ("width", "blocks", "conv")}
            if right["width"] % right["blocks"]:
                raise ConfigError(f"config.json: {where}: {right['width']} channels in {right['blocks']} parts")
            mlp = e.get("mlp")
            m: Optional[Dict[str, Any]] = None
            if mlp is not None:
                if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                    raise ConfigError(f"config.json: {where}: the feed-forward kind must be `dense` or `moe`")
                m = {"kind": mlp["kind"]}
                if mlp["kind"] == "dense":
                    m["ff"] = _int(mlp, "ff", where + " mlp")
                else:
                    r = mlp.get("router")
                    m["ff"] = _int(mlp.get("expert"), "ff", where + " mlp.expert")
                    m["experts"] = _int(r, "experts", where + " mlp.router", 0)
                    m["identity"] = _opt_int(r, "identity", where + " mlp.router", 0, 0)
                    m["top"] = _int(r, "top", where + " mlp.router")
                    g = r.get("groups") if isinstance(r, dict) else None
                    m["groups"] = _opt_int(g, "count", where + " mlp.router.groups", 1, 1)
                    m["keep"] = _opt_int(g, "keep", where + " mlp.router.groups", m["groups"], 1)
                    outputs = m["experts"] + m["identity"]
                    if outputs % m["groups"] or m["keep"] > m["groups"] or (outputs // m["groups"]) * m["keep"] < m["top"]:
                        raise ConfigError(f"config.json: {where}: {outputs} router outputs in {m['groups']} groups, "
                                          f"{m['keep']} kept, top {m['top']}")
                    sh = mlp.get("shared")
                    m["shared_ff"] = _int(sh, "ff", where + " mlp.shared") if sh is not None else None
            layers.append(RapolixLayer(tuple(sorted(left.items())), tuple(sorted(right.items())),
                                       tuple(sorted(m.items())) if m is not None else None))
        streams = None
        if v.get("streams") is not None:
            streams = _int(v, "streams", "the model")
            if streams > 8:
                raise ConfigError("config.json: at most 8 streams")
        cap = v.get("logit_softcap")
        if cap is not None and (isinstance(cap, bool) or not isinstance(cap, (int, float)) or cap <= 0):
            raise ConfigError("config.json: `logit_softcap` must be a positive number")
        eos = v.get("eos_token_id")
        eos_ids = (int(eos),) if isinstance(eos, int) and not isinstance(eos, bool) else \
            tuple(int(x) for x in eos if isinstance(x, int)) if isinstance(eos, list) else ()
        return cls(vocab=require_int(v, "vocab"), width=width, norm_eps=_num(norm, "eps", "norm"), streams=streams,
                   logit_softcap=float(cap) if cap is not None else None, layers=tuple(layers),
                   eos_token_ids=tuple(sorted(set(eos_ids))))


def rapolix_plan(cfg: RapolixConfig) -> ModelPlan:
    W, eps = cfg.width, cfg.norm_eps
    S = cfg.streams if cfg.streams is not None else 1
    emb = TokenEmbedding(cfg.vocab, W, "embed", sinusoid_base=SINUSOID_BASE, streams=S)
    layers, prefixes = [], []
    for i, layer in enumerate(cfg.layers):
        le, ri = dict(layer.left), dict(layer.right)
        attn = GQAttention(W, le["heads"], le["kv_heads"], le["dim"], qk_norm_eps=None, pos=None, scale=le["scale"],
                           v_head_dim=le["vdim"], window=le["window"], keep_first=le["keep_first"], out_gate=True,
                           weight_suffix="", names={"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g"})
        rec = RGLRUMixer(W, ri["width"], ri["blocks"], ri["conv"], decay_c=DECAY_C, weight_suffix="", bias_suffix=".b",
                         names={"y": "y", "x": "x", "conv": "conv", "a": "ra", "i": "ri", "lam": "lam", "o": "o"})
        mixer = ParallelMixer(W, [("left.", attn), ("right.", rec)], eps, norm_name="out", deferred=True)
        ffn = ffn_norm = None
        if layer.mlp is not None:
            m = dict(layer.mlp)
            ffn_norm = LayerNorm(W, eps, "norm2")
            if m["kind"] == "dense":
                ffn = SwiGLU(W, m["ff"], {"gate": "gate", "up": "up", "down": "down"}, weight_suffix="", bias=True,
                             bias_suffix=".b")
            else:
                ffn = SparseMoE(W, m["ff"], m["experts"], m["top"], identity=m["identity"], groups=m["groups"],
                                keep=m["keep"], shared_ff=m["shared_ff"], weight_suffix="",
                                names={"expert": "e{}.", "up": "up", "down": "down", "router": "router",
                                       "correction": "correction", "shared": "shared."})
        layers.append(HyperBlock(S, LayerNorm(W, eps, "norm1"), mixer, ffn_norm, ffn,
                                 {"mixer": "mix.", "ffn": "mlp.", "mixer_hc": "hc1.", "ffn_hc": "hc2."},
                                 learned=cfg.streams is not None))
        prefixes.append(f"l{i}.")
    return ModelPlan(
        architecture="Rapolix", vocab_size=cfg.vocab, hidden_size=W, max_positions=MAX_POSITIONS, embedding=emb,
        layers=layers, layer_prefixes=prefixes, order=[LayerCall(i) for i in range(len(layers))],
        final_norm=LayerNorm(W, eps, "norm"), final_norm_prefix="final.",
        head=OutputHead(cfg.vocab, W, False, emb, "head", softcap=cfg.logit_softcap),
        position_encodings=[], eos_token_ids=cfg.eos_token_ids, config=cfg)


register_architecture(Architecture(name="Rapolix", model_types=("rapolix",), parse=RapolixConfig.from_json, plan=rapolix_plan))
