"""Ruvenex: typed configuration and its translation into a ModelSpec.

A decoder whose layers run their sublayers side by side on ONE normalised input n = rmsnorm(x):

    x <- x + sigmoid(R1 n + r1) * (a * attention(n) + b * recurrence(n)) + sigmoid(R2 n + r2) * feed_forward(n)

attention: grouped-query softmax attention whose q, k, v each pass a short causal filter over time, adjacent-pair
rotation over the first ``rot.dims`` channels of a head, values normalised per head before they are cached, the
configured score scale, a sigmoid gate per head on the context.  recurrence: the gated linear recurrence with a
[dim, vdim] state per head (parts/recurrent.py).  feed_forward: dense with tanh-GELU, or none.  The token table is
scaled by ``embedding.scale``; a final rmsnorm precedes the output matrix.  No biases except on gates.

config.json keys (all sizes and constants come from there; tensor names are fixed by the design):

    architecture "Ruvenex"; vocab; width; embedding.scale; norm.eps; layers[i] = {type: "parallel",
      mixer: {left: {heads, kv_heads, dim, vdim, conv, rot: {base, dims}, scale}, left_scale,
              right: {heads, dim, vdim}, right_scale},
      mlp: {kind: "dense", ff} | null}

Tensors: embed, final.norm, head, and per layer l<i>.: norm1, mix.left.{q,k,v,q.conv,k.conv,v.conv,g,o},
mix.right.{q,f,f.b,lower,v,norm,o}, mlp.{up,down}, rg1, rg1.b, rg2, rg2.b.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple

from ..config.registry import Architecture, ConfigError, register_architecture
from ..config.specs import LayerCall, LayerSpec, ModelSpec, PartSpec

NAME = "Ruvenex"
DEFAULT_MAX_POSITIONS = 1 << 20       # the design states no limit; an engine's own sequence limit sizes the tables


@dataclass(frozen=True)
class AttentionSide:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int                          # 0: no filter
    rot_dims: int                      # 0: no rotation
    rot_base: float
    scale: float


@dataclass(frozen=True)
class RecurrentSide:
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class RuvenexLayer:
    left: AttentionSide
    right: RecurrentSide
    left_scale: float
    right_scale: float
    ff: Optional[int]                  # None: no feed-forward


@dataclass(frozen=True)
class RuvenexConfig:
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: Tuple[RuvenexLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS


def _get(raw: Mapping[str, Any], key: str, where: str):
    if not isinstance(raw, Mapping) or key not in raw:
        raise ConfigError(f"config.json: {where} is missing key {key!r}")
    return raw[key]


def _int(raw, key, where, minimum=1) -> int:
    v = _get(raw, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {minimum}, got {v!r}")
    return v


def _num(raw, key, where, positive=False) -> float:
    v = _get(raw, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and v <= 0):
        raise ConfigError(f"config.json: {where}.{key} must be a{' positive' if positive else ''} number, got {v!r}")
    return float(v)


def _layer(raw: Mapping[str, Any], i: int) -> RuvenexLayer:
    where = f"layers[{i}]"
    kind = _get(raw, "type", where)
    if kind != "parallel":
        raise ConfigError(f"config.json: {where}.type {kind!r} is not a layer of this design ('parallel')")
    mixer = _get(raw, "mixer", where)
    lraw, rraw = _get(mixer, "left", where + ".mixer"), _get(mixer, "right", where + ".mixer")
    lw, rw = where + ".mixer.left", where + ".mixer.right"
    heads, dim = _int(lraw, "heads", lw), _int(lraw, "dim", lw)
    kv = _int(lraw, "kv_heads", lw) if lraw.get("kv_heads") is not None else heads
    if heads % kv:
        raise ConfigError(f"config.json: {lw}.heads ({heads}) must be a multiple of kv_heads ({kv})")
    vdim = _int(lraw, "vdim", lw) if lraw.get("vdim") is not None else dim
    taps = _int(lraw, "conv", lw, 0) if lraw.get("conv") is not None else 0
    rot = lraw.get("rot")
    rot_dims, rot_base = 0, 10000.0
    if rot is not None:
        rot_dims, rot_base = _int(rot, "dims", lw + ".rot", 0), _num(rot, "base", lw + ".rot", positive=True)
        if rot_dims % 2 or rot_dims > dim:
            raise ConfigError(f"config.json: {lw}.rot.dims ({rot_dims}) must be even and at most dim ({dim})")
    left = AttentionSide(heads, kv, dim, vdim, taps, rot_dims, rot_base, _num(lraw, "scale", lw))
    rdim = _int(rraw, "dim", rw)
    right = RecurrentSide(_int(rraw, "heads", rw), rdim, _int(rraw, "vdim", rw) if rraw.get("vdim") is not None else rdim)
    mlp = raw.get("mlp")
    ff = None
    if mlp is not None:
        if _get(mlp, "kind", where + ".mlp") != "dense":
            raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not a feed-forward of this design ('dense')")
        ff = _int(mlp, "ff", where + ".mlp")
    return RuvenexLayer(left, right, _num(mixer, "left_scale", where + ".mixer"), _num(mixer, "right_scale", where + ".mixer"), ff)


def parse(raw: Mapping[str, Any]) -> RuvenexConfig:
    layers = _get(raw, "layers", "the configuration")
    if not isinstance(layers, (list, tuple)) or not layers:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
    if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
        raise ConfigError(f"config.json: max_positions must be a positive integer, got {max_positions!r}")
    return RuvenexConfig(
        vocab=_int(raw, "vocab", "the configuration"), width=_int(raw, "width", "the configuration"),
        embedding_scale=_num(_get(raw, "embedding", "the configuration"), "scale", "embedding"),
        eps=_num(_get(raw, "norm", "the configuration"), "eps", "norm", positive=True),
        layers=tuple(_layer(l, i) for i, l in enumerate(layers)), max_positions=max_positions)


def to_dict(cfg: RuvenexConfig) -> Dict[str, Any]:
    layers = []
    for l in cfg.layers:
        left = {"heads": l.left.heads, "kv_heads": l.left.kv_heads, "dim": l.left.dim, "vdim": l.left.vdim,
                "conv": l.left.taps if l.left.taps else None, "scale": l.left.scale,
                "rot": {"base": l.left.rot_base, "dims": l.left.rot_dims} if l.left.rot_dims else None}
        layers.append({"type": "parallel",
                       "mixer": {"left": left, "left_scale": l.left_scale,
                                 "right": {"heads": l.right.heads, "dim": l.right.dim, "vdim": l.right.vdim},
                                 "right_scale": l.right_scale},
                       "mlp": {"kind": "dense", "ff": l.ff} if l.ff is not None else None})
    d = {"architecture": NAME, "vocab": cfg.vocab, "width": cfg.width, "embedding": {"scale": cfg.embedding_scale},
         "norm": {"eps": cfg.eps}, "layers": layers}
    if cfg.max_positions != DEFAULT_MAX_POSITIONS:
        d["max_positions"] = cfg.max_positions
    return d


def to_spec(cfg: RuvenexConfig) -> ModelSpec:
    W = cfg.width
    layers, optional = [], []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        a = l.left
        position = None
        if a.rot_dims:
            position = PartSpec("rotary_pairs", {"head_dim": a.dim, "rotary_dims": a.rot_dims, "theta": a.rot_base,
                                                 "max_positions": cfg.max_positions})
        left = PartSpec("attention", {
            "hidden_size": W, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
            "qkv_bias": False, "window": None, "softmax_scale": a.scale, "position": position,
            "filter_taps": a.taps, "value_norm_eps": cfg.eps, "head_gate": True,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g",
                      "q_filter": "q.conv", "k_filter": "k.conv", "v_filter": "v.conv"},
        }, "left.")
        right = PartSpec("gated_linear_recurrence", {
            "hidden_size": W, "num_heads": l.right.heads, "head_dim": l.right.dim, "v_head_dim": l.right.vdim,
            "norm_eps": cfg.eps,
            "names": {"q": "q", "f": "f", "f_bias": "f.b", "lower": "lower", "v": "v", "norm": "norm", "o": "o"},
        }, "right.")
        parts = {
            "norm": ("norm", PartSpec("rmsnorm", {"size": W, "eps": cfg.eps, "weight_name": "norm1"}, p)),
            "mixer": ("mixer", PartSpec("side_by_side", {"first": left, "second": right, "first_scale": l.left_scale,
                                                         "second_scale": l.right_scale}, p + "mix.")),
            "gate": ("gate", PartSpec("sigmoid_linear", {"hidden_size": W, "names": ("rg1", "rg2") if l.ff is not None else ("rg1",),
                                                         "bias_suffix": ".b"}, p)),
        }
        if l.ff is not None:
            parts["feed_forward"] = ("feed_forward", PartSpec("dense", {
                "hidden_size": W, "intermediate_size": l.ff, "activation": "gelu_tanh",
                "names": {"up": "up", "down": "down"}}, p + "mlp."))
        else:
            optional += [p + "rg2", p + "rg2.b"]          # a gate with nothing to gate may be stored all the same
        layers.append(LayerSpec("parallel_gated", parts))
    spec = ModelSpec(
        architecture=NAME, hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions, layers=tuple(layers),
        schedule=tuple(LayerCall(i, i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {"size": W, "eps": cfg.eps, "weight_name": "final.norm"}, ""),
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab, "hidden_size": W, "scale": cfg.embedding_scale,
                                           "weight_name": "embed"}, ""),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": False, "weight_name": "head"}, ""),
        eos_token_id=None, optional_tensors=tuple(optional))
    spec.validate()
    return spec


ARCHITECTURE = register_architecture(Architecture(NAME, parse, to_spec, to_dict))
