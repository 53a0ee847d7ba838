"""Fozerax: typed configuration and its translation into a ModelSpec.

A decoder whose layers read the residual stream x itself and normalise what a sublayer RETURNS:

    x <- x + rmsnorm_1(mixer(x));    x <- x + rmsnorm_2(feed_forward(x))          (second line absent without one)

The token table's rows pass an rmsnorm before they enter the stream; a final rmsnorm precedes the output matrix.
Two kinds of layer, in any order:

"gla"       linear attention with a decay per key channel (parts/decayed_attention.py)
"parallel"  two mixers on the same rows, each result normalised over the width, half their sum
            (parts/side_by_side.py): sliding-window attention with biased projections, one norm over all of q and
            one over all of k, a configured score scale, a learned bias per distance bucket and a sink
            (parts/attention.py); and the gated delta rule behind short causal filters (parts/delta_rule.py)

Feed-forwards: dense gated with tanh-GELU (parts/dense_ff.py), a mixture of clipped gated experts with grouped
routing and a shared expert (parts/routed_ff.py), or none.

config.json keys (all sizes and constants come from there or from the tensors' shapes; tensor names are fixed):

    architecture "Fozerax"; vocab; width; norm.eps; layers[i] = {type, mixer, mlp}
      type "gla":      mixer {heads, dim, vdim, tau}                      (the decay's rank is the stored tensors')
      type "parallel": mixer {left: {heads, kv_heads, dim, vdim, scale, bias_max, mask: {size} | null},
                              right: {heads, kv_heads, dim, vdim, conv}}   (the bias table's rows are the stored tensor's)
      mlp {kind: "dense", ff} | {kind: "moe", router: {experts, top, groups: {count, keep} | null}, expert: {ff, limit},
           shared: {ff, limit} | null} | null

A configuration written for a random model also carries ``rank`` (gla) and ``buckets`` (left), which a checkpoint's
tensors otherwise state.

Tensors: embed, embed.norm, final.norm, head, and per layer l<i>.: norm1, norm2, mix.* and mlp.* as the parts name them.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Mapping, Optional, Tuple, Union

from ..config.registry import Architecture, ConfigError, register_architecture
from ..config.specs import LayerCall, LayerSpec, ModelSpec, PartSpec

NAME = "Fozerax"
DEFAULT_MAX_POSITIONS = 1 << 20       # the design states no limit; an engine's own sequence limit sizes its tables
# constants that the design fixes
UNIT_EPS = 1e-6                       # inside the root when q and k of the delta rule are made unit vectors
EXPERT_SLOPE = 1.702                  # an expert's g * sigmoid(slope * g)
WEIGHT_SUM_EPS = 1e-20                # added to the sum of the chosen experts' scores
SIDE_WEIGHT = 0.5                     # a parallel layer's result is half the sum of its two sides


@dataclass(frozen=True)
class DecayedMixer:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: Optional[int]                # None: the stored tensors state it


@dataclass(frozen=True)
class WindowSide:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: float
    window: Optional[int]
    buckets: Optional[int]             # None: the stored table states it


@dataclass(frozen=True)
class DeltaSide:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int


@dataclass(frozen=True)
class ParallelMixer:
    left: WindowSide
    right: DeltaSide


@dataclass(frozen=True)
class DenseFF:
    ff: int


@dataclass(frozen=True)
class RoutedFF:
    experts: int
    top: int
    groups: int
    keep: int
    ff: int
    limit: float
    shared_ff: int                     # 0: no shared expert
    shared_limit: float


@dataclass(frozen=True)
class FozeraxLayer:
    mixer: Union[DecayedMixer, ParallelMixer]
    mlp: Union[DenseFF, RoutedFF, None]


@dataclass(frozen=True)
class FozeraxConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[FozeraxLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS


def _get(raw, key: str, where: str):
    if not isinstance(raw, Mapping) or key not in raw:
        raise ConfigError(f"config.json: {where} is missing key {key!r}")
    return raw[key]


def _int(raw, key, where, minimum=1) -> int:
    v = _get(raw, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {minimum}, got {v!r}")
    return v


def _opt_int(raw, key, where, minimum=1) -> Optional[int]:
    return _int(raw, key, where, minimum) if isinstance(raw, Mapping) and raw.get(key) is not None else None


def _num(raw, key, where, positive=False) -> float:
    v = _get(raw, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or (positive and v <= 0):
        raise ConfigError(f"config.json: {where}.{key} must be a{' positive' if positive else ''} number, got {v!r}")
    return float(v)


def _heads(raw, where) -> Tuple[int, int]:
    heads = _int(raw, "heads", where)
    kv = _opt_int(raw, "kv_heads", where) or heads
    if heads % kv:
        raise ConfigError(f"config.json: {where}.heads ({heads}) must be a multiple of kv_heads ({kv})")
    return heads, kv


def _mixer(kind: str, raw, where: str):
    if kind == "gla":
        dim = _int(raw, "dim", where)
        return DecayedMixer(_int(raw, "heads", where), dim, _opt_int(raw, "vdim", where) or dim, _num(raw, "tau", where, positive=True),
                            _opt_int(raw, "rank", where))
    lraw, rraw = _get(raw, "left", where), _get(raw, "right", where)
    lw, rw = where + ".left", where + ".right"
    heads, kv = _heads(lraw, lw)
    dim = _int(lraw, "dim", lw)
    mask = lraw.get("mask")
    left = WindowSide(heads, kv, dim, _opt_int(lraw, "vdim", lw) or dim, _num(lraw, "scale", lw), _num(lraw, "bias_max", lw, positive=True),
                      _int(mask, "size", lw + ".mask") if mask is not None else None, _opt_int(lraw, "buckets", lw, 2))
    rheads, rkv = _heads(rraw, rw)
    rdim = _int(rraw, "dim", rw)
    right = DeltaSide(rheads, rkv, rdim, _opt_int(rraw, "vdim", rw) or rdim, _opt_int(rraw, "conv", rw, 0) or 0)
    return ParallelMixer(left, right)


def _mlp(raw, where: str):
    if raw is None:
        return None
    kind = _get(raw, "kind", where)
    if kind == "dense":
        return DenseFF(_int(raw, "ff", where))
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not a feed-forward of this design ('dense', 'moe')")
    router, expert = _get(raw, "router", where), _get(raw, "expert", where)
    experts, top = _int(router, "experts", where + ".router"), _int(router, "top", where + ".router")
    groups = router.get("groups")
    count = _int(groups, "count", where + ".router.groups") if groups is not None else 1
    keep = _int(groups, "keep", where + ".router.groups") if groups is not None else 1
    if experts % count or keep > count or top > keep * (experts // count):
        raise ConfigError(f"config.json: {where}.router: {experts} experts in {count} groups of which {keep} are kept "
                          f"cannot give {top} experts a token")
    shared = raw.get("shared")
    return RoutedFF(experts, top, count, keep, _int(expert, "ff", where + ".expert"), _num(expert, "limit", where + ".expert", positive=True),
                    _int(shared, "ff", where + ".shared") if shared is not None else 0,
                    _num(shared, "limit", where + ".shared", positive=True) if shared is not None else 0.0)


def parse(raw: Mapping[str, Any]) -> FozeraxConfig:
    layers = _get(raw, "layers", "the configuration")
    if not isinstance(layers, (list, tuple)) or not layers:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    out = []
    for i, l in enumerate(layers):
        where = f"layers[{i}]"
        kind = _get(l, "type", where)
        if kind not in ("gla", "parallel"):
            raise ConfigError(f"config.json: {where}.type {kind!r} is not a layer of this design ('gla', 'parallel')")
        out.append(FozeraxLayer(_mixer(kind, _get(l, "mixer", where), where + ".mixer"), _mlp(l.get("mlp"), where + ".mlp")))
    max_positions = raw.get("max_positions", DEFAULT_MAX_POSITIONS)
    if isinstance(max_positions, bool) or not isinstance(max_positions, int) or max_positions <= 0:
        raise ConfigError(f"config.json: max_positions must be a positive integer, got {max_positions!r}")
    return FozeraxConfig(vocab=_int(raw, "vocab", "the configuration"), width=_int(raw, "width", "the configuration"),
                         eps=_num(_get(raw, "norm", "the configuration"), "eps", "norm", positive=True),
                         layers=tuple(out), max_positions=max_positions)


def to_dict(cfg: FozeraxConfig) -> Dict[str, Any]:
    layers = []
    for l in cfg.layers:
        m = l.mixer
        if isinstance(m, DecayedMixer):
            mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "tau": m.tau}
            if m.rank is not None:
                mixer["rank"] = m.rank
            kind = "gla"
        else:
            a, b = m.left, m.right
            left = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale, "bias_max": a.bias_max,
                    "mask": {"size": a.window} if a.window is not None else None}
            if a.buckets is not None:
                left["buckets"] = a.buckets
            mixer = {"left": left, "right": {"heads": b.heads, "kv_heads": b.kv_heads, "dim": b.dim, "vdim": b.vdim, "conv": b.taps}}
            kind = "parallel"
        f = l.mlp
        if f is None:
            mlp = None
        elif isinstance(f, DenseFF):
            mlp = {"kind": "dense", "ff": f.ff}
        else:
            mlp = {"kind": "moe", "router": {"experts": f.experts, "top": f.top, "groups": {"count": f.groups, "keep": f.keep}},
                   "expert": {"ff": f.ff, "limit": f.limit},
                   "shared": {"ff": f.shared_ff, "limit": f.shared_limit} if f.shared_ff else None}
        layers.append({"type": kind, "mixer": mixer, "mlp": mlp})
    d = {"architecture": NAME, "vocab": cfg.vocab, "width": cfg.width, "norm": {"eps": cfg.eps}, "layers": layers}
    if cfg.max_positions != DEFAULT_MAX_POSITIONS:
        d["max_positions"] = cfg.max_positions
    return d


def _mixer_spec(m, W: int, eps: float) -> PartSpec:
    if isinstance(m, DecayedMixer):
        return PartSpec("decayed_linear_attention", {
            "hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim, "tau": m.tau, "norm_eps": eps,
            "decay_rank": m.rank,
            "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o", "norm": "norm", "decay_low": "a1", "decay_up": "a2",
                      "decay_bias": "a2.b"}})
    a, b = m.left, m.right
    left = PartSpec("attention", {
        "hidden_size": W, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim,
        "qkv_bias": True, "window": a.window, "softmax_scale": a.scale, "position": None, "qk_row_norm_eps": eps,
        "distance_bias": {"buckets": a.buckets, "max_distance": a.bias_max}, "sink": True,
        "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "q_norm": "q.norm",
                  "k_norm": "k.norm", "rel": "rel", "sink": "sink"}}, "left.")
    right = PartSpec("gated_delta_rule", {
        "hidden_size": W, "num_heads": b.heads, "num_qk_heads": b.kv_heads, "head_dim": b.dim, "v_head_dim": b.vdim,
        "filter_taps": b.taps, "norm_eps": eps, "unit_eps": UNIT_EPS,
        "names": {"q": "q", "k": "k", "v": "v", "q_filter": "q.conv", "k_filter": "k.conv", "v_filter": "v.conv", "beta": "b",
                  "step": "a", "a_log": "A_log", "dt_bias": "dt_bias", "gate": "g", "norm": "norm", "o": "o"}}, "right.")
    return PartSpec("side_by_side", {"first": left, "second": right, "first_scale": SIDE_WEIGHT, "second_scale": SIDE_WEIGHT,
                                     "hidden_size": W, "first_norm": "left.out", "second_norm": "right.out", "norm_eps": eps})


def _mlp_spec(f, W: int) -> PartSpec:
    if isinstance(f, DenseFF):
        return PartSpec("dense", {"hidden_size": W, "intermediate_size": f.ff, "activation": "gelu_tanh", "gated": True,
                                  "names": {"gate": "gate", "up": "up", "down": "down"}})
    return PartSpec("routed_experts", {"hidden_size": W, "experts": f.experts, "top": f.top, "groups": f.groups, "keep": f.keep,
                                       "expert_size": f.ff, "limit": f.limit, "shared_size": f.shared_ff,
                                       "shared_limit": f.shared_limit, "slope": EXPERT_SLOPE, "sum_eps": WEIGHT_SUM_EPS})


def _with_prefix(spec: PartSpec, prefix: str) -> PartSpec:
    return PartSpec(spec.kind, spec.params, prefix)


def to_spec(cfg: FozeraxConfig) -> ModelSpec:
    W = cfg.width
    layers, optional = [], []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {
            "mixer": ("mixer", _with_prefix(_mixer_spec(l.mixer, W, cfg.eps), p + "mix.")),
            "mixer_out_norm": ("norm", PartSpec("rmsnorm", {"size": W, "eps": cfg.eps, "weight_name": "norm1"}, p)),
        }
        if l.mlp is not None:
            parts["feed_forward"] = ("feed_forward", _with_prefix(_mlp_spec(l.mlp, W), p + "mlp."))
            parts["feed_forward_out_norm"] = ("norm", PartSpec("rmsnorm", {"size": W, "eps": cfg.eps, "weight_name": "norm2"}, p))
        else:
            optional.append(p + "norm2")                 # a norm with nothing to normalise may be stored all the same
        layers.append(LayerSpec("sublayer_norm", parts))
    spec = ModelSpec(
        architecture=NAME, hidden_size=W, vocab_size=cfg.vocab, max_positions=cfg.max_positions, layers=tuple(layers),
        schedule=tuple(LayerCall(i, i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm", {"size": W, "eps": cfg.eps, "weight_name": "final.norm"}, ""),
        embedding=PartSpec("token_table", {"vocab_size": cfg.vocab, "hidden_size": W, "weight_name": "embed",
                                           "norm_weight_name": "embed.norm", "norm_eps": cfg.eps}, ""),
        head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": W, "tied": False, "weight_name": "head"}, ""),
        eos_token_id=None, optional_tensors=tuple(optional))
    spec.validate()
    return spec


ARCHITECTURE = register_architecture(Architecture(NAME, parse, to_spec, to_dict))
