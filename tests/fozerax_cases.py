"""Tiny Fozerax configurations for the tests, random weights for them, and the comparison with the plain
implementation (plain_fozerax.py). The configurations differ from each other in every size and option and make
unequal what a model may happen to make equal (key and value sizes, heads of the two sides, kv heads and 1, the
order of the layer types, windows and none, filters of several lengths, groups of experts and none)."""
from __future__ import annotations

import functools
import json
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

import helpers as H
import plain_fozerax as pf
from ruvenex_cases import check_bf16


def _gla(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def _par(left, right):
    return {"left": left, "right": right}


def _left(heads, kv, dim, vdim, scale, bias_max, window, buckets):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max,
            "mask": None if window is None else {"size": window}, "buckets": buckets}


def _right(heads, kv, dim, vdim, conv):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}


def _moe(experts, top, groups, ff, limit, shared):
    return {"kind": "moe", "router": {"experts": experts, "top": top, "groups": None if groups is None else {"count": groups[0], "keep": groups[1]}},
            "expert": {"ff": ff, "limit": limit}, "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}


CASES: Dict[str, dict] = {
    # a decayed layer, then a parallel one: a window of 24 over a bias table of 12 rows, three taps, grouped routing
    "a": {"architecture": "Fozerax", "vocab": 200, "width": 64, "norm": {"eps": 1e-5},
          "layers": [{"type": "gla", "mixer": _gla(2, 16, 32, 8.0, 4), "mlp": {"kind": "dense", "ff": 96}},
                     {"type": "parallel", "mixer": _par(_left(4, 2, 16, 24, 0.2, 40, 24, 12), _right(2, 1, 16, 32, 3)),
                      "mlp": _moe(6, 2, (3, 2), 24, 1.5, (40, 2.5))}]},
    # nothing a multiple of eight; the parallel layer first; no window; a table with an odd number of rows; one tap,
    # five taps; a layer without feed-forward; routing without groups or shared expert in which every expert is used
    "b": {"architecture": "Fozerax", "vocab": 97, "width": 36, "norm": {"eps": 3e-6},
          "layers": [{"type": "parallel", "mixer": _par(_left(3, 3, 10, 7, 0.3, 20, None, 7), _right(3, 3, 5, 9, 1)), "mlp": None},
                     {"type": "gla", "mixer": _gla(1, 40, 20, 3.5, 3), "mlp": _moe(4, 4, None, 10, 0.7, None)},
                     {"type": "parallel", "mixer": _par(_left(2, 1, 12, 12, 0.25, 9, 5, 4), _right(4, 2, 8, 4, 5)),
                      "mlp": {"kind": "dense", "ff": 20}},
                     {"type": "parallel", "mixer": _par(_left(1, 1, 6, 14, 0.5, 30, 33, 16), _right(1, 1, 12, 6, 0)),
                      "mlp": _moe(9, 3, (3, 1), 5, 3.0, (7, 0.5))}]},
    # large heads: keys of 128 and 160 (sixteen and thirty-two state rows a lane), a window of 80 under a table that
    # saturates later, two decayed layers in a row
    "c": {"architecture": "Fozerax", "vocab": 256, "width": 128, "norm": {"eps": 2e-6},
          "layers": [{"type": "gla", "mixer": _gla(2, 128, 64, 16.0, 16), "mlp": _moe(8, 2, (4, 2), 32, 2.0, (64, 1.0))},
                     {"type": "gla", "mixer": _gla(3, 24, 40, 4.0, 8), "mlp": None},
                     {"type": "parallel", "mixer": _par(_left(8, 2, 64, 64, 0.11, 200, 80, 28), _right(4, 2, 160, 128, 4)),
                      "mlp": {"kind": "dense", "ff": 256}}]},
}


def spec_of(cfg: dict):
    return H.spec_of(cfg)


def make_weights(cfg: dict, seed: int, dtype=torch.bfloat16, sharp: float = 0.0) -> Dict[str, torch.Tensor]:
    """Random weights; with ``sharp`` the weights of the query norm are multiplied by it, so that attention weights
    are peaked: a position's result then hangs on single keys at the far end of its window, and a wrong key, a lost
    sink or a window one token off shows."""
    from infer_b200.weights import random_weights
    W = random_weights(spec_of(cfg), seed, dtype)
    if sharp:
        for k in W:
            if k.endswith(".mix.left.q.norm"):
                W[k] = (W[k].float() * sharp).to(dtype)
    return W


def random_ids(cfg: dict, n: int, seed: int) -> List[int]:
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


@functools.lru_cache(maxsize=64)
def _oracle(cfg_json: str, seed: int, sharp: float, compute: str, ids: Tuple[int, ...], rounding: str):
    cfg = json.loads(cfg_json)
    W = H.as_compute(make_weights(cfg, seed, torch.bfloat16, sharp), getattr(torch, compute))
    if rounding == "none":
        return pf.forward(cfg, W, list(ids)).numpy()
    with pf.rounded(getattr(torch, rounding)):
        return pf.forward(cfg, W, list(ids)).numpy()


def oracle(cfg: dict, seed: int, compute: torch.dtype, ids: Sequence[int], rounding=None, sharp: float = 0.0) -> np.ndarray:
    n = lambda d: str(d).replace("torch.", "")
    return _oracle(json.dumps(cfg, sort_keys=True), seed, float(sharp), n(compute), tuple(int(i) for i in ids),
                   "none" if rounding is None else n(rounding))


CLOSE_CALL = 0.02      # a router's gap, in units of its logits' terms, below which bfloat16 roundings may turn the choice


@functools.lru_cache(maxsize=64)
def _router_gaps(cfg_json: str, seed: int, sharp: float, ids: Tuple[int, ...]) -> np.ndarray:
    cfg = json.loads(cfg_json)
    W = H.as_compute(make_weights(cfg, seed, torch.bfloat16, sharp), torch.bfloat16)
    gaps: List[torch.Tensor] = []
    pf.forward(cfg, W, list(ids), None, gaps)
    return torch.stack(gaps).min(dim=0).values.numpy() if gaps else np.full(len(ids), np.inf)


def check(cfg: dict, seed: int, dtype: torch.dtype, got: Dict[str, Dict[int, np.ndarray]], reqs: Dict[str, List[int]],
          sharp: float = 0.0, what: str = ""):
    """The engine's rows against the plain implementation. In bfloat16, positions at which a router's choice is a
    close call are left out (the other expert is as right an answer there). The float32 comparison leaves out nothing
    and is the sharp one; cuttings are compared bit by bit there."""
    for rid, ids in reqs.items():
        ref = oracle(cfg, seed, dtype, ids, None, sharp)
        rows = sorted(got[rid])
        if dtype != torch.float32:
            gaps = _router_gaps(json.dumps(cfg, sort_keys=True), seed, float(sharp), tuple(int(i) for i in ids))
            clear = [p for p in rows if gaps[p] >= CLOSE_CALL]
            assert len(clear) >= 0.6 * len(rows) - 1, f"{what}/{rid}: {len(rows) - len(clear)} of {len(rows)} positions are close calls"
            rows = clear
            if not rows:
                continue
        g = np.stack([got[rid][p] for p in rows])
        if dtype == torch.float32:
            H.check_f32(g, ref[rows], f"{what}/{rid}")
        else:
            check_bf16(g, ref[rows], oracle(cfg, seed, dtype, ids, torch.bfloat16, sharp)[rows], f"{what}/{rid}", factor=4.0)
