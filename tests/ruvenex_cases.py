"""Tiny Ruvenex configurations for the tests, random weights for them, and the comparison with the plain
implementation (plain_ruvenex.py). The configurations differ from each other in every size and option, and make
unequal what a model may happen to make equal (key and value sizes, rotated channels and head size, heads of the
two sides, kv heads and 1)."""
from __future__ import annotations

import functools
import json
from typing import Dict, List, Sequence, Tuple

import numpy as np
import torch

import helpers as H
import plain_ruvenex as pr


def _layer(left, right, ls, rs, ff):
    return {"type": "parallel", "mixer": {"left": left, "left_scale": ls, "right": right, "right_scale": rs},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _left(heads, kv, dim, vdim, conv, rot_dims, base, scale):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv,
            "rot": None if rot_dims is None else {"dims": rot_dims, "base": base}, "scale": scale}


CASES: Dict[str, dict] = {
    # head size 64 on both sides of attention (the tensor-core attention kernels take it), rotation over half a head
    "p": {"architecture": "Ruvenex", "vocab": 200, "width": 64, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
          "layers": [_layer(_left(4, 2, 64, 64, 3, 32, 10000.0, 0.11), {"heads": 2, "dim": 16, "vdim": 48}, 1.0, 0.5, 96),
                     _layer(_left(4, 2, 64, 64, 3, 32, 10000.0, 0.11), {"heads": 2, "dim": 16, "vdim": 48}, 0.7, 1.3, 96)]},
    # values longer than keys, four taps, every channel rotated, three kv heads, a layer without feed-forward, a
    # recurrence whose sizes are no multiples of 32, one layer without filter and one without rotation
    "q": {"architecture": "Ruvenex", "vocab": 301, "width": 96, "embedding": {"scale": 0.8}, "norm": {"eps": 3e-6},
          "layers": [_layer(_left(6, 3, 16, 24, 4, 16, 500.0, 0.3), {"heads": 1, "dim": 40, "vdim": 20}, 0.9, 1.0, 176),
                     _layer(_left(3, 1, 48, 48, 2, 8, 1000000.0, 0.2), {"heads": 3, "dim": 8, "vdim": 8}, 1.2, 0.4, None),
                     _layer(_left(2, 2, 32, 16, None, 32, 7.0, 0.25), {"heads": 2, "dim": 24, "vdim": 56}, 0.5, 0.5, 64),
                     _layer(_left(4, 4, 32, 32, 1, None, 1.0, 0.18), {"heads": 4, "dim": 12, "vdim": 12}, 1.0, 1.0, 64)]},
    # nothing a multiple of eight: odd head sizes (values of 7), a width of 36, five taps, one layer, no feed-forward
    "s": {"architecture": "Ruvenex", "vocab": 97, "width": 36, "embedding": {"scale": 1.7}, "norm": {"eps": 1e-5},
          "layers": [_layer(_left(2, 1, 10, 7, 5, 6, 30.0, 0.4), {"heads": 1, "dim": 5, "vdim": 9}, 1.1, 0.9, None),
                     _layer(_left(3, 3, 9, 11, 2, 8, 30.0, 0.35), {"heads": 2, "dim": 3, "vdim": 3}, 0.9, 1.1, 20)]},
    # head size 128 with eight query heads on two kv heads; a recurrence state of 64 x 64
    "r": {"architecture": "Ruvenex", "vocab": 256, "width": 128, "embedding": {"scale": 11.3}, "norm": {"eps": 2e-6},
          "layers": [_layer(_left(8, 2, 128, 128, 3, 64, 250000.0, 0.09), {"heads": 2, "dim": 64, "vdim": 64}, 0.8, 1.25, 256)]},
}


def spec_of(cfg: dict):
    return H.spec_of(cfg)


def make_weights(cfg: dict, seed: int, dtype=torch.bfloat16, sharp: float = 0.0) -> Dict[str, torch.Tensor]:
    """Random weights; with ``sharp`` the query projections are multiplied by it, so that attention weights are
    peaked: a position's result then hangs on single keys far back, and a wrong or lost key shows."""
    from infer_b200.weights import random_weights
    W = random_weights(spec_of(cfg), seed, dtype)
    if sharp:
        for k in W:
            if k.endswith(".mix.left.q"):
                W[k] = (W[k].float() * sharp).to(dtype)
    return W


def random_ids(cfg: dict, n: int, seed: int) -> List[int]:
    return np.random.default_rng(seed).integers(0, cfg["vocab"], n).tolist()


@functools.lru_cache(maxsize=64)
def _oracle(cfg_json: str, seed: int, sharp: float, compute: str, ids: Tuple[int, ...], rounding: str):
    cfg = json.loads(cfg_json)
    W = H.as_compute(make_weights(cfg, seed, torch.bfloat16, sharp), getattr(torch, compute))
    return pr.forward(cfg, W, list(ids), None, None if rounding == "none" else getattr(torch, rounding)).numpy()


def oracle(cfg: dict, seed: int, compute: torch.dtype, ids: Sequence[int], rounding=None, sharp: float = 0.0) -> np.ndarray:
    n = lambda d: str(d).replace("torch.", "")
    return _oracle(json.dumps(cfg, sort_keys=True), seed, float(sharp), n(compute), tuple(int(i) for i in ids),
                   "none" if rounding is None else n(rounding))


def check_bf16(got: np.ndarray, ref: np.ndarray, ref_rounded: np.ndarray, what: str, factor: float = 3.0):
    """The bfloat16 path against the exact plain implementation. Rounding noise differs much between positions of
    this design (a value head that is nearly zero before its norm, a gate on its slope), so every position is held
    against the noise that the plain implementation with bfloat16 roundings shows AT THAT POSITION (or the average
    over positions, where that is larger), times ``factor``; and all positions together against the average."""
    rms = lambda a: np.sqrt(np.mean(a ** 2, axis=-1))
    noise_rows, noise = rms(ref_rounded - ref), float(rms((ref_rounded - ref).ravel()))
    floor = 1e-3 * float(rms(ref.ravel()))
    err_rows, err = rms(got - ref), float(rms((got - ref).ravel()))
    assert err <= factor * max(noise, floor), f"{what}: rms diff {err:.3e} > {factor} x rounding noise {noise:.3e}"
    bound = factor * np.maximum(noise_rows, max(noise, floor))
    worst = int(np.argmax(err_rows / bound))
    assert err_rows[worst] <= bound[worst], \
        f"{what}: row {worst}: rms diff {err_rows[worst]:.3e} > {bound[worst]:.3e} (its rounding noise {noise_rows[worst]:.3e})"


def check(cfg: dict, seed: int, dtype: torch.dtype, got: Dict[str, Dict[int, np.ndarray]], reqs: Dict[str, List[int]],
          sharp: float = 0.0, what: str = ""):
    for rid, ids in reqs.items():
        ref = oracle(cfg, seed, dtype, ids, None, sharp)
        rows = sorted(got[rid])
        g = np.stack([got[rid][p] for p in rows])
        if dtype == torch.float32:
            H.check_f32(g, ref[rows], f"{what}/{rid}")
        else:
            check_bf16(g, ref[rows], oracle(cfg, seed, dtype, ids, torch.bfloat16, sharp)[rows], f"{what}/{rid}")
