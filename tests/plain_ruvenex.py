"""The Ruvenex decoder written out slowly: whole sequences, no cache, torch on the CPU in float64.

One function per mechanism. It shares no code with ``infer_b200``: it reads the raw config.json dictionary and a
dictionary of checkpoint tensors by their names in the file. Everything the engine does for this design is compared
with this file.

A layer, with n = rms_weighted(x):

    x <- x + sigmoid(R1 n + r1) * mixer(n) + sigmoid(R2 n + r2) * feed_forward(n)         (second term absent without one)
    mixer(n) = a * attention_side(n) + b * recurrent_side(n)

attention_side: q, k, v = projections of n, each passed through a short causal depthwise filter over time; q and k
rotated in adjacent pairs over their first ``rot.dims`` channels; v divided by its root mean square per head; causal
softmax attention with the configured score scale and grouped key/value heads; every head's result times
sigmoid(G n)[head]; output projection.

recurrent_side (per head, state S of [dim, vdim] starting at zero):
    f_t = l + (1 - l) * sigmoid(F n_t + c),   q_t = silu(Q n_t),   v_t = V n_t
    S_t = diag(f_t) S_{t-1} + (1 - f_t) v_t^T,   o_t = S_t^T q_t
then o_t is rms-normalised per head with a weight shared by the heads, heads are joined and projected.

``rounding``: None computes exactly. ``torch.bfloat16`` rounds activations where a bfloat16 serving path stores them
(normalised rows, projected and prepared q/k/v, contexts, feed-forward activations, the recurrence's normalised
output), which gives the size of the rounding noise such a path must have.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Sequence

import torch

F = torch.float64


def _rnd(x: torch.Tensor, rounding) -> torch.Tensor:
    return x if rounding is None else x.to(rounding).to(x.dtype)


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_weighted(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return rms(x, eps) * w.to(F)


def linear(x: torch.Tensor, W: torch.Tensor, b: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = x @ W.to(F).T
    return y if b is None else y + b.to(F)


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def short_filter(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]. y[t] = sum_j w[:, j] * u[t - (taps - 1) + j], zero before the start."""
    T, C = u.shape
    taps = w.shape[1]
    w = w.to(F)
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=u.dtype), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * w[:, j]
    return y


def rotate_pairs(x: torch.Tensor, n_rot: int, base: float, positions: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, heads, dim]. Channels (2i, 2i+1), i < n_rot/2, turn by the angle p * base^(-2i/n_rot); the other
    channels stay. The angle is a float32 product of a float32 position and a float32 frequency."""
    T = x.shape[0]
    p = torch.arange(T, dtype=torch.float32) if positions is None else positions.to(torch.float32)
    i = torch.arange(n_rot // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / n_rot).to(torch.float32)
    ang = (p[:, None] * freq[None, :]).to(F)                       # [T, n_rot/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:n_rot:2], x[..., 1:n_rot:2]
    out[..., 0:n_rot:2] = a * c - b * s
    out[..., 1:n_rot:2] = b * c + a * s
    return out


def causal_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv]; query head h reads key/value head h // (H / G)."""
    T, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    mask = torch.ones(T, T, dtype=torch.bool).tril()
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def attention_side(n: torch.Tensor, W: Mapping[str, torch.Tensor], pre: str, cfg: Mapping, eps: float, rounding=None) -> torch.Tensor:
    H, d = cfg["heads"], cfg["dim"]
    G = cfg["kv_heads"] if cfg.get("kv_heads") is not None else H
    dv = cfg["vdim"] if cfg.get("vdim") is not None else d
    T = n.shape[0]
    q, k, v = (_rnd(linear(n, W[pre + x]), rounding) for x in ("q", "k", "v"))
    if cfg.get("conv"):
        q, k, v = (short_filter(u, W[pre + x + ".conv"]) for u, x in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.view(T, H, d), k.view(T, G, d), v.view(T, G, dv)
    if cfg.get("rot") is not None and cfg["rot"]["dims"]:
        q = rotate_pairs(q, cfg["rot"]["dims"], cfg["rot"]["base"])
        k = rotate_pairs(k, cfg["rot"]["dims"], cfg["rot"]["base"])
    q, k, v = _rnd(q, rounding), _rnd(k, rounding), _rnd(rms(v, eps), rounding)
    o = _rnd(causal_attention(q, k, v, float(cfg["scale"])), rounding)
    gate = torch.sigmoid(_rnd(linear(n, W[pre + "g"]), rounding))   # [T, H]
    o = _rnd(o * gate[:, :, None], rounding)
    return linear(o.reshape(T, H * dv), W[pre + "o"])


def gated_recurrence(q: torch.Tensor, f: torch.Tensor, v: torch.Tensor, state: Optional[torch.Tensor] = None):
    """q, f [T, H, d], v [T, H, dv]; state [H, d, dv] or None (zeros). Returns (o [T, H, dv], last state)."""
    T, H, d = q.shape
    S = torch.zeros(H, d, v.shape[2], dtype=q.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def recurrent_side(n: torch.Tensor, W: Mapping[str, torch.Tensor], pre: str, cfg: Mapping, eps: float, rounding=None) -> torch.Tensor:
    H, d = cfg["heads"], cfg["dim"]
    dv = cfg["vdim"] if cfg.get("vdim") is not None else d
    T = n.shape[0]
    q = torch.nn.functional.silu(linear(n, W[pre + "q"])).view(T, H, d)
    v = linear(n, W[pre + "v"]).view(T, H, dv)
    low = W[pre + "lower"].to(F)
    f = (low + (1.0 - low) * torch.sigmoid(linear(n, W[pre + "f"], W[pre + "f.b"]))).view(T, H, d)
    o, _ = gated_recurrence(q, f, v)
    o = _rnd(rms(o, eps) * W[pre + "norm"].to(F), rounding)
    return linear(o.reshape(T, H * dv), W[pre + "o"])


def feed_forward(n: torch.Tensor, W: Mapping[str, torch.Tensor], pre: str, rounding=None) -> torch.Tensor:
    return linear(_rnd(gelu_tanh(_rnd(linear(n, W[pre + "up"]), rounding)), rounding), W[pre + "down"])


def layer(x: torch.Tensor, W: Mapping[str, torch.Tensor], i: int, lcfg: Mapping, eps: float, rounding=None) -> torch.Tensor:
    if lcfg["type"] != "parallel":
        raise ValueError(f"layer type {lcfg['type']!r}")
    p = f"l{i}."
    n = _rnd(rms_weighted(x, W[p + "norm1"], eps), rounding)
    m = lcfg["mixer"]
    mix = float(m["left_scale"]) * attention_side(n, W, p + "mix.left.", m["left"], eps, rounding) + \
        float(m["right_scale"]) * recurrent_side(n, W, p + "mix.right.", m["right"], eps, rounding)
    y = torch.sigmoid(linear(n, W[p + "rg1"], W[p + "rg1.b"])) * mix
    if lcfg.get("mlp") is not None:
        if lcfg["mlp"]["kind"] != "dense":
            raise ValueError("feed-forward kind")
        y = y + torch.sigmoid(linear(n, W[p + "rg2"], W[p + "rg2.b"])) * feed_forward(n, W, p + "mlp.", rounding)
    return x + y


def forward(cfg: Mapping, W: Mapping[str, torch.Tensor], tokens: Sequence[int], layers_out: Optional[List] = None,
            rounding=None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence. ``layers_out`` collects the stream after every layer."""
    ids = torch.as_tensor(list(tokens), dtype=torch.long)
    x = W["embed"].to(F)[ids] * float(cfg["embedding"]["scale"])
    eps = float(cfg["norm"]["eps"])
    for i, lcfg in enumerate(cfg["layers"]):
        x = layer(x, W, i, lcfg, eps, rounding)
        if layers_out is not None:
            layers_out.append(x.clone())
    return linear(_rnd(rms_weighted(x, W["final.norm"], eps), rounding), W["head"])


def greedy(cfg: Mapping, W: Mapping[str, torch.Tensor], prompt: Sequence[int], n_new: int) -> List[int]:
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(torch.argmax(forward(cfg, W, toks)[-1])))
    return toks[len(prompt):]
