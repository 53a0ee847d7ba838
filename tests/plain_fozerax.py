"""The Fozerax decoder written out slowly: whole sequences, no cache, torch on the CPU in float64.

One function per mechanism. It shares no code with ``infer_b200``: it reads the raw config.json dictionary and a
dictionary of checkpoint tensors by their names in the file. Everything the engine does for this design is compared
with this file.

The residual stream x starts as rms_weighted(table[token]). A layer reads x itself and normalises what a sublayer
returns, not what it reads:

    x <- x + rms_weighted(mixer(x), w1);   x <- x + rms_weighted(feed_forward(x), w2)     (second line absent without one)

Mixers: ``decayed_linear_attention`` (layer type "gla": a matrix state per head whose rows decay by a learned,
input-dependent factor per key channel) and ``window_and_delta`` (layer type "parallel": sliding-window softmax
attention with a learned bias per distance bucket and a sink, beside a gated delta-rule recurrence behind short
causal filters; each side normalised over the width, the mean of the two).
Feed-forwards: ``dense_gated`` and ``routed_experts`` (softmax router, groups of neighbouring experts, a shared expert).

``ROUNDING``: None computes exactly. Set to ``torch.bfloat16`` (see ``rounded``), activations are rounded where a
bfloat16 serving path stores them (the rows a sublayer reads, q/k/v of attention and its contexts, hidden layers of
feed-forwards, what a recurrence hands to its output matrix), which gives the size of the rounding noise such a path
must have.
"""
from __future__ import annotations

import math
from typing import Dict, List, Mapping, Optional, Sequence

import torch

F = torch.float64
UNIT_EPS = 1e-6            # inside the root when q and k of the delta rule are made unit vectors
WEIGHT_SUM_EPS = 1e-20     # added to the sum of the chosen experts' scores
EXPERT_SLOPE = 1.702       # g * sigmoid(EXPERT_SLOPE * g)


ROUNDING = None


class rounded:
    """with rounded(torch.bfloat16): ... computes with activations rounded where a serving path stores them."""

    def __init__(self, dtype):
        self.dtype = dtype

    def __enter__(self):
        global ROUNDING
        self.old, ROUNDING = ROUNDING, self.dtype

    def __exit__(self, *exc):
        global ROUNDING
        ROUNDING = self.old


def _rnd(x: torch.Tensor) -> torch.Tensor:
    return x if ROUNDING is None else x.to(ROUNDING).to(x.dtype)


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


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# ----------------------------------------------------------------------------- recurrences

def decayed_state_scan(q, k, v, decay, S0=None):
    """One head. q, k, decay [T, d]; v [T, dv]. S_t = diag(decay_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.
    Returns (o [T, dv], S_T)."""
    T, d = q.shape
    S = torch.zeros(d, v.shape[1], dtype=F) if S0 is None else S0.clone()
    out = []
    for t in range(T):
        S = decay[t][:, None] * S + k[t][:, None] * v[t][None, :]
        out.append(S.T @ q[t])
    return torch.stack(out) if out else torch.zeros(0, v.shape[1], dtype=F), S


def delta_rule_scan(q, k, v, g, beta, S0=None):
    """One head. q, k [T, d]; v [T, dv]; g, beta [T]. S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q
    (the read-out sees the token's own write). Returns (o [T, dv], S_T)."""
    T, d = q.shape
    S = torch.zeros(d, v.shape[1], dtype=F) if S0 is None else S0.clone()
    out = []
    for t in range(T):
        S = g[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + k[t][:, None] * u[None, :]
        out.append(S.T @ q[t])
    return torch.stack(out) if out else torch.zeros(0, v.shape[1], dtype=F), S


def causal_filter(u: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """u [T, C], w [C, taps]; the last tap multiplies the current row: y[t] = sum_j w[:, j] u[t - (taps - 1) + j],
    zeros before the start."""
    T, C = u.shape
    taps = w.shape[1]
    pad = torch.cat([torch.zeros(taps - 1, C, dtype=F), u])
    y = torch.zeros(T, C, dtype=F)
    for j in range(taps):
        y = y + pad[j:j + T] * w.to(F)[:, j]
    return y


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + UNIT_EPS)


# ----------------------------------------------------------------------------- mixers

def decayed_linear_attention(h, m: Mapping, W: Mapping[str, torch.Tensor], p: str, eps: float):
    """Layer type "gla". h [T, width]; m the layer's 'mixer' dictionary; tensors p + q, k, v, g, o, norm, a1, a2, a2.b."""
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    T = h.shape[0]
    q = (linear(h, W[p + "q"]) * d ** -0.5).view(T, H, d)
    k = linear(h, W[p + "k"]).view(T, H, d)
    v = linear(h, W[p + "v"]).view(T, H, dv)
    z = linear(linear(h, W[p + "a1"]), W[p + "a2"], W[p + "a2.b"]).view(T, H, d)
    decay = torch.exp(torch.nn.functional.logsigmoid(z) / tau)         # sigmoid(z) ** (1 / tau)
    o = torch.stack([decayed_state_scan(q[:, i], k[:, i], v[:, i], decay[:, i])[0] for i in range(H)], dim=1)
    o = rms_weighted(o, W[p + "norm"], eps).reshape(T, H * dv)
    return linear(_rnd(o * silu(linear(h, W[p + "g"]))), W[p + "o"])


def distance_bucket(n: int, B: int, D: float) -> int:
    """Row of the bias table for a distance n >= 0: one row per distance below B // 2, logarithmic steps up to D."""
    half = B // 2
    if n < half:
        return n
    return min(B - 1, half + int(math.floor(math.log(n / half) / math.log(D / half) * (B - half))))


def windowed_attention(h, m: Mapping, W: Mapping[str, torch.Tensor], p: str, eps: float):
    """Left side of layer type "parallel": biased projections, one norm over all of q and one over all of k, a score
    scale from the configuration, a bias per (distance bucket, head), a window, a sink in the softmax denominator."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = _rnd(rms_weighted(_rnd(linear(h, W[p + "q"], W[p + "q.b"])), W[p + "q.norm"], eps)).view(T, H, d)
    k = _rnd(rms_weighted(_rnd(linear(h, W[p + "k"], W[p + "k.b"])), W[p + "k.norm"], eps)).view(T, G, d)
    v = _rnd(linear(h, W[p + "v"], W[p + "v.b"])).view(T, G, dv)
    rel = W[p + "rel"].to(F)
    B = rel.shape[0]
    window = (m.get("mask") or {}).get("size")
    i = torch.arange(T)
    dist = i[:, None] - i[None, :]
    seen = (dist >= 0) & ((dist < window) if window else torch.ones_like(dist, dtype=torch.bool))
    bucket = torch.tensor([distance_bucket(n, B, float(m["bias_max"])) for n in range(max(T, 1))])[dist.clamp(min=0)]
    out = torch.zeros(T, H, dv, dtype=F)
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * float(m["scale"]) + rel[bucket, a]
        s = s.masked_fill(~seen, -math.inf)
        sink = W[p + "sink"].to(F)[a]
        top = torch.maximum(s.max(dim=-1).values, sink)
        e = torch.exp(s - top[:, None])
        out[:, a] = (e / (e.sum(dim=-1) + torch.exp(sink - top))[:, None]) @ v[:, g]
    return linear(_rnd(out.reshape(T, H * dv)), W[p + "o"])


def gated_delta_rule(h, m: Mapping, W: Mapping[str, torch.Tensor], p: str, eps: float):
    """Right side of layer type "parallel"."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    filt = (lambda u, name: causal_filter(u, W[p + name])) if m.get("conv") else (lambda u, name: u)      # conv 0: no filter
    q = silu(filt(linear(h, W[p + "q"]), "q.conv")).view(T, G, d)
    k = silu(filt(linear(h, W[p + "k"]), "k.conv")).view(T, G, d)
    v = silu(filt(linear(h, W[p + "v"]), "v.conv")).view(T, H, dv)
    q, k = unit(q) * d ** -0.5, unit(k)
    beta = torch.sigmoid(linear(h, W[p + "b"]))                                              # [T, H]
    g = torch.exp(-torch.exp(W[p + "A_log"].to(F)) * torch.nn.functional.softplus(linear(h, W[p + "a"]) + W[p + "dt_bias"].to(F)))
    o = torch.stack([delta_rule_scan(q[:, i // (H // G)], k[:, i // (H // G)], v[:, i], g[:, i], beta[:, i])[0]
                     for i in range(H)], dim=1)
    o = rms_weighted(o, W[p + "norm"], eps).reshape(T, H * dv)
    return linear(_rnd(o * silu(linear(h, W[p + "g"]))), W[p + "o"])


def window_and_delta(h, m: Mapping, W: Mapping[str, torch.Tensor], p: str, eps: float):
    left = rms_weighted(windowed_attention(h, m["left"], W, p + "left.", eps), W[p + "left.out"], eps)
    right = rms_weighted(gated_delta_rule(h, m["right"], W, p + "right.", eps), W[p + "right.out"], eps)
    return 0.5 * (left + right)


# ----------------------------------------------------------------------------- feed-forwards

def dense_gated(h, W: Mapping[str, torch.Tensor], p: str):
    return linear(_rnd(gelu_tanh(_rnd(linear(h, W[p + "gate"]))) * _rnd(linear(h, W[p + "up"]))), W[p + "down"])


def clipped_expert(h, W: Mapping[str, torch.Tensor], p: str, limit: float):
    g = torch.clamp(_rnd(linear(h, W[p + "gate"])), max=limit)
    u = torch.clamp(_rnd(linear(h, W[p + "up"])), -limit, limit)
    return linear(_rnd(g * torch.sigmoid(EXPERT_SLOPE * g) * (u + 1.0)), W[p + "down"])


def route(h, mlp: Mapping, W: Mapping[str, torch.Tensor], p: str):
    """(chosen experts [T, top], their weights [T, top])."""
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    s = torch.softmax(linear(h, W[p + "router"]), dim=-1)
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = E // groups["count"]
    best = s.view(-1, groups["count"], per).max(dim=-1).values.topk(groups["keep"], dim=-1).indices      # [T, keep]
    allowed = torch.zeros(s.shape[0], groups["count"], dtype=torch.bool).scatter_(1, best, True).repeat_interleave(per, dim=1)
    chosen = s.masked_fill(~allowed, -1.0).topk(top, dim=-1).indices
    w = s.gather(1, chosen)
    return chosen, w / (w.sum(dim=-1, keepdim=True) + WEIGHT_SUM_EPS)


def route_margin(h, mlp: Mapping, W: Mapping[str, torch.Tensor], p: str) -> torch.Tensor:
    """Per token, how close the router's choice is to another one: the smallest gap between the logit of the last
    group kept (its best expert) and the best group not kept, and between the last expert chosen and the best allowed
    one not chosen, each divided by the size of the two logits' terms, |Wa * x| + |Wb * x| (what a relative rounding
    of x moves them by). Infinite where there is no alternative. A comparison of roundings leaves out tokens whose gap
    is within the rounding."""
    r = mlp["router"]
    E, top = r["experts"], r["top"]
    Wr = W[p + "router"].to(F)
    z = linear(h, Wr)
    size = torch.sqrt(((h[:, None, :] * Wr[None, :, :]) ** 2).sum(dim=-1))                  # [T, E]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per, T = E // groups["count"], h.shape[0]
    gap = torch.full((T,), math.inf, dtype=F)

    def rel(a, b):
        return (z.gather(1, a[:, None]) - z.gather(1, b[:, None]))[:, 0] / (size.gather(1, a[:, None]) + size.gather(1, b[:, None]))[:, 0]
    gz, garg = z.view(T, groups["count"], per).max(dim=-1)
    order = gz.argsort(dim=-1, descending=True)
    expert_of = lambda g: g * per + garg.gather(1, g[:, None])[:, 0]
    if groups["keep"] < groups["count"]:
        gap = rel(expert_of(order[:, groups["keep"] - 1]), expert_of(order[:, groups["keep"]]))
    allowed = torch.zeros(T, groups["count"], dtype=torch.bool).scatter_(1, order[:, :groups["keep"]], True).repeat_interleave(per, dim=1)
    ranked = z.masked_fill(~allowed, -math.inf).argsort(dim=-1, descending=True)
    if top < groups["keep"] * per:
        gap = torch.minimum(gap, rel(ranked[:, top - 1], ranked[:, top]))
    return gap


def routed_experts(h, mlp: Mapping, W: Mapping[str, torch.Tensor], p: str):
    chosen, w = route(h, mlp, W, p)
    out = torch.zeros(h.shape[0], W[p + "e0.down"].shape[0], dtype=F)
    for e in range(mlp["router"]["experts"]):
        for slot in range(chosen.shape[1]):
            rows = (chosen[:, slot] == e).nonzero().flatten()
            if rows.numel():
                out[rows] += w[rows, slot][:, None] * clipped_expert(h[rows], W, f"{p}e{e}.", float(mlp["expert"]["limit"]))
    if mlp.get("shared"):
        out = out + clipped_expert(h, W, p + "shared.", float(mlp["shared"]["limit"]))
    return out


# ----------------------------------------------------------------------------- the model

def forward(cfg: Mapping, W: Mapping[str, torch.Tensor], tokens: Sequence[int], layers_out: Optional[List] = None,
            margins_out: Optional[List] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one whole sequence. ``layers_out`` collects the residual stream after every layer,
    ``margins_out`` the routers' gaps per token (``route_margin``), one tensor per routed layer."""
    eps = float(cfg["norm"]["eps"])
    x = rms_weighted(W["embed"].to(F)[torch.as_tensor(list(tokens), dtype=torch.long)], W["embed.norm"], eps)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mixer = {"gla": decayed_linear_attention, "parallel": window_and_delta}[layer["type"]]
        x = x + rms_weighted(mixer(_rnd(x), layer["mixer"], W, p + "mix.", eps), W[p + "norm1"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            y = dense_gated(_rnd(x), W, p + "mlp.") if mlp["kind"] == "dense" else routed_experts(_rnd(x), mlp, W, p + "mlp.")
            if margins_out is not None and mlp["kind"] != "dense":
                margins_out.append(route_margin(_rnd(x), mlp, W, p + "mlp."))
            x = x + rms_weighted(y, W[p + "norm2"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return linear(_rnd(rms_weighted(x, W["final.norm"], eps)), W["head"])


def greedy(cfg: Mapping, W: Mapping[str, torch.Tensor], prompt: Sequence[int], n_new: int) -> List[int]:
    """n_new tokens, each the first index of the largest logit after the whole sequence so far."""
    ids, out = list(prompt), []
    for _ in range(n_new):
        tok = int(torch.argmax(forward(cfg, W, ids)[-1]))
        ids.append(tok)
        out.append(tok)
    return out
