"""Gated delta rule: a linear recurrence that, before it writes a value under a key, takes out what the state already
returns for that key.

With x the mixer's input row at a position, ``num_qk_heads`` heads of q and k of size dim (value head h reads head
h // (num_heads / num_qk_heads)) and ``num_heads`` heads of v of size v_dim:

    q, k, v = silu(filter(x Wq^T)), silu(filter(x Wk^T)), silu(filter(x Wv^T))     a short causal filter over time per
                                                       channel; zeros before the sequence
    q <- q / sqrt(sum(q^2) + unit_eps) * dim^(-1/2),   k <- k / sqrt(sum(k^2) + unit_eps)              per head
    beta = sigmoid(x Wb^T)[h],    g = exp(-exp(A_log[h]) * softplus(x Wa^T [h] + dt_bias[h]))           per value head
    S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q             S [dim, v_dim], zero for a new request

o is divided by sqrt(mean(o^2) + eps) per head, multiplied by a weight [v_dim] that the heads share and by
silu(x Wg^T); the heads are joined and projected by Wo.  S (float32) and the filters' last taps - 1 projected rows
(float32) are the request's state.  Step sizes, decays, write strengths, unit norms, the state and the head norm are
float32 whatever the compute dtype: the six projections are one matrix product with float32 result rows.

``names`` renames the local tensors by role (q, k, v, q_filter, k_filter, v_filter, beta, step, a_log, dt_bias, gate,
norm, o).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import Mixer, StateNeed, register_mixer
from .linear import Linear

_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "q_filter": "q_proj.filter", "k_filter": "k_proj.filter",
          "v_filter": "v_proj.filter", "beta": "b_proj.weight", "step": "a_proj.weight", "a_log": "A_log", "dt_bias": "dt_bias",
          "gate": "g_proj.weight", "norm": "norm.weight", "o": "o_proj.weight"}


def _names(spec: PartSpec):
    return {**_NAMES, **dict(spec.get("names") or {})}


@register_mixer("gated_delta_rule")
class GatedDeltaRule(Mixer):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden_size"])
        self.n_heads, self.n_qk = int(spec["num_heads"]), int(spec.get("num_qk_heads") or spec["num_heads"])
        self.dim, self.v_dim = int(spec["head_dim"]), int(spec.get("v_head_dim") or spec["head_dim"])
        self.taps = int(spec.get("filter_taps") or 0)
        self.eps, self.unit_eps = float(spec["norm_eps"]), float(spec.get("unit_eps", 1e-6))
        if min(self.hidden, self.n_heads, self.n_qk, self.dim, self.v_dim) <= 0 or self.eps <= 0 or self.taps < 0:
            raise ValueError("gated_delta_rule needs positive sizes and eps")
        if self.n_heads % self.n_qk:
            raise ValueError(f"heads ({self.n_heads}) must be a multiple of the (q, k) heads ({self.n_qk})")
        if self.dim > min(ops.state_scan_max_dim(), ops.delta_prepare_max_dim()):
            raise ValueError(f"a key size of {self.dim} is beyond what the recurrence kernels take")
        self.channels = 2 * self.n_qk * self.dim + self.n_heads * self.v_dim
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.filter_w = None

    @classmethod
    def param_shapes(cls, spec):
        H, nh, d = int(spec["hidden_size"]), int(spec["num_heads"]), int(spec["head_dim"])
        g, dv = int(spec.get("num_qk_heads") or nh), int(spec.get("v_head_dim") or d)
        taps = int(spec.get("filter_taps") or 0)
        n = _names(spec)
        shapes = {n["q"]: (g * d, H), n["k"]: (g * d, H), n["v"]: (nh * dv, H), n["beta"]: (nh, H), n["step"]: (nh, H),
                  n["a_log"]: (nh,), n["dt_bias"]: (nh,), n["gate"]: (nh * dv, H), n["norm"]: (dv,), n["o"]: (H, nh * dv)}
        if taps > 0:
            shapes.update({n["q_filter"]: (g * d, taps), n["k_filter"]: (g * d, taps), n["v_filter"]: (nh * dv, taps)})
        return shapes

    @classmethod
    def init_params(cls, spec, name, shape, gen):
        n = _names(spec)
        kw = dict(generator=gen, dtype=torch.float32, device=gen.device)
        if name in (n["q_filter"], n["k_filter"], n["v_filter"]):
            w = 0.3 * torch.randn(shape, **kw)
            w[:, -1] += 1.0
            return w
        if name == n["norm"]:
            return 1.0 + 0.1 * torch.randn(shape, **kw)
        if name == n["a_log"]:
            return torch.log(0.1 + 2.0 * torch.rand(shape, **kw))
        if name == n["dt_bias"]:
            return torch.randn(shape, **kw) - 2.0
        if name in (n["q"], n["k"], n["v"], n["beta"], n["step"]):
            return 0.3 * torch.randn(shape, **kw)
        return super().init_params(spec, name, shape, gen)

    def load(self, params):
        n = _names(self.spec)
        # result rows [q | k | v | step sizes | write strengths | gate], float32
        self.proj = Linear(self.rt, torch.cat([params[n[r]] for r in ("q", "k", "v", "step", "beta", "gate")], dim=0))
        self.step_col = self.channels
        self.beta_col = self.channels + self.n_heads
        self.gate_col = self.channels + 2 * self.n_heads
        f32 = dict(device=self.rt.device, dtype=torch.float32)
        self.a_log = params[n["a_log"]].to(**f32).contiguous()
        self.dt_bias = params[n["dt_bias"]].to(**f32).contiguous()
        self.norm_w = params[n["norm"]].to(**f32).contiguous()
        self.o = Linear(self.rt, params[n["o"]])
        if self.taps > 0:
            # tap-major [taps, channels]
            self.filter_w = torch.cat([params[n["q_filter"]], params[n["k_filter"]], params[n["v_filter"]]], dim=0).to(**f32).t().contiguous()

    def cache_need(self):
        shapes = {"S": ((self.n_heads, self.dim, self.v_dim), torch.float32)}
        if self.taps > 1:
            shapes["tails"] = ((self.taps - 1, self.channels), torch.float32)
        return StateNeed(shapes)

    def forward(self, x, step, cache, residual, write_cache=True):
        rows = self.proj(x, out_dtype=torch.float32)
        tails = cache.get("tails")
        # with one token per request, the lane that filters a channel is the only reader of its tail and moves it too
        inline_tail = tails is not None and write_cache and step.max_q_len == 1
        prep = ops.delta_prepare(rows, 0, self.step_col, self.beta_col, self.filter_w, tails, self.a_log, self.dt_bias,
                                 self.unit_eps, float(self.dim) ** -0.5, step, self.n_heads, self.n_qk, self.dim, self.v_dim, inline_tail)
        if tails is not None and write_cache and not inline_tail:
            ops.tail_update(rows, 0, tails, step.seg_start, step.seg_slot)
        nqk = self.n_qk * self.dim
        o = ops.state_scan(ops.SCAN_DELTA_RULE, prep, 0, nqk, 2 * nqk, prep, self.channels, cache["S"], step.seg_start,
                           step.seg_slot, self.n_heads, self.n_heads // self.n_qk, self.dim, self.v_dim, write_cache, step.max_q_len)
        y = ops.head_norm_gate(o, self.norm_w, self.eps, rows, self.gate_col, self.n_heads, self.v_dim, self.rt.dtype)
        if residual is None:
            return self.o(y, out_dtype=torch.float32)
        return self.o(y, residual=residual)
