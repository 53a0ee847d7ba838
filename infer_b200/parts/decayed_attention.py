"""Linear attention whose key channels forget at learned, input-dependent rates (gated linear attention).

Per head, with x the mixer's input row at a position:

    q = x Wq^T * dim^(-1/2),   k = x Wk^T            [dim]
    v = x Wv^T                                        [v_dim]
    a = sigmoid(z) ^ (1 / tau),  z = (x Wlow^T) Wup^T + b       [dim]: a decay per key channel, through a low rank
    S <- diag(a) S + k v^T                            S [dim, v_dim], zero for a new request
    o = S^T q                                         [v_dim]

o is divided by sqrt(mean(o^2) + eps) per head and multiplied by a weight [v_dim] that the heads share; the heads are
joined, multiplied by silu(x Wg^T) and projected by Wo.  S lives in float32 in a state slot of the request and is
carried from step to step.  Decays, their logarithm, the scale of q, the state and the head norm are float32 whatever
the compute dtype: the five projections are one matrix product with float32 result rows, and the second factor of the
low-rank product is applied in float32 by the kernel that also takes the power.

``decay_rank`` None in the spec: the rank is read from the stored tensors.  ``names`` renames the local tensors by role
(q, k, v, gate, o, norm, decay_low, decay_up, decay_bias).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import Mixer, StateNeed, register_mixer
from .linear import Linear

_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "gate": "g_proj.weight", "o": "o_proj.weight",
          "norm": "norm.weight", "decay_low": "decay_proj.0.weight", "decay_up": "decay_proj.1.weight", "decay_bias": "decay_proj.1.bias"}


def _names(spec: PartSpec):
    return {**_NAMES, **dict(spec.get("names") or {})}


@register_mixer("decayed_linear_attention")
class DecayedLinearAttention(Mixer):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden_size"])
        self.n_heads, self.dim = int(spec["num_heads"]), int(spec["head_dim"])
        self.v_dim = int(spec.get("v_head_dim") or self.dim)
        self.tau, self.eps = float(spec["tau"]), float(spec["norm_eps"])
        if min(self.hidden, self.n_heads, self.dim, self.v_dim) <= 0 or self.eps <= 0 or self.tau <= 0:
            raise ValueError("decayed_linear_attention needs positive sizes, tau and eps")
        if self.dim > ops.state_scan_max_dim():
            raise ValueError(f"a key size of {self.dim} is beyond what the recurrence kernel keeps in registers ({ops.state_scan_max_dim()})")
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.rank = 0

    @classmethod
    def param_shapes(cls, spec):
        H, nh, d = int(spec["hidden_size"]), int(spec["num_heads"]), int(spec["head_dim"])
        dv = int(spec.get("v_head_dim") or d)
        r = int(spec["decay_rank"]) if spec.get("decay_rank") is not None else -1
        n = _names(spec)
        return {n["q"]: (nh * d, H), n["k"]: (nh * d, H), n["v"]: (nh * dv, H), n["gate"]: (nh * dv, H), n["o"]: (H, nh * dv),
                n["norm"]: (dv,), n["decay_low"]: (r, H), n["decay_up"]: (nh * d, r), n["decay_bias"]: (nh * d,)}

    @classmethod
    def init_params(cls, spec, name, shape, gen):
        n = _names(spec)
        if name == n["norm"]:
            return 1.0 + 0.1 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        if name == n["decay_bias"]:
            return 2.0 + torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        if name in (n["decay_up"], n["decay_low"]):
            return 0.3 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        return super().init_params(spec, name, shape, gen)

    def load(self, params):
        n = _names(self.spec)
        low, up = params[n["decay_low"]], params[n["decay_up"]]
        self.rank = int(low.shape[0])
        if up.shape[1] != self.rank:
            raise ValueError(f"the two factors of the decay's low-rank product disagree: {tuple(low.shape)} and {tuple(up.shape)}")
        nq, nv = self.n_heads * self.dim, self.n_heads * self.v_dim
        # result rows [q | k | v | low | gate], float32
        self.proj = Linear(self.rt, torch.cat([params[n["q"]], params[n["k"]], params[n["v"]], low, params[n["gate"]]], dim=0))
        self.low_col, self.gate_col = 2 * nq + nv, 2 * nq + nv + self.rank
        f32 = dict(device=self.rt.device, dtype=torch.float32)
        # the second factor keeps the values the checkpoint has, widened: its product runs in float32
        self.up = up.to(self.rt.dtype).to(**f32).t().contiguous()              # [rank, channels]
        self.up_bias = params[n["decay_bias"]].to(**f32).contiguous()
        self.norm_w = params[n["norm"]].to(**f32).contiguous()
        self.o = Linear(self.rt, params[n["o"]])

    def cache_need(self):
        return StateNeed({"S": ((self.n_heads, self.dim, self.v_dim), torch.float32)})

    def forward(self, x, step, cache, residual, write_cache=True):
        nq = self.n_heads * self.dim
        rows = self.proj(x, out_dtype=torch.float32)
        decay = ops.decay_gates(rows, 0, self.low_col, self.rank, self.up, self.up_bias, self.tau, float(self.dim) ** -0.5)
        o = ops.state_scan(ops.SCAN_ROW_DECAY, rows, 0, nq, 2 * nq, decay, 0, cache["S"], step.seg_start, step.seg_slot,
                           self.n_heads, 1, self.dim, self.v_dim, write_cache, step.max_q_len)
        y = ops.head_norm_gate(o, self.norm_w, self.eps, rows, self.gate_col, self.n_heads, self.v_dim, self.rt.dtype)
        if residual is None:
            return self.o(y, out_dtype=torch.float32)
        return self.o(y, residual=residual)
