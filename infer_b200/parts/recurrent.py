"""Gated linear recurrence with a matrix state per head (linear attention whose forget gate also weighs what is
written; the HGRN2 form).

Per head, with x the mixer's input row at a position:

    q = silu(x Wq^T)                      [dim]
    v = x Wv^T                            [v_dim]
    f = low + (1 - low) * sigmoid(x Wf^T + bf)        [dim], ``low`` a stored lower bound per channel
    S <- diag(f) S + (1 - f) v^T          S [dim, v_dim], zero for a new request
    o = S^T q                             [v_dim]

o is divided by sqrt(mean(o^2) + eps) per head and multiplied by a weight [v_dim] that the heads share; the heads are
joined and projected by Wo.  There is no key and no further scale.  S lives in float32 in a state slot of the request
and is carried from step to step; the gate, its squashing and the lower bound are float32 whatever the compute dtype
(the three projections are one matrix product with float32 result rows).

``names`` in the spec renames the local tensors by role (q, f, f_bias, lower, v, norm, o).
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import ops
from ..config.specs import PartSpec
from .base import Mixer, StateNeed, own_or_projected, register_mixer
from .linear import Linear

_NAMES = {"q": "q_proj.weight", "f": "f_proj.weight", "f_bias": "f_proj.bias", "lower": "lower_bound",
          "v": "v_proj.weight", "norm": "norm.weight", "o": "o_proj.weight"}


def _names(spec: PartSpec):
    return {**_NAMES, **dict(spec.get("names") or {})}


@register_mixer("gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden_size"])
        self.n_heads, self.dim, self.v_dim = int(spec["num_heads"]), int(spec["head_dim"]), int(spec.get("v_head_dim") or spec["head_dim"])
        self.eps = float(spec["norm_eps"])
        if min(self.hidden, self.n_heads, self.dim, self.v_dim) <= 0 or self.eps <= 0:
            raise ValueError("gated_linear_recurrence needs positive sizes and eps")
        if not ops.gated_recurrence_fits(self.dim, self.v_dim):
            raise ValueError(f"a head's state of {self.dim} x {self.v_dim} is beyond what the recurrence kernel keeps in registers")
        self.proj: Optional[Linear] = None
        self.o: Optional[Linear] = None
        self.lower = self.norm_w = None

    @classmethod
    def param_shapes(cls, spec):
        H, nh, d = int(spec["hidden_size"]), int(spec["num_heads"]), int(spec["head_dim"])
        dv = int(spec.get("v_head_dim") or d)
        n = _names(spec)
        return {n["q"]: (nh * d, H), n["f"]: (nh * d, H), n["f_bias"]: (nh * d,), n["lower"]: (nh * d,),
                n["v"]: (nh * dv, H), n["norm"]: (dv,), n["o"]: (H, nh * dv)}

    @classmethod
    def init_params(cls, spec, name, shape, gen):
        n = _names(spec)
        if name == n["lower"]:
            return torch.rand(shape, generator=gen, dtype=torch.float32, device=gen.device) * 0.9
        if name == n["norm"]:
            return 1.0 + 0.1 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        if name == n["f_bias"]:
            return torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        return super().init_params(spec, name, shape, gen)

    def load(self, params):
        n = _names(self.spec)
        w = torch.cat([params[n["q"]], params[n["f"]], params[n["v"]]], dim=0)
        nq = self.n_heads * self.dim
        fb = params[n["f_bias"]].float()
        b = torch.cat([torch.zeros(nq, device=fb.device), fb, torch.zeros(self.n_heads * self.v_dim, device=fb.device)])
        self.proj = Linear(self.rt, w, b)
        self.o = Linear(self.rt, params[n["o"]])
        self.lower = params[n["lower"]].to(device=self.rt.device, dtype=torch.float32).contiguous()
        self.norm_w = params[n["norm"]].to(device=self.rt.device, dtype=torch.float32).contiguous()

    def cache_need(self):
        return StateNeed({"S": ((self.n_heads, self.dim, self.v_dim), torch.float32)})

    def input_product(self):
        return self.proj, "float32"

    def drop_input_product(self):
        self.proj = None

    def forward(self, x, step, cache, residual, write_cache=True):
        nq = self.n_heads * self.dim
        proj, c0 = own_or_projected(self, x, self.proj, torch.float32)   # [T, q | f | v] from column c0, bias of f added
        o = ops.gated_recurrence(proj, c0, c0 + nq, c0 + 2 * nq, self.lower, self.norm_w, self.eps, cache["S"], step.seg_start,
                                 step.seg_slot, self.n_heads, self.dim, self.v_dim, self.rt.dtype, write_cache, step.max_q_len)
        if residual is None:
            return self.o(o, out_dtype=torch.float32)
        return self.o(o, residual=residual)
