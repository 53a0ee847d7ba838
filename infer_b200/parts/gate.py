"""Gates on sublayer results: logits = x W^T + b, one row of W per gated channel; the block's sum multiplies a
sublayer's result by sigmoid(logits), element by element.

A part gates ``count`` sublayers of ``hidden_size`` channels each; their matrices ``names[i]`` and biases
``names[i] + bias_suffix`` are joined into one product whose result rows are [gate 0 | gate 1 | ...] in float32.
"""
from __future__ import annotations

import torch

from ..config.specs import PartSpec
from .base import Gate, own_or_projected, register_gate
from .linear import Linear


@register_gate("sigmoid_linear")
class SigmoidLinearGate(Gate):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.hidden = int(spec["hidden_size"])
        self.names = list(spec["names"])
        self.bias_suffix = str(spec.get("bias_suffix", ".bias"))
        if self.hidden <= 0 or not self.names:
            raise ValueError("a gate needs a positive size and at least one matrix")
        self.count = len(self.names)
        self.linear = None

    @classmethod
    def param_shapes(cls, spec):
        H, suffix = int(spec["hidden_size"]), str(spec.get("bias_suffix", ".bias"))
        shapes = {}
        for n in spec["names"]:
            shapes[n] = (H, H)
            shapes[n + suffix] = (H,)
        return shapes

    def load(self, params):
        w = torch.cat([params[n] for n in self.names], dim=0)
        b = torch.cat([params[n + self.bias_suffix].float() for n in self.names])
        self.linear = Linear(self.rt, w, b)

    def input_product(self):
        return self.linear, "float32"

    def drop_input_product(self):
        self.linear = None

    def forward(self, x):
        """(rows, first column): the gates' logits are columns [first, first + count * hidden) of float32 rows."""
        return own_or_projected(self, x, self.linear, torch.float32)
