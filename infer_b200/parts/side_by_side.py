"""Two mixers that read the same rows; the result is a * first(x) + b * second(x).

The spec holds the two mixers' own specs under ``first`` and ``second`` (family "mixer", any registered kinds; their
prefixes are relative to this part's) and the two constants.  Each keeps its own pages or state: the part's need is
the two needs by name.  Tensors are declared and loaded through the two mixers' classes.

With ``first_norm`` / ``second_norm`` (local names of two weights [hidden_size]) and ``norm_eps``, each result is
divided by its root mean square over the width and multiplied by its weight before the two are weighed and added:
a * first(x) / rms * w1 + b * second(x) / rms * w2.
"""
from __future__ import annotations

import torch

from ..config.specs import PartSpec
from .base import CompositeNeed, Mixer, build_part, part_class, register_mixer

_SIDES = ("first", "second")


@register_mixer("side_by_side")
class SideBySide(Mixer):
    def __init__(self, spec: PartSpec, runtime):
        super().__init__(spec, runtime)
        self.sides = {s: build_part("mixer", spec[s], runtime) for s in _SIDES}
        self.scales = {"first": float(spec.get("first_scale", 1.0)), "second": float(spec.get("second_scale", 1.0))}
        self.graph_safe = all(getattr(m, "graph_safe", True) for m in self.sides.values())
        self.norm_names = {s: spec.get(s + "_norm") for s in _SIDES}
        self.normed = any(v is not None for v in self.norm_names.values())
        if self.normed and (None in self.norm_names.values() or not float(spec.get("norm_eps") or 0.0) > 0):
            raise ValueError("side_by_side norms need both weights' names, hidden_size and a positive norm_eps")
        self.norm_eps = float(spec.get("norm_eps") or 0.0)
        self.norm_w = {}

    @classmethod
    def param_shapes(cls, spec):
        shapes = {}
        for s in _SIDES:
            sub = spec[s]
            for local, shape in part_class("mixer", sub.kind).param_shapes(sub).items():
                shapes[sub.prefix + local] = shape
        for s in _SIDES:
            if spec.get(s + "_norm") is not None:
                shapes[str(spec[s + "_norm"])] = (int(spec["hidden_size"]),)
        return shapes

    @classmethod
    def init_params(cls, spec, name, shape, gen):
        if name in (spec.get("first_norm"), spec.get("second_norm")):
            return 1.0 + 0.1 * torch.randn(shape, generator=gen, dtype=torch.float32, device=gen.device)
        for s in _SIDES:
            sub = spec[s]
            sub_cls = part_class("mixer", sub.kind)
            if name.startswith(sub.prefix) and name[len(sub.prefix):] in sub_cls.param_shapes(sub):
                return sub_cls.init_params(sub, name[len(sub.prefix):], shape, gen)
        return super().init_params(spec, name, shape, gen)

    def load(self, params):
        for s, m in self.sides.items():
            sub = self.spec[s]
            m.load({local: params[sub.prefix + local] for local in type(m).param_shapes(sub)})
            if self.normed:
                self.norm_w[s] = params[str(self.norm_names[s])].to(device=self.rt.device, dtype=torch.float32).contiguous()

    def members(self):
        """The two mixers, for a block that joins first products across its parts."""
        return list(self.sides.values())

    def cache_need(self):
        return CompositeNeed({s: m.cache_need() for s, m in self.sides.items()})

    def forward_sides(self, x, step, cache, write_cache=True, side_stream=None):
        """(first(x), second(x)) as float32, and the two constants: for a block whose sum applies them. With
        ``side_stream`` the second mixer's kernels go to that stream (the two read the same rows and write nothing in
        common); the caller has made it wait for the rows and waits for ``side_stream`` before it reads the result."""
        from .base import DeferredNorm, ProjectedInput

        def arg(m):
            if not isinstance(x, ProjectedInput) or hasattr(m, "input_product"):
                return x
            return x.rows_in.materialize() if isinstance(x.rows_in, DeferredNorm) else x.rows_in
        if side_stream is not None:
            with torch.cuda.stream(side_stream):
                b = self.sides["second"].forward(arg(self.sides["second"]), step, cache["second"], None, write_cache)
        a = self.sides["first"].forward(arg(self.sides["first"]), step, cache["first"], None, write_cache)
        if side_stream is None:
            b = self.sides["second"].forward(arg(self.sides["second"]), step, cache["second"], None, write_cache)
        return a, b, self.scales["first"], self.scales["second"]

    def forward_normed(self, x, step, cache, write_cache, h, out_norm, copy_dtype, side_stream=None):
        """For a block that normalises what the mixer returns and adds it to h: with norms on the two sides, the two
        norms, the weighing, the block's norm and the sum are one kernel. Returns (h, its copy in copy_dtype) or None.
        With ``side_stream`` the second mixer runs there, beside the first (forked and joined by events here)."""
        if not self.normed:
            return None
        from .. import ops
        if side_stream is not None:
            main = torch.cuda.current_stream(h.device)
            fork = torch.cuda.Event()
            fork.record(main)
            side_stream.wait_event(fork)
        a, b, sa, sb = self.forward_sides(x, step, cache, write_cache, side_stream)
        if side_stream is not None:
            done = torch.cuda.Event()
            done.record(side_stream)
            main.wait_event(done)
        return ops.dual_norm_sum(a, self.norm_w["first"], sa, b, self.norm_w["second"], sb, self.norm_eps, h, out_norm.weight,
                                 out_norm.eps, copy_dtype)

    def forward(self, x, step, cache, residual, write_cache=True):
        from .. import ops
        a, b, sa, sb = self.forward_sides(x, step, cache, write_cache)
        if self.normed:
            m, _ = ops.dual_norm_sum(a, self.norm_w["first"], sa, b, self.norm_w["second"], sb, self.norm_eps)
            return m if residual is None else ops.gated_sum(residual, None, m)
        if residual is None:
            residual = torch.zeros_like(a)
        return ops.gated_sum(residual, None, a, sa, b, sb)
