"""Ruvenex without a GPU: configuration, tensor names, cache needs, and the plain implementation's own consistency."""
import copy

import pytest
import torch

import helpers as H
import infer_b200.models  # noqa: F401  (registers the architectures)
import infer_b200.parts  # noqa: F401
import plain_ruvenex as pr
import ruvenex_cases as RC
from infer_b200.cache.manager import CacheManager
from infer_b200.config import parse_config
from infer_b200.config.registry import ConfigError
from infer_b200.parts.base import CompositeNeed, PagedKVNeed, StateNeed
from infer_b200.weights.binder import expected_tensors


@pytest.mark.parametrize("name", sorted(RC.CASES))
def test_config_round_trip_and_tensor_names(name):
    cfg = RC.CASES[name]
    arch, typed = parse_config(cfg)
    assert arch.name == "Ruvenex"
    assert arch.parse(arch.to_dict(typed)) == typed
    names = expected_tensors(arch.to_spec(typed))
    assert {"embed", "final.norm", "head"} <= set(names)
    for i, l in enumerate(cfg["layers"]):
        p = f"l{i}."
        left, right = l["mixer"]["left"], l["mixer"]["right"]
        assert names[p + "mix.left.q"][0] == (left["heads"] * left["dim"], cfg["width"])
        assert names[p + "mix.left.v"][0] == (left["kv_heads"] * left["vdim"], cfg["width"])
        assert names[p + "mix.left.o"][0] == (cfg["width"], left["heads"] * left["vdim"])
        assert names[p + "mix.left.g"][0] == (left["heads"], cfg["width"])
        assert ((p + "mix.left.k.conv") in names) == bool(left["conv"])
        if left["conv"]:
            assert names[p + "mix.left.k.conv"][0] == (left["kv_heads"] * left["dim"], left["conv"])
        assert names[p + "mix.right.lower"][0] == (right["heads"] * right["dim"],)
        assert names[p + "mix.right.norm"][0] == (right["vdim"],)
        assert names[p + "rg1.b"][0] == (cfg["width"],)
        assert ((p + "mlp.up") in names) == (l["mlp"] is not None) == ((p + "rg2") in names)


def test_config_refusals():
    base = RC.CASES["p"]
    for path, value in ((("layers", 0, "type"), "serial"), (("layers", 0, "mlp", "kind"), "routed"),
                        (("layers", 1, "mixer", "left", "kv_heads"), 3), (("layers", 0, "mixer", "left", "rot", "dims"), 66),
                        (("layers", 0, "mixer", "left", "rot", "dims"), 7), (("norm", "eps"), 0), (("vocab",), "many"),
                        (("layers", 0, "mixer", "right", "heads"), 0)):
        cfg = copy.deepcopy(base)
        node = cfg
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError):
            parse_config(cfg)
    for missing in ("width", "embedding", "layers", "norm"):
        cfg = copy.deepcopy(base)
        del cfg[missing]
        with pytest.raises(ConfigError):
            parse_config(cfg)


def test_composite_needs_get_pages_state_and_views():
    pages = PagedKVNeed(2, 16, None, 24)
    need = CompositeNeed({"first": CompositeNeed({"pages": pages, "tails": StateNeed({"qkv": ((2, 10), None)})}),
                          "second": StateNeed({"S": ((3, 4, 5), torch.float32)})})
    cm = CacheManager({0: need, 1: need, 2: PagedKVNeed(2, 16)}, n_pages=6, page_size=16, n_slots=2)
    assert len(cm.groups) == 2                                   # values of 24 and values of 16 do not share pages
    cm.make_storage(torch.bfloat16, "cpu")
    v = cm.view(1)
    assert v["first"]["pages"].k.shape == (6, 2, 16, 16) and v["first"]["pages"].v.shape == (6, 2, 16, 24)
    assert v["first"]["tails"]["qkv"].shape == (2, 2, 10) and v["first"]["tails"]["qkv"].dtype == torch.bfloat16
    assert v["second"]["S"].shape == (2, 3, 4, 5) and v["second"]["S"].dtype == torch.float32
    assert cm.view(0)["first"]["pages"].group == v["first"]["pages"].group != cm.view(2).group
    # a slot that is used again starts from zeros
    cm.admit("a")
    slot = cm.slot("a")
    v["second"]["S"][slot] = 7.0
    v["first"]["tails"]["qkv"][slot] = 3.0
    cm.reserve("a", 20), cm.advance("a", 20)
    cm.release("a")
    cm.admit("b")
    assert cm.slot("b") == slot
    assert float(v["second"]["S"][slot].abs().sum()) == 0.0 and float(v["first"]["tails"]["qkv"][slot].abs().sum()) == 0.0
    cm.check_invariants()


def test_plain_recurrence_and_filter_carry_over_cuts():
    g = torch.Generator().manual_seed(3)
    T, Hh, d, dv = 23, 2, 5, 7
    q, v = torch.randn(T, Hh, d, generator=g, dtype=pr.F), torch.randn(T, Hh, dv, generator=g, dtype=pr.F)
    f = torch.rand(T, Hh, d, generator=g, dtype=pr.F)
    whole, S = pr.gated_recurrence(q, f, v)
    a, Sa = pr.gated_recurrence(q[:9], f[:9], v[:9])
    b, Sb = pr.gated_recurrence(q[9:], f[9:], v[9:], Sa)
    assert torch.allclose(torch.cat([a, b]), whole) and torch.allclose(Sb, S)
    # a forget gate of one keeps the state and writes nothing; of zero, the state is the last value alone
    o1, S1 = pr.gated_recurrence(q[:1], torch.ones(1, Hh, d, dtype=pr.F), v[:1], S)
    assert torch.equal(S1, S)
    _, S0 = pr.gated_recurrence(q[:1], torch.zeros(1, Hh, d, dtype=pr.F), v[:1], S)
    assert torch.allclose(S0, v[0][:, None, :].expand(Hh, d, dv))
    u, w = torch.randn(T, 6, generator=g, dtype=pr.F), torch.randn(6, 3, generator=g, dtype=pr.F)
    y = pr.short_filter(u, w)
    assert torch.allclose(y[0], w[:, 2] * u[0]) and torch.allclose(y[5], w[:, 0] * u[3] + w[:, 1] * u[4] + w[:, 2] * u[5])


def test_plain_rotation_keeps_norms_and_relative_angles():
    g = torch.Generator().manual_seed(4)
    x = torch.randn(9, 2, 12, generator=g, dtype=pr.F)
    y = pr.rotate_pairs(x, 8, 100.0)
    assert torch.equal(y[..., 8:], x[..., 8:]) and torch.allclose(y[0], x[0])
    assert torch.allclose((y[..., :8] ** 2).sum(-1), (x[..., :8] ** 2).sum(-1))
    # the product of a rotated query and key depends on the distance only
    q, k = x[0:1].expand(9, 2, 12).clone(), x[1:2].expand(9, 2, 12).clone()
    rq, rk = pr.rotate_pairs(q, 8, 100.0), pr.rotate_pairs(k, 8, 100.0)
    assert torch.allclose((rq[5] * rk[3]).sum(-1), (rq[7] * rk[5]).sum(-1), atol=1e-5)
