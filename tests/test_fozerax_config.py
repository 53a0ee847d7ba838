"""Fozerax without a GPU: configuration, tensor names, sizes that only a checkpoint states, cache needs, and the plain
implementation's own consistency."""
import copy
import json
import math

import pytest
import torch

import fozerax_cases as FC
import infer_b200.models  # noqa: F401  (registers the architectures)
import infer_b200.parts  # noqa: F401
import plain_fozerax as pf
from infer_b200.config import parse_config
from infer_b200.config.registry import ConfigError
from infer_b200.parts.attention import distance_bias_table, log_bucket
from infer_b200.parts.base import CompositeNeed, PagedKVNeed, StateNeed, part_class
from infer_b200.weights.binder import WeightsError, check_weights, expected_tensors, shape_fits


@pytest.mark.parametrize("name", sorted(FC.CASES))
def test_config_round_trip_and_tensor_names(name):
    cfg = FC.CASES[name]
    arch, typed = parse_config(cfg)
    assert arch.name == "Fozerax"
    assert arch.parse(arch.to_dict(typed)) == typed
    names = expected_tensors(arch.to_spec(typed))
    W = cfg["width"]
    assert {"embed", "embed.norm", "final.norm", "head"} <= set(names)
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.", l["mixer"]
        assert names[p + "norm1"][0] == (W,)
        assert ((p + "norm2") in names) == (l["mlp"] is not None)
        if l["type"] == "gla":
            assert names[p + "mix.q"][0] == names[p + "mix.k"][0] == (m["heads"] * m["dim"], W)
            assert names[p + "mix.v"][0] == names[p + "mix.g"][0] == (m["heads"] * m["vdim"], W)
            assert names[p + "mix.a1"][0] == (m["rank"], W) and names[p + "mix.a2"][0] == (m["heads"] * m["dim"], m["rank"])
            assert names[p + "mix.a2.b"][0] == (m["heads"] * m["dim"],) and names[p + "mix.norm"][0] == (m["vdim"],)
        else:
            a, b = m["left"], m["right"]
            assert names[p + "mix.left.q"][0] == (a["heads"] * a["dim"], W) and names[p + "mix.left.q.b"][0] == (a["heads"] * a["dim"],)
            assert names[p + "mix.left.k.norm"][0] == (a["kv_heads"] * a["dim"],)
            assert names[p + "mix.left.v"][0] == (a["kv_heads"] * a["vdim"], W)
            assert names[p + "mix.left.rel"][0] == (a["buckets"], a["heads"]) and names[p + "mix.left.sink"][0] == (a["heads"],)
            assert names[p + "mix.left.out"][0] == names[p + "mix.right.out"][0] == (W,)
            assert names[p + "mix.right.q"][0] == (b["kv_heads"] * b["dim"], W) and names[p + "mix.right.v"][0] == (b["heads"] * b["vdim"], W)
            assert ((p + "mix.right.v.conv") in names) == bool(b["conv"])
            if b["conv"]:
                assert names[p + "mix.right.v.conv"][0] == (b["heads"] * b["vdim"], b["conv"])
            assert names[p + "mix.right.b"][0] == names[p + "mix.right.a"][0] == (b["heads"], W)
            assert names[p + "mix.right.A_log"][0] == names[p + "mix.right.dt_bias"][0] == (b["heads"],)
        if l["mlp"] and l["mlp"]["kind"] == "moe":
            r = l["mlp"]["router"]
            assert names[p + "mlp.router"][0] == (r["experts"], W)
            assert names[p + f"mlp.e{r['experts'] - 1}.down"][0] == (W, l["mlp"]["expert"]["ff"])
            assert ((p + "mlp.shared.up") in names) == (l["mlp"]["shared"] is not None)
        elif l["mlp"]:
            assert names[p + "mlp.gate"][0] == names[p + "mlp.up"][0] == (l["mlp"]["ff"], W)


def test_config_refusals():
    base = FC.CASES["a"]
    for path, value in ((("layers", 0, "type"), "serial"), (("layers", 0, "mlp", "kind"), "routed"),
                        (("layers", 1, "mixer", "left", "kv_heads"), 3), (("layers", 1, "mixer", "right", "kv_heads"), 3),
                        (("layers", 0, "mixer", "tau"), 0), (("norm", "eps"), 0), (("vocab",), "many"),
                        (("layers", 1, "mlp", "router", "top"), 5), (("layers", 1, "mlp", "router", "groups", "keep"), 4),
                        (("layers", 1, "mlp", "expert", "limit"), -1.0), (("layers", 1, "mixer", "left", "mask", "size"), 0)):
        cfg = copy.deepcopy(base)
        node = cfg
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError):
            parse_config(cfg)
    cfg = copy.deepcopy(base)
    del cfg["layers"][1]["mixer"]["left"]["scale"]
    with pytest.raises(ConfigError, match="scale"):
        parse_config(cfg)


def test_sizes_that_only_the_checkpoint_states():
    """Without ``rank`` and ``buckets`` in the configuration the tensors' own shapes are taken; other sizes still bind."""
    cfg = copy.deepcopy(FC.CASES["a"])
    W = FC.make_weights(cfg, 3)
    del cfg["layers"][0]["mixer"]["rank"], cfg["layers"][1]["mixer"]["left"]["buckets"]
    arch, typed = parse_config(cfg)
    assert "rank" not in json.dumps(arch.to_dict(typed)) and "buckets" not in json.dumps(arch.to_dict(typed))
    spec = arch.to_spec(typed)
    names = expected_tensors(spec)
    assert names["l0.mix.a1"][0] == (-1, 64) and names["l1.mix.left.rel"][0] == (-1, 4)
    check_weights(W, spec)
    assert shape_fits((-1, 4), (9, 4)) and not shape_fits((-1, 4), (9, 5)) and not shape_fits((3,), (3, 1))
    bad = dict(W)
    bad["l0.mix.a2"] = torch.zeros(32, 5, 2)
    with pytest.raises(WeightsError, match="l0.mix.a2"):
        check_weights(bad, spec)
    from infer_b200.weights import random_weights
    with pytest.raises(ValueError, match="only a checkpoint states"):
        random_weights(spec, 1)


def test_cache_needs_windows_and_slots_used_again():
    """What the two kinds of layer ask of the cache manager: pages behind a window beside two state tensors, and a
    state matrix alone. A layer's pages go back behind its window; a slot that is used again starts from zeros."""
    from infer_b200.cache.manager import CacheManager
    spec = FC.spec_of(FC.CASES["a"])
    gla, par = spec.layers[0].part("mixer"), spec.layers[1].part("mixer")
    assert gla.kind == "decayed_linear_attention" and par.kind == "side_by_side"
    assert par["first"].kind == "attention" and par["second"].kind == "gated_delta_rule"
    assert par["first"]["window"] == 24 and par["first_scale"] == par["second_scale"] == 0.5
    left = PagedKVNeed(2, 16, 24, 24)
    right = StateNeed({"S": ((2, 16, 32), torch.float32), "tails": ((2, 2 * 16 + 2 * 32), torch.float32)})
    needs = {0: StateNeed({"S": ((2, 16, 32), torch.float32)}), 1: CompositeNeed({"first": left, "second": right})}
    cm = CacheManager(needs, n_pages=6, page_size=16, n_slots=2)
    cm.make_storage(torch.bfloat16, "cpu")
    v = cm.view(1)
    assert v["first"].k.shape == (6, 2, 16, 16) and v["first"].v.shape == (6, 2, 16, 24) and v["first"].window == 24
    assert v["second"]["S"].dtype == v["second"]["tails"].dtype == torch.float32 and cm.view(0)["S"].shape == (2, 2, 16, 32)
    cm.admit("x")
    slot = cm.slot("x")
    v["second"]["S"][slot] = 7.0
    v["second"]["tails"][slot] = 3.0
    cm.view(0)["S"][slot] = 5.0
    assert cm.reserve("x", 70)
    cm.advance("x", 70)
    assert cm.block_table("x", 0)[:2] == [-1, -1] and cm.pages_in_use() == [3]       # positions 47 .. 69 are still read
    cm.release("x")
    cm.admit("y")
    assert cm.slot("y") == slot
    assert float(v["second"]["S"][slot].abs().sum()) == float(v["second"]["tails"][slot].abs().sum()) == float(cm.view(0)["S"][slot].abs().sum()) == 0.0
    cm.check_invariants()


def test_bucket_function_and_bias_table():
    B, D = 24, 90.0
    rows = [log_bucket(n, B, D) for n in range(200)]
    assert rows[:12] == list(range(12)) and rows[12] == 12 and max(rows) == B - 1 and rows == sorted(rows)
    assert all(log_bucket(n, B, D) == pf.distance_bucket(n, B, D) for n in range(300))
    assert rows[89] < B - 1 or rows[90] == B - 1
    assert log_bucket(int(D), B, D) == B - 1
    assert [log_bucket(n, 7, 20.0) for n in range(4)] == [0, 1, 2, 3]                      # an odd table: B // 2 single rows
    rel = torch.arange(B * 2, dtype=torch.float32).view(B, 2)
    t = distance_bias_table(rel, D, 50)
    assert t.shape == (50, 2) and torch.equal(t[5], rel[5]) and torch.equal(t[49], rel[log_bucket(49, B, D)])
    t = distance_bias_table(rel, D, None)
    assert torch.equal(t[-1], rel[B - 1]) and log_bucket(t.shape[0] - 2, B, D) < B - 1       # the last row stands for all beyond
    with pytest.raises(ValueError):
        distance_bias_table(rel, 12.0, None)


def test_plain_scans_can_be_cut_anywhere():
    g = torch.Generator().manual_seed(0)
    T, d, dv = 23, 6, 5
    q, k, v = (torch.randn(T, n, generator=g, dtype=torch.float64) for n in (d, d, dv))
    decay = torch.rand(T, d, generator=g, dtype=torch.float64)
    gate, beta = torch.rand(T, generator=g, dtype=torch.float64), torch.rand(T, generator=g, dtype=torch.float64)
    whole, S = pf.decayed_state_scan(q, k, v, decay)
    a, Sa = pf.decayed_state_scan(q[:9], k[:9], v[:9], decay[:9])
    b, Sb = pf.decayed_state_scan(q[9:], k[9:], v[9:], decay[9:], Sa)
    assert torch.allclose(torch.cat([a, b]), whole) and torch.allclose(Sb, S)
    whole, S = pf.delta_rule_scan(q, k, v, gate, beta)
    a, Sa = pf.delta_rule_scan(q[:2], k[:2], v[:2], gate[:2], beta[:2])
    b, Sb = pf.delta_rule_scan(q[2:], k[2:], v[2:], gate[2:], beta[2:], Sa)
    assert torch.allclose(torch.cat([a, b]), whole) and torch.allclose(Sb, S)
    # a write strength of one with a unit key replaces what the state returned for that key
    kk = pf.unit(k)
    _, S1 = pf.delta_rule_scan(q[:1], kk[:1], v[:1], torch.ones(1, dtype=torch.float64), torch.ones(1, dtype=torch.float64), S)
    assert torch.allclose(S1.T @ kk[0], v[0], atol=1e-4)
    # decays of one and keys of zero keep the state
    o, S2 = pf.decayed_state_scan(q[:3], torch.zeros(3, d, dtype=torch.float64), v[:3], torch.ones(3, d, dtype=torch.float64), S)
    assert torch.equal(S2, S)


def test_plain_router_keeps_to_its_groups():
    g = torch.Generator().manual_seed(1)
    mlp = FC.CASES["b"]["layers"][3]["mlp"]                      # nine experts in three groups, one kept, three chosen
    W = {"r.router": torch.randn(9, 12, generator=g, dtype=torch.float64)}
    h = torch.randn(50, 12, generator=g, dtype=torch.float64)
    chosen, w = pf.route(h, mlp, W, "r.")
    s = torch.softmax(h @ W["r.router"].T, dim=-1)
    best_group = s.view(50, 3, 3).max(dim=-1).values.argmax(dim=-1)
    assert torch.equal(chosen // 3, best_group[:, None].expand(-1, 3))
    assert torch.allclose(w.sum(dim=-1), torch.ones(50, dtype=torch.float64)) and (w > 0).all()
    assert torch.allclose(w, s.gather(1, chosen) / s.gather(1, chosen).sum(dim=-1, keepdim=True))


def test_plain_window_and_sink():
    """A query sees itself and window - 1 tokens before it; the sink takes weight but gives nothing."""
    cfg = copy.deepcopy(FC.CASES["a"])
    m = cfg["layers"][1]["mixer"]["left"]
    W = {k: v.double() for k, v in FC.make_weights(cfg, 5).items()}
    p = "l1.mix.left."
    g = torch.Generator().manual_seed(2)
    h = torch.randn(40, 64, generator=g, dtype=torch.float64)
    base = pf.windowed_attention(h, m, W, p, 1e-5)
    h2 = h.clone()
    h2[3] += 1.0                                                  # position 3 is seen by 3 .. 26 and by no later one
    moved = (pf.windowed_attention(h2, m, W, p, 1e-5) - base).abs().sum(dim=-1) > 1e-9
    assert moved[3:27].all() and not moved[27:].any() and not moved[:3].any()
    W2 = dict(W)
    W2[p + "sink"] = W[p + "sink"] + 50.0                          # a sink that takes all the weight leaves only the bias of o
    assert pf.windowed_attention(h, m, W2, p, 1e-5).abs().max() < 1e-9
