"""The kernels behind Ruvenex's parts, each alone against the plain implementation's function for the same
mechanism (float64), in float and bfloat16 storage, over segments of unequal length with state carried between steps."""
import numpy as np
import pytest
import torch

import plain_ruvenex as pr
from infer_b200 import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class _Step:
    """What a kernel reads of a step: segments of the given lengths, packed, at the given start positions and slots."""

    def __init__(self, lens, pos0, slots):
        seg = np.concatenate([[0], np.cumsum(lens)])
        i32 = lambda a: torch.tensor(np.asarray(a), dtype=torch.int32, device=DEV)
        self.seg_start, self.seg_slot = i32(seg), i32(slots)
        self.token_seg = i32(np.concatenate([np.full(n, s) for s, n in enumerate(lens)]))
        self.positions = i32(np.concatenate([np.arange(p, p + n) for p, n in zip(pos0, lens)]))
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.lens, self.pos0, self.slots = list(lens), list(pos0), list(slots)


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("taps", [2, 3, 5])
def test_short_filter_with_tails_over_steps(dtype, taps):
    g = torch.Generator().manual_seed(taps)
    C, slots = 20, 3
    w = torch.randn(C, taps, generator=g)
    seqs = {0: torch.randn(40, C, generator=g).to(dtype).double(), 2: torch.randn(9, C, generator=g).to(dtype).double()}
    ref = {s: pr.short_filter(u, w) for s, u in seqs.items()}
    tails = torch.zeros(slots, taps - 1, C, dtype=dtype, device=DEV)
    at = {0: 0, 2: 0}
    # portions down to one and two tokens, shorter than the filter
    for lens in ([1, 2], [2, 1], [17, 3], [1, 1], [19, 2]):
        step = _Step(lens, [at[0], at[2]], [0, 2])
        rows = torch.cat([seqs[0][at[0]:at[0] + lens[0]], seqs[2][at[2]:at[2] + lens[1]]]).to(dtype).to(DEV)
        pad = torch.cat([torch.full((rows.shape[0], 3), 9.0, dtype=dtype, device=DEV), rows], dim=1).contiguous()   # columns before
        y = ops.short_filter(pad, 3, w.to(DEV), tails, step.token_seg, step.seg_start, step.seg_slot).double().cpu()
        ops.filter_tail_update(pad, 3, tails, step.seg_start, step.seg_slot)
        want = torch.cat([ref[0][at[0]:at[0] + lens[0]], ref[2][at[2]:at[2] + lens[1]]])
        assert torch.allclose(y, want, **_tol(dtype))
        at[0] += lens[0]
        at[2] += lens[1]
    assert float(tails[1].abs().sum()) == 0.0                    # a slot that no segment names stays untouched
    assert torch.equal(tails[0].double().cpu(), seqs[0][at[0] - (taps - 1):at[0]])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("sizes", [(4, 2, 32, 32, 16), (3, 1, 16, 24, 16), (2, 2, 96, 40, 50), (5, 5, 8, 8, 0), (2, 1, 12, 10, 4), (1, 1, 256, 128, 256), (3, 1, 7, 5, 4)])
def test_prepare_rotates_normalises_and_fills_the_pages(dtype, sizes):
    from infer_b200.parts.rotary import pair_rotation_tables
    H, G, d, dv, n_rot = sizes
    g = torch.Generator().manual_seed(d)
    lens, pos0 = [21, 1, 6], [13, 40, 0]
    step = _Step(lens, pos0, [0, 1, 2])
    T, C = sum(lens), (H + G) * d + G * dv
    rows = torch.randn(T, C + 8, generator=g).to(dtype)
    taps, eps = 3, 1e-5
    fw = torch.randn(C, taps, generator=g)
    tails_cpu = torch.randn(3, taps - 1, C, generator=g).to(dtype)
    tails_cpu[2] = 0
    n_pages, ps = 12, 16
    table = torch.tensor([[3, 7, 1, -1], [5, 0, 2, 9], [4, -1, -1, -1]], dtype=torch.int32, device=DEV)
    k_cache = torch.full((n_pages, G, ps, d), float("nan"), dtype=dtype, device=DEV)
    v_cache = torch.full((n_pages, G, ps, dv), float("nan"), dtype=dtype, device=DEV)
    cos = sin = None
    if n_rot:
        cos, sin = (t.to(DEV) for t in pair_rotation_tables(n_rot, 777.0, 64))
    q = ops.qkv_prepare(rows.to(DEV), fw.t().contiguous().to(DEV), tails_cpu.to(DEV), cos, sin, n_rot, True, eps, step, table, k_cache, v_cache,
                        H, G, d, dv)
    assert int(step.status.item()) == 0
    r0 = 0
    for s, (n, p0) in enumerate(zip(lens, pos0)):
        u = torch.cat([tails_cpu[s].double(), rows[r0:r0 + n, :C].double()])
        y = pr.short_filter(u, fw)[taps - 1:]                     # the tail stands for what came before
        pos = torch.arange(p0, p0 + n)
        qs, ks, vs = y[:, :H * d].view(n, H, d), y[:, H * d:(H + G) * d].view(n, G, d), y[:, (H + G) * d:].view(n, G, dv)
        if n_rot:
            qs, ks = pr.rotate_pairs(qs, n_rot, 777.0, pos), pr.rotate_pairs(ks, n_rot, 777.0, pos)
        vs = pr.rms(vs, eps)
        assert torch.allclose(q[r0:r0 + n].double().cpu().view(n, H, d), qs, **_tol(dtype))
        for i in range(n):
            page, off = int(table[s, (p0 + i) // ps]), (p0 + i) % ps
            assert torch.allclose(k_cache[page, :, off].double().cpu(), ks[i], **_tol(dtype))
            assert torch.allclose(v_cache[page, :, off].double().cpu(), vs[i], **_tol(dtype))
        r0 += n
    assert int(torch.isnan(k_cache.float()).logical_not().sum()) == T * G * d      # nothing else was written


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("sizes", [(2, 16, 48), (1, 40, 20), (3, 8, 8), (2, 64, 64), (1, 128, 128), (4, 12, 12), (1, 30, 500)])
def test_gated_recurrence_over_steps_and_slots(out_dtype, sizes):
    Hh, d, dv = sizes
    g = torch.Generator().manual_seed(d * dv)
    slots, eps = 4, 1e-5
    n = {1: 50, 3: 19}
    ld = 2 * Hh * d + Hh * dv + 4
    proj = {s: torch.randn(t, ld, generator=g) for s, t in n.items()}
    lower = torch.rand(Hh * d, generator=g) * 0.95
    lower[0] = 0.0
    nw = 1.0 + 0.2 * torch.randn(dv, generator=g)
    ref = {}
    for s, pj in proj.items():
        pj = pj.double()
        q = torch.nn.functional.silu(pj[:, 2:2 + Hh * d]).view(-1, Hh, d)
        f = (lower.double() + (1 - lower.double()) * torch.sigmoid(pj[:, 2 + Hh * d:2 + 2 * Hh * d])).view(-1, Hh, d)
        v = pj[:, 4 + 2 * Hh * d:].view(-1, Hh, dv)
        o, S = pr.gated_recurrence(q, f, v)
        ref[s] = ((pr.rms(o, eps) * nw.double()).reshape(-1, Hh * dv), S)
    state = torch.zeros(slots, Hh, d, dv, device=DEV)
    state[0] = 5.0
    at = {1: 0, 3: 0}
    for lens in ([1, 1], [2, 3], [30, 1], [1, 2], [16, 12]):
        step = _Step(lens, [at[1], at[3]], [1, 3])
        rows = torch.cat([proj[1][at[1]:at[1] + lens[0]], proj[3][at[3]:at[3] + lens[1]]]).to(DEV).contiguous()
        # the longest segment chooses the form: one CTA per head, or a head's columns spread over CTAs
        o = ops.gated_recurrence(rows, 2, 2 + Hh * d, 4 + 2 * Hh * d, lower.to(DEV), nw.to(DEV), eps, state, step.seg_start,
                                 step.seg_slot, Hh, d, dv, out_dtype, True, max(lens)).double().cpu()
        want = torch.cat([ref[1][0][at[1]:at[1] + lens[0]], ref[3][0][at[3]:at[3] + lens[1]]])
        assert torch.allclose(o, want, **(dict(rtol=2e-2, atol=2e-2) if out_dtype == torch.bfloat16 else dict(rtol=2e-4, atol=2e-5)))
        at[1] += lens[0]
        at[3] += lens[1]
    assert torch.allclose(state[1].double().cpu(), ref[1][1], rtol=1e-4, atol=1e-5)
    assert torch.allclose(state[3].double().cpu(), ref[3][1], rtol=1e-4, atol=1e-5)
    assert float((state[0] - 5.0).abs().sum()) == 0.0 and float(state[2].abs().sum()) == 0.0
    # a run that must not write leaves the state alone
    before = state.clone()
    step = _Step([3], [at[1]], [1])
    ops.gated_recurrence(proj[1][:3].to(DEV).contiguous(), 2, 2 + Hh * d, 4 + 2 * Hh * d, lower.to(DEV), nw.to(DEV), eps, state,
                         step.seg_start, step.seg_slot, Hh, d, dv, out_dtype, write_state=False)
    assert torch.equal(state, before)


@pytest.mark.parametrize("sizes", [(2, 16, 48), (1, 40, 20), (2, 64, 128), (1, 128, 128)])
def test_both_forms_of_the_recurrence_give_the_same_bits(sizes):
    Hh, d, dv = sizes
    g = torch.Generator().manual_seed(11)
    lens = [37, 1, 9]
    step = _Step(lens, [0, 5, 3], [2, 0, 1])
    ld = 2 * Hh * d + Hh * dv
    proj = torch.randn(sum(lens), ld, generator=g).to(DEV)
    lower, nw = (torch.rand(Hh * d, generator=g) * 0.9).to(DEV), (1.0 + 0.1 * torch.randn(dv, generator=g)).to(DEV)
    state0 = torch.randn(3, Hh, d, dv, generator=g).to(DEV)
    outs, states = [], []
    for max_len in (1, max(lens)):
        st = state0.clone()
        outs.append(ops.gated_recurrence(proj.clone(), 0, Hh * d, 2 * Hh * d, lower, nw, 1e-6, st, step.seg_start, step.seg_slot,
                                         Hh, d, dv, torch.float32, True, max_len))
        states.append(st)
    assert torch.equal(outs[0], outs[1]) and torch.equal(states[0], states[1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_attention_with_values_of_another_size_and_a_far_key(dtype):
    g = torch.Generator().manual_seed(5)
    H, G, d, dv, ps = 6, 3, 16, 40, 16
    n = 300
    q = torch.randn(n, H, d, generator=g).to(dtype)
    k = torch.randn(n, G, d, generator=g).to(dtype)
    v = torch.randn(n, G, dv, generator=g).to(dtype)
    # one key far back answers the last queries: its score stands out among hundreds
    k[17] = (q[-1, 0::2] * 2.0).to(dtype)
    pages = torch.randperm(40, generator=g)[: -(-n // ps)]
    k_cache = torch.full((40, G, ps, d), float("nan"), dtype=dtype)
    v_cache = torch.full((40, G, ps, dv), float("nan"), dtype=dtype)
    for i in range(n):
        k_cache[pages[i // ps], :, i % ps], v_cache[pages[i // ps], :, i % ps] = k[i], v[i]
    lo = n - 9
    step = _Step([9], [lo], [0])
    table = pages[None].to(torch.int32).to(DEV)
    out = ops.attention_plain(q[lo:].reshape(9, H * d).to(DEV).contiguous(), k_cache.to(DEV), v_cache.to(DEV), table,
                              step.token_seg, step.positions, H, G, d, None, 0.31, step.status, dv)
    ref = pr.causal_attention(q.double(), k.double(), v.double(), 0.31)[lo:]
    assert int(step.status.item()) == 0
    assert torch.allclose(out.double().cpu().view(9, H, dv), ref, **_tol(dtype))
    w = torch.softmax((q[-1, 0].double() @ k[:, 0].double().T) * 0.31, dim=-1)
    assert float(w[17]) > 0.5                                    # the far key does carry the result


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_elementwise_pieces(dtype):
    g = torch.Generator().manual_seed(6)
    x = (torch.randn(37, 50, generator=g) * 3).to(dtype)
    assert torch.allclose(ops.gelu_tanh(x.to(DEV)).double().cpu(), pr.gelu_tanh(x.double()), **_tol(dtype))
    T, H, dv = 11, 3, 10
    ctx = torch.randn(T, H * dv, generator=g).to(dtype)
    rows = torch.randn(T, 7 + H, generator=g).to(dtype)
    got = ops.head_gate(ctx.to(DEV).clone(), rows.to(DEV), 7, H, dv).double().cpu()
    want = (ctx.double().view(T, H, dv) * torch.sigmoid(rows[:, 7:].double())[:, :, None]).view(T, H * dv)
    assert torch.allclose(got, want, **_tol(dtype))
    W = 24
    xs, p, q, r = (torch.randn(T, W, generator=g) for _ in range(4))
    gates = torch.randn(T, 2 * W, generator=g)
    dev = lambda t: t.to(DEV).clone()
    full = ops.gated_sum(dev(xs), dev(gates), dev(p), 0.7, dev(q), 1.3, dev(r)).cpu()
    want = xs + torch.sigmoid(gates[:, :W]) * (0.7 * p + 1.3 * q) + torch.sigmoid(gates[:, W:]) * r
    assert torch.allclose(full, want, rtol=1e-5, atol=1e-5)
    one = ops.gated_sum(dev(xs), dev(gates[:, :W].contiguous()), dev(p), 2.0).cpu()
    assert torch.allclose(one, xs + torch.sigmoid(gates[:, :W]) * 2.0 * p, rtol=1e-5, atol=1e-5)
    bare = ops.gated_sum(dev(xs), None, dev(p), 1.0, dev(q), 1.0).cpu()
    assert torch.allclose(bare, xs + p + q, rtol=1e-6, atol=1e-6)
