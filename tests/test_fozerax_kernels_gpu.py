"""The kernels behind Fozerax's parts, each alone against the plain implementation's function for the same
mechanism (float64), in float and bfloat16 storage, over segments of unequal length with state carried between steps."""
import math

import numpy as np
import pytest
import torch

import plain_fozerax as pf
from infer_b200 import ops
from test_ruvenex_kernels_gpu import _Step

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _tol(dtype):
    return dict(rtol=2e-2, atol=2e-2) if dtype == torch.bfloat16 else dict(rtol=2e-5, atol=2e-5)


@pytest.mark.parametrize("width", [36, 192, 1000])
def test_norm_add_and_its_copy(width):
    g = torch.Generator().manual_seed(width)
    x, y = torch.randn(7, width, generator=g), 5.0 * torch.randn(7, width, generator=g)
    w = torch.randn(width, generator=g)
    want = x.double() + pf.rms_weighted(y.double(), w, 1e-5)
    out, copy = ops.norm_add(x.to(DEV), y.to(DEV), w.to(DEV), 1e-5, torch.bfloat16)
    assert torch.allclose(out.double().cpu(), want, rtol=1e-5, atol=1e-5)
    assert torch.equal(copy.cpu(), out.cpu().to(torch.bfloat16))
    alone, none = ops.norm_add(None, y.to(DEV), w.to(DEV), 1e-5, torch.float32)
    assert none is None and torch.allclose(alone.double().cpu(), pf.rms_weighted(y.double(), w, 1e-5), rtol=1e-5, atol=1e-5)
    assert torch.equal(ops.cast_rows(out, torch.bfloat16).cpu(), copy.cpu())


@pytest.mark.parametrize("width", [36, 200])
def test_two_normalised_sides_and_the_layer_norm_in_one_pass(width):
    g = torch.Generator().manual_seed(width)
    a, b, x = (torch.randn(5, width, generator=g) * s for s in (3.0, 0.1, 1.0))
    wa, wb, wo = (torch.randn(width, generator=g) for _ in range(3))
    m = 0.5 * pf.rms_weighted(a.double(), wa, 1e-5) + 0.25 * pf.rms_weighted(b.double(), wb, 1e-5)
    got, _ = ops.dual_norm_sum(a.to(DEV), wa.to(DEV), 0.5, b.to(DEV), wb.to(DEV), 0.25, 1e-5)
    assert torch.allclose(got.double().cpu(), m, rtol=1e-5, atol=1e-5)
    out, copy = ops.dual_norm_sum(a.to(DEV), wa.to(DEV), 0.5, b.to(DEV), wb.to(DEV), 0.25, 1e-5, x.to(DEV), wo.to(DEV), 3e-6, torch.bfloat16)
    assert torch.allclose(out.double().cpu(), x.double() + pf.rms_weighted(m, wo, 3e-6), rtol=1e-5, atol=1e-5)
    assert torch.equal(copy.cpu(), out.cpu().to(torch.bfloat16))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("sizes", [(3, 5, 7, 2), (3, 16, 24, 8)], ids=["odd", "by-eights"])
def test_gated_activations(dtype, sizes):
    g = torch.Generator().manual_seed(3)
    T = 9
    E, ff, fs, c0 = sizes
    width = E * ff + fs
    rows = (3.0 * torch.randn(T, c0 + 2 * width, generator=g)).to(dtype)
    gate, up = rows[:, c0:c0 + width].double(), rows[:, c0 + width:].double()
    got = ops.glu_act(rows.to(DEV), c0, c0 + width, width, "gelu_tanh").double().cpu()
    assert torch.allclose(got, pf.gelu_tanh(gate) * up, **_tol(dtype))
    scale = torch.rand(T, E, generator=g)
    scale[:, 1] = 0.0
    lim, lim2 = 1.5, 0.4

    def expert(gv, uv, limit):
        gv, uv = torch.clamp(gv, max=limit), torch.clamp(uv, -limit, limit)
        return gv * torch.sigmoid(pf.EXPERT_SLOPE * gv) * (uv + 1.0)
    want = torch.cat([expert(gate[:, :E * ff], up[:, :E * ff], lim) * scale.double().repeat_interleave(ff, dim=1),
                      expert(gate[:, E * ff:], up[:, E * ff:], lim2)], dim=1)
    got = ops.glu_act(rows.to(DEV), c0, c0 + width, width, "clipped_swish", lim, lim2, pf.EXPERT_SLOPE, scale.to(DEV), ff, E).double().cpu()
    assert torch.allclose(got, want, **_tol(dtype))
    assert float(got[:, ff:2 * ff].abs().sum()) == 0.0


@pytest.mark.parametrize("shape", [(8, 4, 2, 1), (9, 3, 3, 1), (6, 2, 3, 2), (4, 4, 1, 1), (64, 6, 8, 3), (5, 1, 1, 1), (40, 40, 5, 5)])
def test_router(shape):
    E, top, groups, keep = shape
    g = torch.Generator().manual_seed(E)
    logits = 2.0 * torch.randn(33, E, generator=g)
    mlp = {"router": {"experts": E, "top": top, "groups": {"count": groups, "keep": keep}}}
    chosen, w = pf.route(logits.double(), mlp, {"r.router": torch.eye(E, dtype=torch.float64)}, "r.")     # logits = h . I
    want = torch.zeros(33, E, dtype=torch.float64).scatter_(1, chosen, w)
    got, idx = ops.route(logits.to(DEV), top, groups, keep, pf.WEIGHT_SUM_EPS, want_chosen=True)
    assert torch.allclose(got.double().cpu(), want, rtol=1e-5, atol=1e-7)
    assert torch.equal(idx.cpu().long().sort(dim=1).values, chosen.sort(dim=1).values)
    assert torch.allclose(got.sum(dim=1).cpu(), torch.ones(33), atol=1e-5)


def _paged(seqs_k, seqs_v, tables, n_pages, G, d, dv, dtype, ps=16):
    k_cache = torch.full((n_pages, G, ps, d), float("nan"), dtype=dtype)
    v_cache = torch.full((n_pages, G, ps, dv), float("nan"), dtype=dtype)
    for s, (k, v) in enumerate(zip(seqs_k, seqs_v)):
        for p in range(k.shape[0]):
            page = tables[s][p // ps]
            if page >= 0:
                k_cache[page, :, p % ps] = k[p].to(dtype)
                v_cache[page, :, p % ps] = v[p].to(dtype)
    return k_cache, v_cache


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("sizes", [(6, 2, 64, 48), (3, 3, 10, 7), (2, 1, 12, 12), (4, 1, 32, 40)])
def test_row_norms_of_q_and_k_and_the_cache_write(dtype, sizes):
    H, G, d, dv = sizes
    g = torch.Generator().manual_seed(d)
    lens, pos0 = [21, 1, 6], [13, 40, 0]
    step = _Step(lens, pos0, [0, 1, 2])
    T, C = sum(lens), (H + G) * d + G * dv
    rows = torch.randn(T, C + 5, generator=g).to(dtype)
    wq, wk = torch.randn(H * d, generator=g), torch.randn(G * d, generator=g)
    table = torch.tensor([[3, 7, 1, -1], [5, 0, 2, 9], [4, -1, -1, -1]], dtype=torch.int32, device=DEV)
    k_cache = torch.full((12, G, 16, d), float("nan"), dtype=dtype, device=DEV)
    v_cache = torch.full((12, G, 16, dv), float("nan"), dtype=dtype, device=DEV)
    q = ops.rownorm_store(rows.to(DEV), 3, wq.to(DEV), wk.to(DEV), 1e-5, step, table, k_cache, v_cache, H, G, d, dv).double().cpu()
    r = rows.double()[:, 3:]
    assert torch.allclose(q, pf.rms_weighted(r[:, :H * d], wq, 1e-5), **_tol(dtype))
    kn = pf.rms_weighted(r[:, H * d:(H + G) * d], wk, 1e-5).view(T, G, d)
    t = 0
    for s, (n, p0) in enumerate(zip(lens, pos0)):
        for i in range(n):
            page, place = int(table[s, (p0 + i) // 16]), (p0 + i) % 16
            assert torch.allclose(k_cache[page, :, place].double().cpu(), kn[t], **_tol(dtype))
            assert torch.equal(v_cache[page, :, place].cpu(), rows[t, 3 + (H + G) * d:3 + C].view(G, dv))
            t += 1
    assert int(torch.isnan(k_cache).logical_not().sum()) == T * G * d          # nothing else was written
    assert int(step.status.item()) == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("window", [None, 5, 16, 33, 70])
def test_attention_with_distance_bias_window_and_sink(dtype, window):
    """Keys at the window's two edges carry the result: the key at distance window - 1 is made to stand out for one
    head, the key at distance window (just outside) for another, by scaling those keys along the query."""
    from infer_b200.parts.attention import distance_bias_table
    H, G, d, dv, B, D = 4, 2, 16, 24, 12, 40.0
    g = torch.Generator().manual_seed(window or 1)
    n = 150
    q = torch.randn(n, H, d, generator=g).to(dtype).double()
    k = torch.randn(n, G, d, generator=g).to(dtype).double()
    v = torch.randn(n, G, dv, generator=g).to(dtype).double()
    rel, sink = torch.randn(B, H, generator=g), torch.randn(H, generator=g)
    sink[1] = 4.0
    probe = 140
    if window is not None:
        k[probe - (window - 1), 0] = 3.0 * q[probe, 0] / q[probe, 0].norm() * math.sqrt(d)      # just inside, head 0
        k[probe - window, 1] = 3.0 * q[probe, 2] / q[probe, 2].norm() * math.sqrt(d)             # just outside, head 2
        k = k.to(dtype).double()
    scale = 0.3
    want = torch.zeros(n, H, dv, dtype=torch.float64)
    idx = torch.arange(n)
    dist = idx[:, None] - idx[None, :]
    seen = (dist >= 0) & ((dist < window) if window else (dist >= 0))
    bucket = torch.tensor([pf.distance_bucket(i, B, D) for i in range(n)])[dist.clamp(min=0)]
    for h in range(H):
        s = (q[:, h] @ k[:, h // 2].T) * scale + rel.double()[bucket, h]
        s = s.masked_fill(~seen, -math.inf)
        top = torch.maximum(s.max(dim=-1).values, sink.double()[h])
        e = torch.exp(s - top[:, None])
        want[:, h] = (e / (e.sum(dim=-1) + torch.exp(sink.double()[h] - top))[:, None]) @ v[:, h // 2]
    if window is not None:
        w_in = torch.softmax(((q[probe, 0] @ k[:, 0].T) * scale).masked_fill(~seen[probe], -math.inf), dim=-1)
        assert w_in[probe - (window - 1)] > 0.5                  # the test's own premise: the edge key dominates
    table_row = [7, 2, 9, 0, 5, 11, 3, 8, 1, 10]
    kc, vc = _paged([k], [v], [table_row], 12, G, d, dv, dtype)
    table = torch.tensor([table_row], dtype=torch.int32, device=DEV)
    bias = distance_bias_table(rel, D, window).to(DEV)
    rows = list(range(100, n))                                   # a portion in the middle of a request, then nothing
    step_seg = torch.zeros(len(rows), dtype=torch.int32, device=DEV)
    pos = torch.tensor(rows, dtype=torch.int32, device=DEV)
    out = ops.attention_plain(q[rows].reshape(len(rows), H * d).to(dtype).to(DEV).contiguous(), kc.to(DEV), vc.to(DEV), table, step_seg, pos,
                              H, G, d, window, scale, None, dv, bias, sink.to(DEV)).double().cpu().view(len(rows), H, dv)
    assert torch.allclose(out, want[rows], **_tol(dtype))


def _biased_attention(q, k, v, rel, sink, B, D, window, scale):
    """Plain windowed attention of one sequence with a bucketed distance bias and a sink. q [n, H, d], k, v [n, G, .]."""
    n, H = q.shape[:2]
    G = k.shape[1]
    idx = torch.arange(n)
    dist = idx[:, None] - idx[None, :]
    seen = (dist >= 0) & ((dist < window) if window else (dist >= 0))
    bucket = torch.tensor([pf.distance_bucket(i, B, D) for i in range(n)])[dist.clamp(min=0)]
    out = torch.zeros(n, H, v.shape[2], dtype=torch.float64)
    for h in range(H):
        s = (q[:, h] @ k[:, h // (H // G)].T) * scale + rel.double()[bucket, h]
        s = s.masked_fill(~seen, -math.inf)
        top = torch.maximum(s.max(dim=-1).values, sink.double()[h])
        e = torch.exp(s - top[:, None])
        out[:, h] = (e / (e.sum(dim=-1) + torch.exp(sink.double()[h] - top))[:, None]) @ v[:, h // (H // G)]
    return out


@pytest.mark.parametrize("window", [None, 33, 130, 300])
@pytest.mark.parametrize("sizes", [(4, 2, 64), (8, 1, 128)])
def test_tensor_core_attention_with_distance_bias_and_sink(sizes, window):
    """A prompt portion of several query tiles behind a context, beside a one-token segment of another request: the
    portion on the tensor-core kernel, the single token on the plain one, into one result; keys at the window's edges
    stand out for two heads of the portion's last rows."""
    from infer_b200.parts.attention import distance_bias_table
    H, G, d = sizes
    B, D, scale, dtype = 28, 150.0, 0.11, torch.bfloat16
    g = torch.Generator().manual_seed(d + (window or 0))
    n, m = 500, 90                                              # the portion's request; the single token's request
    seqs = []
    for length in (n, m):
        seqs.append([torch.randn(length, hh, d, generator=g).to(dtype).double() for hh in (H, G, G)])
    rel, sink = torch.randn(B, H, generator=g), torch.randn(H, generator=g)
    sink[1] = 5.0
    q, k, v = seqs[0]
    if window is not None:
        for probe in (n - 1, n - 70):
            k[probe - (window - 1), 0] = 4.0 * q[probe, 0] / q[probe, 0].norm() * math.sqrt(d) / (scale * math.sqrt(d)) * 0.3
            k[probe - window, G - 1] = 4.0 * q[probe, H - 1] / q[probe, H - 1].norm() * math.sqrt(d) / (scale * math.sqrt(d)) * 0.3
        seqs[0][1] = k = k.to(dtype).double()
    want = [_biased_attention(*sq, rel, sink, B, D, window, scale) for sq in seqs]
    tables = [list(range(3, 35)), [40, 36, 38, 37, 41, 39]]
    kc, vc = _paged([s_[1] for s_ in seqs], [s_[2] for s_ in seqs], tables, 44, G, d, d, dtype)
    width = 32
    table = torch.full((2, width), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        table[i, :len(t)] = torch.tensor(t, dtype=torch.int32)
    first = 230                                                 # the portion: positions 230 .. 499 (three query tiles, the last ragged)
    step = _Step([n - first, 1], [first, m - 1], [0, 1])
    step.seg_lens, step.seg_pos0 = step.lens, torch.tensor(step.pos0, dtype=torch.int32, device=DEV)
    step.max_q_len, step.max_ctx_len = n - first, n
    rows = torch.cat([q[first:].reshape(n - first, H * d), seqs[1][0][m - 1:].reshape(1, H * d)]).to(dtype).to(DEV).contiguous()
    bias = distance_bias_table(rel, D, window).to(DEV)
    by_head = (bias / scale).t().contiguous()
    before = dict(ops.LAUNCH_KINDS)
    out = ops.attention_window(rows, kc.to(DEV), vc.to(DEV), table.to(DEV), step, H, G, d, d, window, scale, bias, sink.to(DEV), by_head)
    assert out is not None and ops.LAUNCH_KINDS["ib_attention_prefill_tc_biased"] == before.get("ib_attention_prefill_tc_biased", 0) + 1
    assert int(step.status.item()) == 0
    got = out.double().cpu().view(-1, H, d)
    ref = torch.cat([want[0][first:], want[1][m - 1:]])
    assert torch.allclose(got, ref, rtol=3e-2, atol=3e-2)
    assert float((got - ref).pow(2).mean().sqrt()) < 4e-3


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("window", [None, 5, 70, 128, 300])
@pytest.mark.parametrize("sizes", [(6, 2, 64, 48), (3, 3, 10, 7), (16, 1, 128, 128), (4, 2, 24, 40)])
def test_single_tokens_with_their_keys_split_over_ctas(sizes, window, dtype):
    """Decoded tokens at positions around chunk borders (multiples of 128), page borders and the first positions; one
    key at each edge of the window stands out; a longer segment in the same step is left alone."""
    from infer_b200.parts.attention import distance_bias_table
    H, G, d, dv = sizes
    B, D, scale = 12, 40.0, 0.2
    g = torch.Generator().manual_seed(d + (window or 0))
    n = 420
    q = torch.randn(n, H, d, generator=g).to(dtype).double()
    k = torch.randn(n, G, d, generator=g).to(dtype).double()
    v = torch.randn(n, G, dv, generator=g).to(dtype).double()
    rel, sink = torch.randn(B, H, generator=g), torch.randn(H, generator=g)
    probes = [0, 1, 15, 16, 127, 128, 129, 255, 256, 300, 383, 384, 419]
    if window is not None:
        for pr_ in probes:
            if pr_ - window >= 0:
                k[pr_ - (window - 1), 0] += 2.0 * q[pr_, 0] / q[pr_, 0].norm() * math.sqrt(d)
                k[pr_ - window, G - 1] += 2.0 * q[pr_, H - 1] / q[pr_, H - 1].norm() * math.sqrt(d)
        k = k.to(dtype).double()
    want = _biased_attention(q, k, v, rel, sink, B, D, window, scale)
    table_row = list(np.random.default_rng(1).permutation(30))[:27]
    kc, vc = _paged([k], [v], [table_row], 30, G, d, dv, dtype)
    # every probe is a request of its own that shares the pages (one row of the table each), plus one longer segment
    S = len(probes) + 1
    table = torch.tensor([table_row] * S, dtype=torch.int32, device=DEV)
    step = _Step([1] * len(probes) + [3], probes + [200], list(range(S)))
    step.seg_lens, step.max_q_len, step.max_ctx_len = step.lens, 3, n
    rows = torch.cat([q[probes], q[200:203]]).reshape(-1, H * d).to(dtype).to(DEV).contiguous()
    bias = distance_bias_table(rel, D, window).to(DEV)
    out = torch.full((rows.shape[0], H * dv), 7.0, dtype=dtype, device=DEV)
    ops.attention_split(rows, kc.to(DEV), vc.to(DEV), table, step, H, G, d, dv, window, scale, bias, sink.to(DEV), out, single_only=True)
    got = out.double().cpu().view(-1, H, dv)
    assert torch.allclose(got[:len(probes)], want[probes], **_tol(dtype))
    assert float((got[len(probes):] - 7.0).abs().sum()) == 0.0               # the longer segment's rows were left alone
    step.max_q_len = 1
    every = ops.attention_split(rows, kc.to(DEV), vc.to(DEV), table, step, H, G, d, dv, window, scale, bias, sink.to(DEV))
    assert torch.allclose(every.double().cpu().view(-1, H, dv)[len(probes):], want[200:203], **_tol(dtype))
    assert int(step.status.item()) == 0


@pytest.mark.parametrize("sizes", [(2, 16, 4), (1, 40, 3), (3, 128, 16)])
def test_decays_through_a_low_rank(sizes):
    H, d, r = sizes
    g = torch.Generator().manual_seed(d)
    T, C = 11, H * d
    rows = torch.randn(T, 3 + C + r, generator=g)
    up, bias = torch.randn(C, r, generator=g), 2.0 + torch.randn(C, generator=g)
    tau = 7.0
    z = rows[:, 3 + C:].double() @ up.double().T + bias.double()
    want = torch.sigmoid(z) ** (1.0 / tau)
    dev = rows.to(DEV)
    decay = ops.decay_gates(dev, 3, 3 + C, r, up.t().contiguous().to(DEV), bias.to(DEV), tau, d ** -0.5)
    assert torch.allclose(decay.double().cpu(), want, rtol=1e-5, atol=1e-6)
    assert torch.allclose(dev[:, 3:3 + C].double().cpu(), rows[:, 3:3 + C].double() * d ** -0.5, rtol=1e-6, atol=1e-7)
    assert torch.equal(dev[:, :3].cpu(), rows[:, :3]) and torch.equal(dev[:, 3 + C:].cpu(), rows[:, 3 + C:])


# a key size below, at and above each number of state rows a lane keeps; value sizes that are no multiple of four
SCAN_SIZES = [(2, 1, 16, 32), (1, 1, 40, 20), (3, 1, 5, 9), (2, 1, 128, 64), (4, 2, 8, 4), (4, 2, 160, 128), (1, 1, 33, 3), (2, 2, 64, 130)]


def _portions(total):
    """Ways of cutting two requests of these lengths into steps: long portions, portions of two, single tokens."""
    return [[1, 2], [2, 1], [17, 3], [1, 1], [9, 2], [total[0] - 30, total[1] - 9]]


@pytest.mark.parametrize("sizes", SCAN_SIZES)
def test_scan_with_a_decay_per_key_channel(sizes):
    H, _, d, dv = sizes
    g = torch.Generator().manual_seed(d + dv)
    total = [70, 12]
    seqs = {}
    for slot, n in zip((0, 2), total):
        seqs[slot] = dict(q=torch.randn(n, H, d, generator=g), k=torch.randn(n, H, d, generator=g), v=torch.randn(n, H, dv, generator=g),
                          a=0.8 + 0.2 * torch.rand(n, H, d, generator=g))
    ref = {s: torch.stack([pf.decayed_state_scan(x["q"][:, h].double(), x["k"][:, h].double(), x["v"][:, h].double(), x["a"][:, h].double())[0]
                           for h in range(H)], dim=1) for s, x in seqs.items()}
    state = torch.zeros(3, H, d, dv, device=DEV)
    state[1] = 9.0
    at = {0: 0, 2: 0}
    for lens in _portions(total):
        step = _Step(lens, [at[0], at[2]], [0, 2])
        cut = lambda name: torch.cat([seqs[0][name][at[0]:at[0] + lens[0]], seqs[2][name][at[2]:at[2] + lens[1]]])
        T = sum(lens)
        rows = torch.cat([torch.full((T, 1), 7.0), cut("q").reshape(T, -1), cut("k").reshape(T, -1), cut("v").reshape(T, -1)], dim=1).contiguous().to(DEV)
        aux = torch.cat([torch.full((T, 2), 7.0), cut("a").reshape(T, -1)], dim=1).contiguous().to(DEV)
        o = ops.state_scan(ops.SCAN_ROW_DECAY, rows, 1, 1 + H * d, 1 + 2 * H * d, aux, 2, state, step.seg_start, step.seg_slot, H, 1, d, dv,
                           True, max(lens)).double().cpu().view(T, H, dv)
        want = torch.cat([ref[0][at[0]:at[0] + lens[0]], ref[2][at[2]:at[2] + lens[1]]])
        assert torch.allclose(o, want, rtol=1e-4, atol=1e-4), lens
        at[0] += lens[0]
        at[2] += lens[1]
    assert float((state[1] - 9.0).abs().sum()) == 0.0             # a slot that no segment names stays untouched
    # a step that must not write the state leaves it, and gives the same result twice
    step = _Step([3], [0], [1])
    rows = torch.randn(3, 1 + 2 * H * d + H * dv, generator=g).to(DEV)
    aux = torch.rand(3, 2 + H * d, generator=g).to(DEV)
    o1 = ops.state_scan(ops.SCAN_ROW_DECAY, rows, 1, 1 + H * d, 1 + 2 * H * d, aux, 2, state, step.seg_start, step.seg_slot, H, 1, d, dv, False, 3)
    o2 = ops.state_scan(ops.SCAN_ROW_DECAY, rows, 1, 1 + H * d, 1 + 2 * H * d, aux, 2, state, step.seg_start, step.seg_slot, H, 1, d, dv, False, 3)
    assert torch.equal(o1, o2) and float((state[1] - 9.0).abs().sum()) == 0.0


@pytest.mark.parametrize("taps", [0, 1, 2, 4])
@pytest.mark.parametrize("sizes", SCAN_SIZES)
def test_delta_rule_from_projected_rows(sizes, taps):
    """Filters with their tails, silu, unit vectors, step sizes and write strengths, then the recurrence, over steps
    that cut two requests anywhere; against the plain functions on the whole sequences."""
    H, G, d, dv = sizes
    if taps in (1, 2) and d > 40:
        pytest.skip("the filter lengths are covered on the small heads")
    g = torch.Generator().manual_seed(d + dv + taps)
    total = [70, 12]
    C = 2 * G * d + H * dv
    fw = torch.randn(C, max(taps, 1), generator=g) * 0.5
    a_log, dt_bias = torch.randn(H, generator=g) * 0.5, torch.randn(H, generator=g) - 1.0
    seqs, ref = {}, {}
    for slot, n in zip((0, 2), total):
        raw = torch.randn(n, C + 2 * H, generator=g)
        seqs[slot] = raw
        x = raw.double()
        f = pf.silu(pf.causal_filter(x[:, :C], fw) if taps else x[:, :C])
        q, k = pf.unit(f[:, :G * d].view(n, G, d)) * d ** -0.5, pf.unit(f[:, G * d:2 * G * d].view(n, G, d))
        v = f[:, 2 * G * d:].view(n, H, dv)
        gate = torch.exp(-torch.exp(a_log.double()) * torch.nn.functional.softplus(x[:, C:C + H] + dt_bias.double()))
        beta = torch.sigmoid(x[:, C + H:])
        ref[slot] = torch.stack([pf.delta_rule_scan(q[:, h // (H // G)], k[:, h // (H // G)], v[:, h], gate[:, h], beta[:, h])[0]
                                 for h in range(H)], dim=1)
    state = torch.zeros(3, H, d, dv, device=DEV)
    tails = torch.zeros(3, taps - 1, C, device=DEV) if taps > 1 else None
    at = {0: 0, 2: 0}
    for lens in _portions(total):
        step = _Step(lens, [at[0], at[2]], [0, 2])
        T = sum(lens)
        rows = torch.cat([torch.full((T, 3), 7.0), torch.cat([seqs[0][at[0]:at[0] + lens[0]], seqs[2][at[2]:at[2] + lens[1]]])], dim=1).contiguous().to(DEV)
        inline = tails is not None and max(lens) == 1           # steps of single tokens: the kernel moves the tails itself
        prep = ops.delta_prepare(rows, 3, 3 + C, 3 + C + H, fw.t().contiguous().to(DEV) if taps else None, tails, a_log.to(DEV), dt_bias.to(DEV),
                                 pf.UNIT_EPS, d ** -0.5, step, H, G, d, dv, inline)
        if tails is not None and not inline:
            ops.tail_update(rows, 3, tails, step.seg_start, step.seg_slot)
        o = ops.state_scan(ops.SCAN_DELTA_RULE, prep, 0, G * d, 2 * G * d, prep, C, state, step.seg_start, step.seg_slot, H, H // G, d, dv,
                           True, max(lens)).double().cpu().view(T, H, dv)
        want = torch.cat([ref[0][at[0]:at[0] + lens[0]], ref[2][at[2]:at[2] + lens[1]]])
        assert torch.allclose(o, want, rtol=2e-4, atol=2e-4), lens
        at[0] += lens[0]
        at[2] += lens[1]
    if tails is not None:
        assert float(tails[1].abs().sum()) == 0.0
        assert torch.equal(tails[0].cpu(), seqs[0][at[0] - (taps - 1):at[0], :C])


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("gate_dtype", [None, torch.float32, torch.bfloat16])
def test_head_norm_with_an_output_gate(out_dtype, gate_dtype):
    g = torch.Generator().manual_seed(5)
    T, H, dv = 6, 3, 20
    o, w = 4.0 * torch.randn(T, H * dv, generator=g), torch.randn(dv, generator=g)
    gate = None if gate_dtype is None else torch.randn(T, 5 + H * dv, generator=g).to(gate_dtype)
    want = pf.rms_weighted(o.double().view(T, H, dv), w, 1e-5).reshape(T, H * dv)
    if gate is not None:
        want = want * pf.silu(gate[:, 5:].double())
    got = ops.head_norm_gate(o.to(DEV), w.to(DEV), 1e-5, None if gate is None else gate.to(DEV), 5, H, dv, out_dtype).double().cpu()
    assert torch.allclose(got, want, **_tol(out_dtype))
