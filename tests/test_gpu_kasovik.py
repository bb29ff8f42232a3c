"""Kasovik on the GPU. Each new kernel alone against its plain twin (tests/ref_kernels.py) and, where a mechanism has a
formula of its own in tests/plain_kasovik.py, against that, with inputs made so that a fault shows (one key whose score
stands out just inside or just outside the window, a sink that takes most of the denominator, a write hundreds of
tokens back that only a slow decay keeps); then the replayer in 32-bit and bfloat16 against the plain implementation:
whole prompts, prefill against token-by-token decoding, portions down to two tokens, unequal requests mixed in a pool
whose pages and slots are used again, the first tokens, long decoding, sizes that are multiples of nothing; and greedy
generation through the engine's scheduler and graphs."""
from __future__ import annotations

import math
import types

import pytest
import torch

import plain_kasovik as plain
from helpers import random_prompt
from holon_b200.replay import Replayer
from kasovik_tools import CONFIGS, compare, exact_logits, make_folder, read_folder
from ref_kernels import RefKernels
from replay_tools import mixed_trace, portions, run

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
REF = RefKernels()
F64 = torch.float64


@pytest.fixture(scope="module")
def K():
    from holon_b200.kernels import load_kernels
    return load_kernels(DEV)


def rand(*shape, dtype=torch.float32, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype)


def close(got, want, dtype, scale=1.0):
    tol = (3e-5 if dtype == torch.float32 else 1.6e-2) * scale
    diff = (got.float().cpu() - want.float()).abs().max().item()
    assert diff <= tol, f"difference {diff} > {tol}"


def rows_of(counts, slots, kv_len=None, device=DEV):
    """The rows of a step: `counts` tokens each, in slots `slots`."""
    qs = [0]
    for n in counts:
        qs.append(qs[-1] + n)
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=device)      # noqa: E731
    kv = kv_len or counts
    return types.SimpleNamespace(query_start=t(qs), row_slot=t(slots), kv_len=t(kv), n_rows=len(counts), n_tokens=qs[-1],
                                 n_decode=sum(1 for n in counts if n == 1), max_q=max(counts), max_kv=max(kv),
                                 host_query_start=qs, host_kv_len=kv, plan={})


# ---------------------------------------------------------------- the scan over a matrix state per head
@pytest.mark.parametrize("heads,kv_heads,dim,vdim", [(2, 2, 16, 24), (4, 2, 32, 64), (3, 1, 12, 20), (2, 2, 96, 80),
                                                     (2, 1, 160, 48), (1, 1, 64, 300), (2, 2, 300, 16)])
@pytest.mark.parametrize("mode", ["delta", "fixed"])
def test_recurrent_scan(K, heads, kv_heads, dim, vdim, mode):
    """Rows of 1, 2, 11 and 37 tokens in slots of their own, on states that hold something already; once more on the
    states that the first call left (a state is read at a row's start and written back at its end)."""
    counts, slots = [1, 1, 2, 11, 37], [3, 0, 5, 1, 4]
    t = sum(counts)
    qk = rand(t, 2, kv_heads, dim, seed=1) / dim ** 0.5
    qk[:, 1] = qk[:, 1] / qk[:, 1].norm(dim=-1, keepdim=True)
    v = rand(t, heads, vdim, seed=2)
    decay = torch.sigmoid(rand(t, heads, dim, seed=3) + 2.0) if mode == "delta" else None
    fixed = torch.tensor([0.9, 0.99, 0.5, 0.97][:heads]) if mode == "fixed" else None
    beta = torch.sigmoid(rand(t, heads, seed=4)) if mode == "delta" else None
    state = rand(7, heads, vdim, dim, seed=5) * 0.3
    sg, sw = state.clone().to(DEV), state.clone()
    for _ in range(2):
        out, want = torch.full((t, heads, vdim), float("nan"), device=DEV), torch.zeros(t, heads, vdim)
        K.recurrent_scan(out, qk.to(DEV), v.to(DEV), decay.to(DEV) if decay is not None else None,
                         fixed.to(DEV) if fixed is not None else None, beta.to(DEV) if beta is not None else None, sg,
                         rows_of(counts, slots))
        REF.recurrent_scan(want, qk, v, decay, fixed, beta, sw, rows_of(counts, slots, device="cpu"))
        close(out, want, torch.float32, scale=4.0)
        close(sg, sw, torch.float32, scale=4.0)
    assert torch.equal(sg[2].cpu(), state[2]) and torch.equal(sg[6].cpu(), state[6])      # slots of no row are untouched


def test_the_scan_keeps_a_far_write(K):
    """One head, a decay of 0.999: what token 3 wrote is read 600 tokens later by a query along its key, beside hundreds
    of other writes (every other key is orthogonal to that query); with a decay of 0.9 nothing of it is left."""
    dim, vdim, t = 32, 16, 640
    qk = torch.zeros(t, 2, 1, dim)
    qk[:, 1, 0, 1:] = rand(t, dim - 1, seed=1)
    qk[3, 1, 0] = 0
    qk[3, 1, 0, 0] = 1.0                       # the far key: channel 0, which no other key uses
    qk[603, 0, 0, 0] = 1.0                     # the query that asks for it
    v = rand(t, 1, vdim, seed=2)
    for decay, kept in ((0.999, 0.999 ** 600), (0.9, 0.0)):
        out = torch.empty(t, 1, vdim, device=DEV)
        state = torch.zeros(1, 1, vdim, dim, device=DEV)
        K.recurrent_scan(out, qk.to(DEV), v.to(DEV), None, torch.tensor([decay], device=DEV), None, state, rows_of([t], [0]))
        assert torch.allclose(out[603, 0].cpu(), kept * v[3, 0], atol=1e-5)


# ---------------------------------------------------------------- from the first product to the scan's inputs
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,dim,vdim,taps", [(4, 2, 16, 32, 4), (6, 2, 12, 20, 2), (2, 2, 96, 80, 1), (3, 3, 8, 8, 7)])
def test_delta_prepare_and_the_carried_inputs(K, dtype, heads, kv_heads, dim, vdim, taps):
    """Rows of 1, 2, 5 and 9 tokens: shorter than, as long as and longer than the convolution's reach, so the carried
    inputs are read, shifted and replaced; three steps in a row on the same slots."""
    counts, slots = [1, 2, 5, 9], [2, 0, 3, 1]
    t = sum(counts)
    nq, nv = kv_heads * dim, heads * vdim
    c = 2 * nq + nv
    conv = rand(c, taps, dtype=dtype, seed=1, scale=0.6)
    dt_bias, rate_log = rand(heads * dim, seed=4), rand(heads, seed=5) - 1.0
    carried = rand(5, max(taps - 1, 0), c, dtype=dtype, seed=6) if taps > 1 else None
    cg, cw = (carried.clone().to(DEV), carried.clone()) if taps > 1 else (None, None)
    for step in range(3):
        first, low2 = rand(t, c + heads, dtype=dtype, seed=10 + step), rand(t, heads * dim + nv, seed=20 + step, scale=2.0)
        shapes = [(t, 2, kv_heads, dim), (t, heads, vdim), (t, heads), (t, heads, dim), (t, nv)]
        got = [torch.full(s, float("nan"), device=DEV) for s in shapes]
        want = [torch.zeros(s) for s in shapes]
        K.delta_prepare(*got, first.to(DEV), conv.to(DEV), cg, low2.to(DEV), dt_bias.to(DEV), rate_log.to(DEV),
                        rows_of(counts, slots), dim ** -0.5, 1e-6)
        K.conv_carry(cg, first.to(DEV), c, taps, rows_of(counts, slots))
        REF.delta_prepare(*want, first, conv, cw, low2, dt_bias, rate_log, rows_of(counts, slots, device="cpu"), dim ** -0.5, 1e-6)
        REF.conv_carry(cw, first, c, taps, rows_of(counts, slots, device="cpu"))
        for g, w in zip(got, want):
            close(g, w, torch.float32, scale=8.0)
        if taps > 1:
            assert torch.equal(cg.cpu(), cw)
            assert torch.equal(cg[4].cpu(), carried[4])           # a slot of no row


def test_the_convolution_against_its_formula(K):
    """One request fed in portions of 1, 2, 3, 1 and 6 tokens gives the causal convolution of the whole sequence."""
    heads = kv_heads = 1
    dim, vdim, taps = 8, 8, 4
    c, t = 24, 13
    x = rand(t, c + heads, seed=1)
    conv = rand(c, taps, seed=2)
    want = plain.silu(plain.short_conv(x[:, :c].double(), conv.double()))
    carried = torch.zeros(2, taps - 1, c, device=DEV)
    rest = [rand(heads * dim, seed=4), rand(heads, seed=5)]
    at, got = 0, []
    for n in (1, 2, 3, 1, 6):
        first = x[at:at + n].contiguous().to(DEV)
        out = [torch.empty(s, device=DEV) for s in [(n, 2, 1, dim), (n, 1, vdim), (n, 1), (n, 1, dim), (n, vdim)]]
        K.delta_prepare(*out, first, conv.to(DEV), carried, torch.zeros(n, heads * dim + vdim, device=DEV), rest[0].to(DEV),
                        rest[1].to(DEV), rows_of([n], [1]), 1.0, 1e-6)
        K.conv_carry(carried, first, c, taps, rows_of([n], [1]))
        got.append(out[1].view(n, vdim).cpu())
        at += n
    assert torch.allclose(torch.cat(got).double(), want[:, 16:], atol=1e-5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,vdim,rot_dims", [(2, 32, 48, 16), (3, 24, 40, 8), (2, 160, 64, 160), (1, 16, 16, 0)])
def test_retention_prepare_and_head_norm_gate(K, dtype, heads, dim, vdim, rot_dims):
    t, extra = 9, heads * vdim
    first = rand(t, 2 * heads * dim + heads * vdim + extra, dtype=dtype, seed=1)
    positions = torch.tensor([0, 1, 2, 3, 100, 7, 8, 9, 63], dtype=torch.int32)
    table = None
    if rot_dims:
        freq = torch.tensor([300.0 ** (-2.0 * i / rot_dims) for i in range(rot_dims // 2)])
        angle = torch.arange(128, dtype=torch.float32)[:, None] * freq[None]
        table = torch.cat((angle.cos(), angle.sin()), -1).contiguous()
    qk_g, v_g = torch.empty(t, 2, heads, dim, device=DEV), torch.empty(t, heads, vdim, device=DEV)
    qk_w, v_w = torch.zeros(t, 2, heads, dim), torch.zeros(t, heads, vdim)
    K.retention_prepare(qk_g, v_g, first.to(DEV), positions.to(DEV), table.to(DEV) if rot_dims else None, rot_dims, dim ** -0.5)
    REF.retention_prepare(qk_w, v_w, first, positions, table, rot_dims, dim ** -0.5)
    close(qk_g, qk_w, torch.float32, scale=4.0)
    close(v_g, v_w, torch.float32, scale=4.0)
    if rot_dims:                                     # against the written-out rotation
        q = first[:, :heads * dim].double().view(t, heads, dim)
        assert torch.allclose(qk_g[:, 0].cpu().double(), plain.rotate(q, positions.tolist(), 300.0, rot_dims), atol=2e-5)
    o = rand(t, heads, vdim, seed=2) * 3.0
    weight, gate_mul = 1 + rand(vdim, seed=3) * 0.1, torch.sigmoid(rand(t, heads * vdim, seed=4))
    gate_pre = first[:, -extra:]
    for w, gm, gp in ((weight, gate_mul, None), (None, None, gate_pre), (None, None, None), (weight, None, gate_pre)):
        out, want = torch.empty(t, heads, vdim, dtype=dtype, device=DEV), torch.zeros(t, heads, vdim, dtype=dtype)
        K.head_norm_gate(out, o.to(DEV), w.to(DEV) if w is not None else None, gm.to(DEV) if gm is not None else None,
                         first.to(DEV)[:, -extra:] if gp is not None else None, 1e-5)
        REF.head_norm_gate(want, o, w, gm, gp, 1e-5)
        close(out, want, dtype, scale=4.0)


# ---------------------------------------------------------------- embedding, the block's sum, the gated unit
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_pair_sum_into_and_glu(K, dtype):
    vocab, hidden, buckets = 97, 72, 31
    table, pair = rand(vocab, hidden, dtype=dtype, seed=1), rand(buckets + 1, hidden, dtype=dtype, seed=2)
    counts, slots = [1, 1, 3, 6], [2, 0, 3, 1]
    ids = torch.randint(0, vocab, (11,), generator=torch.Generator().manual_seed(3), dtype=torch.int32)
    positions = torch.tensor([5, 0, 0, 1, 2, 7, 8, 9, 10, 11, 12], dtype=torch.int32)
    prev = torch.tensor([9, 8, 7, 6, 5], dtype=torch.int32)
    pg, pw = prev.clone().to(DEV), prev.clone()
    out, want = torch.empty(11, hidden, device=DEV), torch.zeros(11, hidden)
    K.embed_pair(out, table.to(DEV), 2.5, pair.to(DEV), ids.to(DEV), positions.to(DEV), rows_of(counts, slots), pg, 13, 5, buckets)
    REF.embed_pair(want, table, 2.5, pair, ids, positions, rows_of(counts, slots, device="cpu"), pw, 13, 5, buckets)
    close(out, want, torch.float32, scale=4.0)
    assert torch.equal(pg.cpu(), pw) and pw.tolist() == [int(ids[1]), int(ids[10]), int(ids[0]), int(ids[4]), 5]
    x = table.double()[ids.long()] * 2.5                                  # against the formula, by hand
    first = x[1] + pair.double()[buckets]                                 # position 0: the table's last row
    later = x[5] + pair.double()[(8 * 13 + int(ids[5]) * 5) % buckets]    # a row's first token: the slot's previous token
    inner = x[3] + pair.double()[(int(ids[2]) * 13 + int(ids[3]) * 5) % buckets]
    for at, value in ((1, first), (5, later), (3, inner)):
        assert torch.allclose(out[at].cpu().double(), value, atol=1e-5)
    h = rand(11, hidden, seed=4)
    terms = [(rand(11, hidden, dtype=dtype, seed=5 + i), s) for i, s in enumerate((0.7, 1.3, 1.0))]
    bias = rand(hidden, dtype=dtype, seed=9)
    for n, b in ((1, None), (2, bias), (3, bias)):
        hg, hw = h.clone().to(DEV), h.clone()
        K.sum_into(hg, [(x.to(DEV), s) for x, s in terms[:n]], b.to(DEV) if b is not None else None)
        REF.sum_into(hw, terms[:n], b)
        close(hg, hw, torch.float32, scale=4.0)
        for gain in (1 + rand(hidden, seed=12) * 0.1, (1 + rand(hidden, seed=12) * 0.1).to(dtype)):      # the sum and the next norm in one
            hg, hw = h.clone().to(DEV), h.clone()
            og, ow = torch.empty(11, hidden, dtype=dtype, device=DEV), torch.zeros(11, hidden, dtype=dtype)
            K.sum_norm(hg, [(x.to(DEV), s) for x, s in terms[:n]], b.to(DEV) if b is not None else None, og, gain.to(DEV), 1e-5, 0.0)
            REF.sum_norm(hw, terms[:n], b, ow, gain, 1e-5, 0.0)
            close(hg, hw, torch.float32, scale=4.0)
            close(og, ow, dtype, scale=4.0)
    inter = 100
    gate_up, b2 = rand(11, 2 * inter, dtype=dtype, seed=10, scale=2.0), rand(2 * inter, dtype=dtype, seed=11)
    for limit, b in ((0.75, b2), (2.0, None)):
        act, want = torch.empty(11, inter, dtype=dtype, device=DEV), torch.zeros(11, inter, dtype=dtype)
        K.glu_clamped(act, gate_up.to(DEV), b.to(DEV) if b is not None else None, limit, 1.702)
        REF.glu_clamped(want, gate_up, b, limit, 1.702)
        close(act, want, dtype, scale=4.0)


# ---------------------------------------------------------------- attention with a window and a sink
def _paged(keys, values, page, dtype):
    """A cache [pages, 2, kv_heads, page, dim] and a one-row block table for keys and values [n, kv_heads, dim], the
    pages in reverse order."""
    n, kvh, d = keys.shape
    pages = -(-n // page)
    kv = torch.zeros(pages + 1, 2, kvh, page, d, dtype=dtype)
    table = torch.full((1, pages + 2), pages, dtype=torch.int32)
    for i in range(pages):
        phys = pages - 1 - i
        table[0, i] = phys
        m = min(page, n - i * page)
        kv[phys, 0, :, :m] = keys[i * page:i * page + m].transpose(0, 1)
        kv[phys, 1, :, :m] = values[i * page:i * page + m].transpose(0, 1)
    return kv, table


def _attend(q, keys, values, scale, window, sink):
    """Softmax over the last `window` keys with exp(sink) in the denominator, in 64-bit; q [queries, heads, d], the
    queries being the last ones of the n keys."""
    n, (nq, heads, d) = keys.shape[0], q.shape
    group = heads // keys.shape[1]
    out = torch.zeros(nq, heads, d, dtype=F64)
    for i in range(nq):
        pos = n - nq + i
        lo = max(0, pos - window + 1) if window else 0
        for h in range(heads):
            s = (keys[lo:pos + 1, h // group].double() @ q[i, h].double()) * scale
            top = max(float(s.max()), float(sink[h]))
            e = torch.exp(s - top)
            out[i, h] = (e[:, None] * values[lo:pos + 1, h // group].double()).sum(0) / (e.sum() + math.exp(float(sink[h]) - top))
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,d,window,n,nq,page", [(4, 2, 32, 9, 40, 1, 4), (8, 1, 96, 72, 300, 1, 64), (8, 1, 96, 72, 300, 130, 64),
                                                               (3, 3, 20, 5, 33, 7, 16), (2, 1, 64, 70, 200, 1, 64), (2, 1, 64, 70, 200, 2, 16),
                                                               (4, 4, 128, 100, 400, 1, 64), (4, 4, 128, 100, 400, 150, 64), (2, 2, 48, 1000, 700, 1, 64)])
def test_attention_with_a_sink_at_the_window_s_edges(K, dtype, heads, kv_heads, d, window, n, nq, page):
    """The last query's key just inside the window and the key just outside it both point along the query, far more than
    any other: the inner one must take the weight, the outer one none (where the window is longer than the row, the
    fourth key of 700 stands out instead); the sink takes a visible share. Rows of one token
    (the split kernel and its merge), of several (the prompt kernel), head sizes the tensor cores take and others."""
    keys, values = rand(n, kv_heads, d, seed=1), rand(n, kv_heads, d, seed=2)
    q = rand(nq, heads, d, seed=3)
    scale = 2.0 / d ** 0.5
    inside, outside = n - window, n - window - 1
    direction = q[-1, 0] / q[-1, 0].norm()
    if inside >= 0:
        keys[inside, 0] = 3.0 * direction * d ** 0.5 / 2
    else:                                               # the window is longer than the row: a far key among hundreds
        keys[3, 0] = 3.0 * direction * d ** 0.5 / 2
    if outside >= 0:
        keys[outside, 0] = 6.0 * direction * d ** 0.5 / 2
    keys, values, q = keys.to(dtype), values.to(dtype), q.to(dtype)
    lo = max(0, n - window)                             # each head's sink near the log-sum of its last query's scores:
    group = heads // kv_heads                           # it takes about half of that denominator
    lse = torch.stack([torch.logsumexp(keys[lo:, h // group].float() @ q[-1, h].float() * scale, 0) for h in range(heads)])
    sink = lse + torch.tensor([0.5, -0.5, 0.3, 1.0, 0.0, -1.0, 1.0, 0.7][:heads])
    want = _attend(q.float(), keys.float(), values.float(), scale, window, sink)
    without = _attend(q.float(), keys.float(), values.float(), scale, window, sink - 30.0)
    assert float((want - without).abs().max()) > 0.05                       # the sink matters here
    kv, table = _paged(keys, values, page, dtype)
    rows = rows_of([nq], [0], kv_len=[n])
    out = torch.full((nq, heads, d), float("nan"), dtype=dtype, device=DEV)
    K.paged_attention(out, q.to(DEV), kv.to(DEV), table.to(DEV), rows, scale, window, sink.to(DEV))
    close(out, want, dtype, scale=4.0)
    twin = torch.zeros(nq, heads, d, dtype=dtype)
    REF.paged_attention(twin, q, kv, table, rows_of([nq], [0], kv_len=[n], device="cpu"), scale, window, sink)
    close(twin, want, dtype, scale=4.0)


@pytest.mark.parametrize("cluster", [False, True])
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_one_token_rows_with_a_sink_in_parts(K, splits, cluster, monkeypatch):
    """The keys of a one-token row cut into parts, merged by a second kernel or inside a thread-block cluster: the sink
    enters the denominator once."""
    heads, kv_heads, d, window, n = 4, 2, 64, 0, 700
    keys, values, q = rand(n, kv_heads, d, dtype=torch.bfloat16, seed=1), rand(n, kv_heads, d, dtype=torch.bfloat16, seed=2), rand(1, heads, d, dtype=torch.bfloat16, seed=3)
    sink = torch.tensor([4.0, 2.0, 0.0, 5.0])
    want = _attend(q.float(), keys.float(), values.float(), 0.2, window, sink)
    kv, table = _paged(keys, values, 64, torch.bfloat16)
    monkeypatch.setattr(K, "decode_splits", lambda *a, **k: splits)
    monkeypatch.setattr(K, "decode_cluster", cluster)
    if cluster:
        monkeypatch.setattr(K, "decode_cluster_splits", lambda *a, **k: splits if splits > 1 else 0)
    out = torch.empty(1, heads, d, dtype=torch.bfloat16, device=DEV)
    K.paged_attention(out, q.to(DEV), kv.to(DEV), table.to(DEV), rows_of([1], [0], kv_len=[n]), 0.2, window, sink.to(DEV))
    close(out, want, torch.bfloat16)


# ---------------------------------------------------------------- the model through the replayer and the engine
@pytest.fixture(scope="module", params=sorted(CONFIGS))
def model(request, tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("models"), request.param, seed=7)
    config = CONFIGS[request.param]
    prompts = {f"r{i}": random_prompt(config["vocab"], n, 40 + i) for i, n in enumerate((70, 133, 37, 96))}
    return folder, config, prompts, {rid: exact_logits(folder, ids) for rid, ids in prompts.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_then_tail_then_portions(model, dtype):
    folder, config, prompts, want = model
    r = Replayer(str(folder), dtype, max_tokens=192)
    compare(run(r, [([(rid, ids)], [rid]) for rid, ids in prompts.items()]), want, dtype)
    steps = []
    for rid, ids in prompts.items():                     # most of it in one step, the last 32 tokens one by one
        cut = len(ids) - 32
        steps.append(([(rid, ids[:cut])], []))
        steps += [([(rid, [t])], [rid] if i == 31 else []) for i, t in enumerate(ids[cut:])]
    compare(run(r, steps), want, dtype)
    steps = []
    for rid, ids in prompts.items():                     # portions of changing size, down to two tokens
        parts = portions(ids, [7, 2, 19, 3, 2, 64, 5])
        steps += [([(rid, p)], [rid] if i == len(parts) - 1 else []) for i, p in enumerate(parts)]
    compare(run(r, steps), want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [64, 16])
def test_mixed_requests_in_a_small_pool(model, dtype, page_size):
    """Four unequal requests live at once in 448 tokens of pool: three arrive in portions while one decodes; when it
    ends, the last one grows into pages it gave back. Every row must equal the request run alone."""
    folder, config, prompts, want = model
    r = Replayer(str(folder), dtype, max_tokens=448, page_size=page_size)
    got = run(r, mixed_trace(prompts))
    assert len(got) == sum(map(len, prompts.values())) and not r.built.cache.live
    compare(got, want, dtype)
    got = run(r, mixed_trace(prompts))                   # once more in the same engine: every page and slot used again
    compare(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_the_first_tokens(model, dtype):
    folder, config, _, _ = model
    ids = random_prompt(config["vocab"], 330, 77)
    want = {"x": exact_logits(folder, ids)}
    r = Replayer(str(folder), dtype, max_tokens=384)
    got = run(r, [([("x", [t])], ["x"] if i == len(ids) - 1 else []) for i, t in enumerate(ids)])   # all one by one
    compare(got, want, dtype)
    compare({k: v for k, v in got.items() if k[1] < 4}, want, dtype)
    # a prompt of 260 tokens (past four page borders, the window over pages given back), then single tokens
    got = run(r, [([("x", ids[:260])], [])] + [([("x", [t])], []) for t in ids[260:]])
    compare(got, want, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_heads_of_128_and_large_key_sizes(tmp_path, dtype):
    """Whole prompts of 300 and 133 tokens (the tcgen05 prompt attention with a window of 100 and a sink), their last 32
    tokens one by one, and portions, at sizes where a thread of the scan holds 8 and 16 key channels."""
    from kasovik_tools import KD
    folder = make_folder(tmp_path, "d", seed=3, config=KD)
    prompts = {f"r{i}": random_prompt(KD["vocab"], n, 50 + i) for i, n in enumerate((300, 133))}
    want = {rid: exact_logits(folder, ids) for rid, ids in prompts.items()}
    r = Replayer(str(folder), dtype, max_tokens=512)
    compare(run(r, [([(rid, ids)], [rid]) for rid, ids in prompts.items()]), want, dtype)
    steps = []
    for rid, ids in prompts.items():
        cut = len(ids) - 32
        steps.append(([(rid, ids[:cut])], []))
        steps += [([(rid, [t])], [rid] if i == 31 else []) for i, t in enumerate(ids[cut:])]
    compare(run(r, steps), want, dtype)
    steps = []
    for rid, ids in prompts.items():
        parts = portions(ids, [7, 2, 130, 3, 64])
        steps += [([(rid, p)], [rid] if i == len(parts) - 1 else []) for i, p in enumerate(parts)]
    compare(run(r, steps), want, dtype)


def test_a_token_far_back_is_remembered(tmp_path):
    """The matrix states must carry a token from 300 places back: the logits of the last rows change when token 7
    changes, and the engine follows the plain implementation through that change, in a prompt and in decoding, with the
    two requests side by side in one batch."""
    folder = make_folder(tmp_path, "b", seed=11)
    vocab = CONFIGS["b"]["vocab"]
    ids = random_prompt(vocab, 320, 5)
    other = list(ids)
    other[7] = (ids[7] + 1) % vocab
    want = {"x": exact_logits(folder, ids), "y": exact_logits(folder, other)}
    assert float((want["x"][-1] - want["y"][-1]).abs().max()) > 1e-3         # the far token matters to the last row
    r = Replayer(str(folder), "float32", max_tokens=768)
    steps = [([("x", ids[:300]), ("y", other[:300])], [])] + [([("x", [a]), ("y", [b])], []) for a, b in zip(ids[300:], other[300:])]
    compare(run(r, steps), want, "float32")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(model, dtype, graphs):
    from holon_b200.engine import Engine, EngineConfig, SamplingParams
    folder, config, prompts, _ = model
    stored, weights = read_folder(folder)
    engine = Engine(EngineConfig(model=str(folder), dtype=dtype, page_size=64, max_seqs=4, max_model_len=256,
                                 max_step_tokens=96, state_memory=1 << 26, cuda_graphs=graphs, chunk_with_decode=32))
    asked = [prompts["r0"], prompts["r2"], prompts["r1"], prompts["r3"], prompts["r0"][:40] + prompts["r2"]]
    with torch.inference_mode():
        got = engine.generate(asked, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    engine.close()
    margin, off = (1e-3 if dtype == "float32" else 0.25), []
    for prompt, tokens in zip(asked, got):
        ids = list(prompt)
        assert len(tokens) == 12
        for token in tokens:                             # (each token judged after the engine's own earlier ones)
            logits = plain.forward(weights, stored, ids)[-1]
            if float(logits.max() - logits[token]) > margin * float(logits.std()):
                off.append((len(ids), token, int(logits.argmax())))
            ids.append(token)
    assert len(off) <= (0 if dtype == "float32" else 2), off


def test_generate_on_the_command_line(tmp_path, capsys):
    """`holon-b200 generate` with the engine's own sizing of the cache (activation peaks measured on the largest step)."""
    import json

    from holon_b200 import cli
    folder = make_folder(tmp_path, "a", seed=8)
    config, weights = read_folder(folder)
    assert cli.main(["generate", str(folder), "--prompt-ids", "5,17,3,90,12,7", "--prompt-ids", "9 8 7 6", "--max-tokens", "6",
                     "--dtype", "float32", "--max-model-len", "128", "--max-seqs", "4", "--max-step-tokens", "128", "--ignore-eos",
                     "--memory-fraction", "0.05"]) == 0
    captured = capsys.readouterr()
    lines = [json.loads(line) for line in captured.out.splitlines()]
    assert [o["prompt_ids"] for o in lines] == [[5, 17, 3, 90, 12, 7], [9, 8, 7, 6]]
    for o in lines:
        ids = list(o["prompt_ids"])
        assert len(o["token_ids"]) == 6
        for token in o["token_ids"]:
            logits = plain.forward(weights, config, ids)[-1]
            assert float(logits.max() - logits[token]) <= 1e-3 * float(logits.std()), (len(ids), token)
            ids.append(token)
