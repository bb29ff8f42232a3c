"""Rulorax on the GPU. Each new kernel alone against its plain twin (tests/ref_kernels.py) and, where a mechanism has a
formula of its own in tests/plain_rulorax.py, against that; then the replayer in 32-bit and bfloat16 against the plain
implementation: whole prompts, prefill against token-by-token decoding, portions down to two tokens, unequal requests
mixed in a pool whose pages and slots are used again, keys far away and at page borders, the first tokens, long
decoding, sizes that are multiples of nothing; and greedy generation through the engine's scheduler and graphs."""
from __future__ import annotations

import numpy as np
import pytest
import torch

import plain_rulorax as plain
from helpers import random_prompt
from holon_b200.engine.batch import Rows
from holon_b200.replay import Replayer
from ref_kernels import RefKernels
from replay_tools import mixed_trace, portions, run
from rulorax_tools import CONFIGS, RX_E, compare, exact_logits, make_folder

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]
REF = RefKernels()


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


def dev(*tensors):
    return [None if t is None else t.to(DEV) for t in tensors]


# ---------------------------------------------------------------- hyper-connections
@pytest.mark.parametrize("streams,dim", [(1, 200), (2, 200), (3, 200), (4, 200), (7, 200), (4, 2048), (3, 2560), (2, 5000), (8, 2048), (11, 3000)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_hyper_mix_norm(K, streams, dim, dtype):
    """(Rows of up to 4,096 columns and four streams are held whole by the block's threads; wider rows and more streams
    take the general path, the latter with fewer threads.)"""
    t = 6
    xs, src, y = rand(t, streams, dim, seed=1), rand(t, dim, seed=2), rand(t, dim, dtype=dtype, seed=3)
    mix, outc, inc = torch.eye(streams) + rand(streams, streams, seed=4) * 0.3, 1 + rand(streams, seed=5) * 0.3, rand(streams, seed=6)
    w = (1 + rand(dim, seed=7) * 0.1).to(dtype)
    cases = [dict(src=src, y=None), dict(src=None, y=y), dict(src=None, y=None), dict(src=src, y=y),
             dict(src=None, y=y, inc=None, index=torch.tensor([4, 0, 4], dtype=torch.int32))]
    for case in cases:
        index, inc_ = case.get("index"), case.get("inc", inc)
        rows = t if index is None else index.shape[0]
        fold = case["y"] is not None
        xg, xw = xs.clone().to(DEV), xs.clone()
        out, want = torch.empty(rows, dim, dtype=dtype, device=DEV), torch.empty(rows, dim, dtype=dtype)
        K.hyper_mix_norm(out, xg, *dev(case["src"], case["y"], mix if fold else None, outc if fold else None, inc_, w), 1e-5, 0.0,
                         index.to(DEV) if index is not None else None)
        REF.hyper_mix_norm(want, xw, case["src"], case["y"], mix if fold else None, outc if fold else None, inc_, w, 1e-5, 0.0, index)
        close(out, want, dtype, scale=4.0)
        assert torch.allclose(xg.cpu(), xw, atol=1e-5), "the streams written differ"
        if index is not None:
            assert torch.equal(xg.cpu(), xs), "a gather must write nothing"
    # against the written-out formulas: read with `in`, write with `mix` and `out`
    wd = {"p.in": inc.double(), "p.mix": mix.double(), "p.out": outc.double()}
    new = plain.hyper_write(xs.double().transpose(0, 1), y.double(), wd, "p.")
    u = plain.hyper_read(new, wd, "p.")
    xg = xs.clone().to(DEV)
    out = torch.empty(t, dim, dtype=dtype, device=DEV)
    K.hyper_mix_norm(out, xg, None, *dev(y, mix, outc, inc, w), 1e-5, 0.0, None)
    close(out, plain.rms_norm(u, w.double(), 1e-5), dtype, scale=4.0)
    assert torch.allclose(xg.cpu().double().transpose(0, 1), new, atol=1e-5)


# ---------------------------------------------------------------- latent attention: preparation
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dim,rot,rank,rot_dims", [(3, 20, 12, 40, 8), (4, 64, 32, 64, 32), (1, 16, 64, 512, 64), (2, 8, 0, 24, 0)])
def test_latent_prepare(K, dtype, heads, dim, rot, rank, rot_dims):
    t, page, pages = 9, 4, 5
    n_q, extra = heads * (dim + rot), 11
    ld = n_q + extra + rank + rot
    first = rand(t, ld, dtype=dtype, seed=1)
    positions = torch.tensor([0, 1, 2, 3, 100, 7, 8, 9, 63], dtype=torch.int32)
    widx = torch.tensor([0, 1, 2, 3, 19, 7, -1, 9, 12], dtype=torch.int32)
    table = None
    if rot_dims:
        freq = torch.tensor([300.0 ** (-2.0 * i / rot_dims) for i in range(rot_dims // 2)])
        angle = torch.arange(128, dtype=torch.float32)[:, None] * freq[None]
        table = torch.cat((angle.cos(), angle.sin()), -1).contiguous()
    w = (1 + rand(rank, seed=2) * 0.1).to(dtype)
    for fills in (True, False):
        qa_g, qa_w = torch.zeros(t, heads, rank + rot, dtype=dtype, device=DEV), torch.zeros(t, heads, rank + rot, dtype=dtype)
        cg, cw = torch.zeros(pages, page, rank + rot, dtype=dtype, device=DEV), torch.zeros(pages, page, rank + rot, dtype=dtype)
        args = (heads, dim, rot, rank, n_q + extra if fills else -1)
        K.latent_prepare(qa_g, first.to(DEV), *args, positions.to(DEV), *dev(table), rot_dims, *dev(w if fills else None), 1e-5,
                         cg if fills else None, widx.to(DEV) if fills else None)
        REF.latent_prepare(qa_w, first, *args, positions, table, rot_dims, w if fills else None, 1e-5, cw if fills else None,
                           widx if fills else None)
        close(qa_g, qa_w, dtype, scale=4.0)
        close(cg, cw, dtype, scale=4.0)
        if fills:
            assert float(cg[1, 2].abs().sum()) == 0.0          # the skipped token's row (write index -1) stays empty
            filled = cg
    if rot_dims:                                                # against the written-out rotation
        m = {"kv_rank": rank, "rot": {"base": 300.0, "dims": rot_dims}}
        wd = {"l0.mix.dkv": torch.eye(rank + rot, dtype=torch.float64), "l0.mix.dkv.norm": w.double()}
        c, k_r = plain.latent_kv(first[:, n_q + extra:].double(), wd, 0, m, positions.tolist(), 1e-5)
        rows = filled.view(-1, rank + rot)[widx[widx >= 0].long()].cpu()
        close(rows, torch.cat((c, k_r), -1)[widx >= 0], dtype, scale=4.0)


# ---------------------------------------------------------------- latent attention: the attention itself
def _rows(lens, new):
    """Rows for a step: request b holds lens[b] tokens afterwards and brings new[b] of them; one-token rows first."""
    order = sorted(range(len(lens)), key=lambda i: new[i] != 1)
    lens, new = [lens[i] for i in order], [new[i] for i in order]
    qs = np.zeros(len(lens) + 1, dtype=np.int32)
    np.cumsum(new, out=qs[1:])
    kv = np.array(lens, dtype=np.int32)
    slots = np.arange(len(lens), dtype=np.int32)
    return lambda device: Rows(torch.from_numpy(slots).to(device), torch.from_numpy(qs).to(device),
                               torch.from_numpy(kv).to(device), len(lens), int(qs[-1]), sum(1 for n in new if n == 1),
                               max(new), int(kv.max()), qs, kv)


def _paged(lens, page, rank, rot, dtype, seed):
    """A cache whose pages are handed out in a scrambled order, and each request's block-table row."""
    need = [-(-n // page) for n in lens]
    pages = sum(need) + 3
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(pages - 1, generator=g).tolist()
    table = torch.full((len(lens), max(need) + 1), pages - 1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(need):
        table[b, :n] = torch.tensor(perm[at:at + n], dtype=torch.int32)
        at += n
    cache = rand(pages, page, rank + rot, dtype=dtype, seed=seed + 1)
    return cache, table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("splits", [None, 3, 7])
@pytest.mark.parametrize("heads,rank,rot,page", [(4, 64, 32, 64), (3, 40, 12, 4), (16, 128, 64, 64), (1, 512, 64, 16), (5, 32, 16, 64),
                                                 (24, 64, 16, 64), (40, 256, 32, 64), (3, 144, 16, 16), (70, 80, 48, 64)])
def test_latent_attention(K, dtype, heads, rank, rot, page, splits, monkeypatch):
    """Rows of one token (short, at a tile's edge, long) beside portions of prompts; the bfloat16 kernel with the keys
    of one-token rows whole, in 3 and in 7 parts (some of them empty for the short rows)."""
    if splits and dtype == torch.float32:
        pytest.skip("the 32-bit kernel does not cut the keys")
    monkeypatch.setattr(K, "latent_split", splits)
    lens, new = [130, 1, 64, 65, 300, 7, 129, 641], [1, 1, 64, 2, 37, 7, 1, 1]
    cache, table = _paged(lens, page, rank, rot, dtype, 5)
    rows = _rows(lens, new)
    t = sum(new)
    qa = rand(t, heads, rank + rot, dtype=dtype, seed=9)
    scale = 2.0 / (rank + rot) ** 0.5
    rows_host = rows("cpu")
    lens_sorted = rows_host.host_kv_len.tolist()
    table = table[torch.tensor(sorted(range(len(lens)), key=lambda i: new[i] != 1))]
    # one key far back dominates the last query of the longest row; one at a page border another query
    b = lens_sorted.index(300)
    q_last = int(rows_host.host_query_start[b + 1]) - 1
    for key, q in ((3, q_last), (page * (256 // page) - 1 if page < 256 else 255, q_last - 1), (page, q_last - 2)):
        row = cache[int(table[b, key // page]), key % page]
        qa[q] = (row * (16.0 / float(row.float().pow(2).sum()) / scale)).to(dtype)[None, :]
    out, want = torch.empty(t, heads, rank, dtype=dtype, device=DEV), torch.empty(t, heads, rank, dtype=dtype)
    K.latent_attention(out, qa.to(DEV), cache.to(DEV), table.to(DEV), rows(DEV), scale, rank, 0)
    REF.latent_attention(want, qa, cache, table, rows_host, scale, rank, 0)
    close(out, want, dtype, scale=2.0)
    assert float((want[q_last].float() - cache[int(table[b, 0]), 3, :rank].float()).abs().max()) < 0.35   # the far key took the row


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_heads_on_views(K, dtype):
    t, heads, k, n, extra = 37, 5, 24, 40, 12
    wide = rand(t, heads * (k + extra) + 7, dtype=dtype, seed=1)
    x = wide[:, :heads * (k + extra)].view(t, heads, k + extra)[:, :, :k]
    w = rand(heads, n, k, dtype=dtype, seed=2, scale=0.2)
    out_wide = torch.zeros(t, heads, n + 9, dtype=dtype, device=DEV)
    xg = wide.to(DEV)[:, :heads * (k + extra)].view(t, heads, k + extra)[:, :, :k]
    K.linear_heads(out_wide[:, :, :n], xg, w.to(DEV))
    want = torch.empty(t, heads, n, dtype=dtype)
    REF.linear_heads(want, x, w)
    close(out_wide[:, :, :n], want, dtype, scale=2.0)
    assert float(out_wide[:, :, n:].abs().sum()) == 0.0


# ---------------------------------------------------------------- routed experts
@pytest.mark.parametrize("experts,top", [(16, 4), (5, 5), (1, 1), (300, 8), (9, 1)])
def test_route_top(K, experts, top):
    t = 33
    z = rand(t, experts + 1, seed=4, scale=2.0)
    z[3, :experts] = 0.25                                                    # all equal: the lowest experts win
    if experts > 2:
        z[5, 1] = z[5, 2] = 9.0                                              # two equal leaders: ascending
    for renorm in (False, True):
        chosen, weight = torch.empty(t, top, dtype=torch.int32, device=DEV), torch.empty(t, top, device=DEV)
        counts = torch.zeros(2 * experts + 1, dtype=torch.int32, device=DEV)
        K.route_top(chosen, weight, counts, z.to(DEV), experts, 1.7, renorm)
        c_w, w_w, n_w = torch.empty(t, top, dtype=torch.int32), torch.empty(t, top), torch.zeros(2 * experts + 1, dtype=torch.int32)
        REF.route_top(c_w, w_w, n_w, z, experts, 1.7, renorm)
        assert torch.equal(chosen.cpu(), c_w) and torch.equal(counts.cpu()[:experts], n_w[:experts])
        assert torch.allclose(weight.cpu(), w_w, rtol=1e-5, atol=1e-7)
        if not renorm:                                                       # against the written-out router
            _, s = plain.route(z[:, :experts].double(), {"router": torch.eye(experts, dtype=torch.float64)}, "", {"top": top, "scale": 1.7})
            assert torch.allclose(weight.cpu().double().sort(-1).values, s.sort(-1).values, rtol=1e-5)


@pytest.mark.parametrize("experts,top,tokens", [(16, 4, 8), (5, 5, 64), (1, 1, 3), (300, 8, 33), (9, 2, 300), (1100, 3, 20)])
def test_route_rows_in_one_call(K, experts, top, tokens):
    """Few tokens take one launch, many (or more than 1,024 experts) the separate kernels: the same choices, counts and
    first rows as the twin, every pair a row of its own in its expert's stretch, and the (0, tokens) pair behind them."""
    z = rand(tokens, experts + 1, seed=4, scale=2.0)
    chosen, weight = torch.empty(tokens, top, dtype=torch.int32, device=DEV), torch.empty(tokens, top, device=DEV)
    counts = torch.full((2 * experts + 3,), -7, dtype=torch.int32, device=DEV)
    place, token_of = (torch.empty(tokens * top, dtype=torch.int32, device=DEV) for _ in range(2))
    K.route_rows(chosen, weight, counts, place, token_of, z.to(DEV), experts, 0.6, True)
    c_w, w_w, n_w = torch.empty(tokens, top, dtype=torch.int32), torch.empty(tokens, top), torch.empty(2 * experts + 3, dtype=torch.int32)
    p_w, t_w = (torch.empty(tokens * top, dtype=torch.int32) for _ in range(2))
    REF.route_rows(c_w, w_w, n_w, p_w, t_w, z, experts, 0.6, True)
    assert torch.equal(chosen.cpu(), c_w) and torch.equal(counts.cpu(), n_w)
    assert torch.allclose(weight.cpu(), w_w, rtol=1e-5, atol=1e-7)
    place, token_of, starts = place.cpu().long(), token_of.cpu().long(), counts.cpu()[experts:2 * experts + 1].long()
    assert sorted(place.tolist()) == list(range(tokens * top))
    assert torch.equal(token_of[place], torch.arange(tokens * top) // top)
    e = c_w.long().reshape(-1)
    assert bool(((place >= starts[e]) & (place < starts[e + 1])).all())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tile_rows", [0, 8, 16, 64, 128])
@pytest.mark.parametrize("experts,top,tokens,hidden,inter,act", [(6, 2, 50, 72, 40, 1), (16, 4, 3, 64, 96, 1), (3, 3, 130, 40, 20, 2),
                                                                 (40, 1, 9, 32, 8, 0), (5, 2, 200, 328, 136, 1), (3, 1, 70, 100, 52, 1)])
def test_expert_rows_products_and_sum(K, dtype, experts, top, tokens, hidden, inter, act, tile_rows, monkeypatch):
    """(hidden 100 and inter 52 are multiples of 4 only: the bfloat16 engine takes the CUDA-core kernel there.)"""
    if tile_rows and dtype == torch.float32:
        pytest.skip("the 32-bit kernel has one tile size")
    monkeypatch.setattr(K, "expert_tile_rows", tile_rows)
    z = rand(tokens, experts + 1, seed=1, scale=2.0)
    if experts > 4:
        z[:, 1] = -50.0                                                      # an expert nobody chooses
    x = rand(tokens, hidden, dtype=dtype, seed=2)
    up, down = rand(experts, inter, hidden, dtype=dtype, seed=3, scale=hidden ** -0.5), rand(experts, hidden, inter, dtype=dtype, seed=4, scale=inter ** -0.5)
    shared = rand(tokens, hidden, dtype=dtype, seed=5)
    res = []
    for k_, d in ((K, DEV), (REF, "cpu")):
        chosen, weight = torch.empty(tokens, top, dtype=torch.int32, device=d), torch.empty(tokens, top, device=d)
        counts = torch.zeros(2 * experts + 1, dtype=torch.int32, device=d)
        k_.route_top(chosen, weight, counts, z.to(d), experts, 1.0, False)
        place, token_of = torch.empty(tokens * top, dtype=torch.int32, device=d), torch.empty(tokens * top, dtype=torch.int32, device=d)
        k_.expert_rows(place, token_of, counts, chosen, experts)
        starts = counts[experts:]
        hid = torch.empty(tokens * top, inter, dtype=dtype, device=d)
        k_.expert_linear(hid, x.to(d), token_of, up.to(d), starts, act)
        y = torch.empty(tokens * top, hidden, dtype=dtype, device=d)
        k_.expert_linear(y, hid, None, down.to(d), starts, 0)
        out = torch.empty(tokens, hidden, dtype=dtype, device=d)
        k_.expert_combine(out, y, place, weight, shared.to(d), z.to(d), experts)
        res.append((out, counts, place, token_of, chosen))
    (out, counts, place, token_of, chosen), (want, counts_w, _, _, _) = res
    assert torch.equal(counts.cpu(), counts_w)
    # every pair has a row of its own inside its expert's stretch, and the row knows its token
    place, token_of, starts = place.cpu().long(), token_of.cpu().long(), counts.cpu()[experts:].long()
    assert sorted(place.tolist()) == list(range(tokens * top))
    assert torch.equal(token_of[place], torch.arange(tokens * top) // top)
    e = chosen.cpu().long().reshape(-1)
    assert bool(((place >= starts[e]) & (place < starts[e + 1])).all())
    close(out, want, dtype, scale=8.0)
    if act == 1:                                                             # against the written-out mixture
        wd = {f"e{j}.up": up[j].double() for j in range(experts)} | {f"e{j}.down": down[j].double() for j in range(experts)}
        wd["router"] = torch.eye(experts, dtype=torch.float64)
        chosen_p, weight_p = plain.route(z[:, :experts].double(), wd, "", {"top": top, "scale": 1.0})
        ref = torch.zeros(tokens, hidden, dtype=torch.float64)
        for t in range(tokens):
            for j, g in zip(chosen_p[t].tolist(), weight_p[t]):
                ref[t] += g * plain.expert(x[t:t + 1].double(), wd, f"e{j}.")[0]
        ref += torch.sigmoid(z[:, experts:].double()) * shared.double()
        close(out, ref, dtype, scale=8.0 if dtype == torch.float32 else 16.0)


@pytest.mark.parametrize("experts,rows,n,k,act,gather", [(4, 700, 264, 136, 1, True), (3, 130, 512, 64, 0, False), (6, 40, 72, 328, 2, True),
                                                         (2, 1, 8, 8, 1, True), (9, 2000, 1408, 256, 1, False)])
def test_expert_products_on_tcgen05(K, experts, rows, n, k, act, gather, monkeypatch):
    """The prompt kernel at sizes that leave partial tiles everywhere: experts of 0 to hundreds of rows, widths that
    end inside a 256-column tile and inside a 64-wide k block, gathered rows and rows already in order."""
    monkeypatch.setattr(K, "expert_products", "tcgen05")
    g = torch.Generator().manual_seed(rows)
    cuts = torch.sort(torch.randint(0, rows + 1, (experts - 1,), generator=g)).values.tolist()
    if experts > 2:
        cuts[1] = cuts[0]                                                    # an expert without rows
    starts = torch.tensor([0, *cuts, rows], dtype=torch.int32)
    tokens = max(1, rows // 2)
    x = rand(tokens if gather else rows, k, dtype=torch.bfloat16, seed=1)
    token_of = torch.randint(0, tokens, (rows,), generator=g).to(torch.int32) if gather else None
    w = rand(experts, n, k, dtype=torch.bfloat16, seed=2, scale=k ** -0.5)
    out, want = torch.full((rows, n), 7.0, dtype=torch.bfloat16, device=DEV), torch.empty(rows, n, dtype=torch.bfloat16)
    K.expert_linear(out, x.to(DEV), token_of.to(DEV) if gather else None, w.to(DEV), starts.to(DEV), act)
    REF.expert_linear(want, x, token_of, w, starts, act)
    close(out, want, torch.bfloat16, scale=4.0)
    assert K.tcgen05_status() == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_gate_and_activation(K, dtype):
    o, wide = rand(13, 70, dtype=dtype, seed=1), rand(13, 200, dtype=dtype, seed=2)
    og = o.clone().to(DEV)
    K.sigmoid_gate(og, wide.to(DEV)[:, 50:120])
    want = o.clone()
    REF.sigmoid_gate(want, wide[:, 50:120])
    close(og, want, dtype)
    for act in (1, 2):
        xg, xw = o.clone().to(DEV), o.clone()
        K.activation(xg, act)
        REF.activation(xw, act)
        close(xg, xw, dtype, scale=2.0)


# ---------------------------------------------------------------- the replayer against the plain implementation
@pytest.fixture(scope="module", params=sorted(CONFIGS))
def model(request, tmp_path_factory):
    folder = make_folder(tmp_path_factory.mktemp("models"), request.param, seed=5)
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
def test_long_decoding_first_tokens_and_far_keys(model, dtype):
    folder, config, _, _ = model
    ids = random_prompt(config["vocab"], 330, 77)
    want = {"x": exact_logits(folder, ids)}
    r = Replayer(str(folder), dtype, max_tokens=384)
    got = run(r, [([("x", [t])], ["x"] if i == len(ids) - 1 else []) for i, t in enumerate(ids)])   # all one by one
    compare(got, want, dtype)
    compare({k: v for k, v in got.items() if k[1] < 4}, want, dtype)
    # a prompt of 260 tokens (past four page borders), then single tokens: the same rows
    got = run(r, [([("x", ids[:260])], [])] + [([("x", [t])], []) for t in ids[260:]])
    compare(got, want, dtype)


def test_a_repeated_token_far_back_is_found(tmp_path):
    """Attention must reach a key hundreds of tokens back: with the sharpened weights a query attends mostly to earlier
    occurrences of related tokens, so logits change visibly when one token 300 places back changes. The engine must
    follow the plain implementation through that change, in a prompt and in decoding."""
    folder = make_folder(tmp_path, "c", seed=11)
    ids = random_prompt(CONFIGS["c"]["vocab"], 320, 5)
    other = list(ids)
    other[7] = (ids[7] + 1) % CONFIGS["c"]["vocab"]
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
    _, weights = plain.read_folder(folder)
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
            logits = plain.forward(config, weights, ids)[-1]
            if float(logits.max() - logits[token]) > margin * float(logits.std()):
                off.append((len(ids), token, int(logits.argmax())))
            ids.append(token)
    # bfloat16: rounding may tip a router's close call and with it a token; never more than a few of the sixty
    assert len(off) <= (0 if dtype == "float32" else 4), off


def test_generate_on_the_command_line(tmp_path, capsys):
    """`holon-b200 generate` with the engine's own sizing of the cache (activation peaks measured on the largest step)."""
    import json

    from holon_b200 import cli
    folder = make_folder(tmp_path, "a", seed=8)
    config, weights = plain.read_folder(folder)
    assert cli.main(["generate", str(folder), "--prompt-ids", "5,17,3,90,12,7", "--prompt-ids", "9 8 7 6", "--max-tokens", "6",
                     "--dtype", "float32", "--max-model-len", "128", "--max-seqs", "4", "--max-step-tokens", "128", "--ignore-eos",
                     "--memory-fraction", "0.05"]) == 0
    captured = capsys.readouterr()
    assert "holon-b200: memory: weights" in captured.err and "cache pools" in captured.err
    lines = [json.loads(line) for line in captured.out.splitlines()]
    assert [o["prompt_ids"] for o in lines] == [[5, 17, 3, 90, 12, 7], [9, 8, 7, 6]]
    for o in lines:
        ids = list(o["prompt_ids"])
        assert len(o["token_ids"]) == 6
        for token in o["token_ids"]:
            logits = plain.forward(config, weights, ids)[-1]
            assert float(logits.max() - logits[token]) <= 1e-3 * float(logits.std()), (len(ids), token)
            ids.append(token)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_then_decoding(tmp_path, dtype):
    """700 tokens in one step (hundreds of rows an expert: the prompt kernels), cut in two portions at an odd place, and
    40 tokens one by one over eleven pages (the keys of a one-token row in parts), with a latent wider than 128."""
    folder = make_folder(tmp_path, "e", seed=4, config=RX_E)
    ids = random_prompt(RX_E["vocab"], 740, 21)
    exact = exact_logits(folder, ids)
    want = {"x": exact, "y": exact}
    r = Replayer(str(folder), dtype, max_tokens=1536)
    steps = [([("x", ids[:700])], [])] + [([("x", [t])], []) for t in ids[700:]]
    compare(run(r, steps), {"x": want["x"]}, dtype)
    steps = [([("y", ids[:333])], []), ([("y", ids[333:700]), ("x", ids[700:701])], [])] + [([("y", [t])], []) for t in ids[700:]]
    got = run(r, steps)
    compare({k: v for k, v in got.items() if k[0] == "y"}, {"y": want["y"]}, dtype)
