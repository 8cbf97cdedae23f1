"""The Netanex design on the GPU against its plain statement (tests/plain_netanex.py): every kernel it brought or
extended alone, then whole models of small sizes (tests/netanex_cases.py) through the step function, the cache, the
generation loop and the replay program."""
import copy
import io
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import bitnet_c_b200 as bn
import netanex_cases as nc
import plain_netanex as pn
from helpers import (BF16_GAP_FACTOR, TOL_F32, collect_trace_output, compare, random_tokens, replay, steps_to_jsonl,
                     trace_batches, trace_chunks, trace_tail, trace_whole)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _give_device_memory_back():
    """The models and caches of this module leave the allocator's pool when it is done."""
    yield
    import gc
    gc.collect()
    if torch.cuda.is_available():
        torch.cuda.empty_cache()


ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
bf = pn.to_bf16


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to("cuda", dtype)


def ints(a):
    return torch.tensor(list(a), dtype=torch.int32, device="cuda")


def _paged(lens, G, d, Gv, dv, t, k=None, v=None):
    """A paged cache for sequences of the given lengths in scattered pages (sequence s lives in slot s + 1);
    what nobody wrote is NaN and Inf.  With k, v ([sum(lens), G, d] and [.., Gv, dv]) the rows are written in."""
    pages = [(n + 63) // 64 for n in lens]
    order = np.random.default_rng(5).permutation(sum(pages) + 3)
    table = np.zeros((len(lens) + 2, max(pages)), dtype=np.int32)
    at = 0
    for s, p in enumerate(pages):
        table[s + 1, :p] = order[at:at + p]
        at += p
    kc = torch.full((sum(pages) + 3, G, 64, d), float("nan"), dtype=t, device="cuda")
    vc = torch.full((sum(pages) + 3, Gv, 64, dv), float("inf"), dtype=t, device="cuda") if Gv else None
    if k is not None:
        at = 0
        for s, n in enumerate(lens):
            for pos in range(n):
                page = int(table[s + 1, pos // 64])
                kc[page, :, pos % 64] = dev(k[at + pos], t)
                if vc is not None:
                    vc[page, :, pos % 64] = dev(v[at + pos], t)
            at += n
    return kc, vc, torch.from_numpy(table).cuda()


# ---- kernels alone -----------------------------------------------------------------------------------
PREP_SHAPES = [  # heads, key/value heads, key width, value width, maps, norm, coef, every
    (4, 2, 16, 24, 1, "whole", 0.0, 0), (6, 2, 8, 16, 2, "head", 0.8, 16), (3, 1, 10, 12, 2, "head", 1.5, 1),
    (3, 3, 10, 7, 1, "whole", 0.0, 0), (8, 4, 16, 32, 2, "head", 0.4, 50), (2, 2, 128, 64, 1, "none", 0.25, 7),
    (16, 2, 64, 128, 1, "whole", 0.0, 0), (5, 5, 6, 6, 1, "head", 0.0, 0),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", PREP_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_queries_keys_and_values_from_the_rows_of_their_projection(cuda_device, dtype, shape):
    """Bias, norms per head or over the whole projection, the factor by position, the rounding to the compute type
    and the rows in the pages, in one launch, against the plain functions."""
    from bitnet_c_b200.csrc import ops
    H, G, d, dv, maps, norm, coef, every = shape
    rng = np.random.default_rng(int(sum(x if isinstance(x, (int, float)) else len(x) for x in shape) * 8))
    t = DT[dtype]
    lens = [70, 3, 130]
    new = [6, 3, 67]
    q_len, k_len, v_len = H * maps * d, G * maps * d, G * dv
    row = q_len + k_len + v_len + 5  # five more columns ride along (gates)
    n = sum(new)
    src = rng.standard_normal((n, row)) * 2
    bias = rng.standard_normal(row) * 0.5
    bias[q_len + k_len + v_len:] = 0.0
    span_q = {"whole": q_len, "head": d, "none": 0}[norm]
    span_k = {"whole": k_len, "head": d, "none": 0}[norm]
    wq, wk = 1 + 0.3 * rng.standard_normal(max(span_q, 1)), 1 + 0.3 * rng.standard_normal(max(span_k, 1))
    pos = np.concatenate([np.arange(l - c, l) for l, c in zip(lens, new)])
    seq = np.concatenate([np.full(c, s) for s, c in enumerate(new)])
    x = src.astype(np.float32).astype(np.float64) + bias.astype(np.float32)
    want = x.copy()
    if span_q:
        want[:, :q_len] = pn.norm_plain(x[:, :q_len].reshape(n, -1, span_q), wq.astype(np.float32), 1e-5).reshape(n, q_len)
        want[:, q_len:q_len + k_len] = pn.norm_plain(x[:, q_len:q_len + k_len].reshape(n, -1, span_k), wk.astype(np.float32), 1e-5).reshape(n, k_len)
    if every:
        want[:, :q_len] *= np.array([pn.query_temperature(int(p), coef, every) for p in pos])[:, None]
    kc, vc, table = _paged(lens, G * maps, d, G, dv, t)
    out = torch.full((n, row), float("nan"), dtype=t, device="cuda")
    ops.qk_norm_append(dev(src), out, ints(pos), q_len=q_len, k_off=q_len, k_len=k_len, bias=dev(bias), q_span=span_q,
                       wq=dev(wq) if span_q else None, k_span=span_k, wk=dev(wk) if span_k else None, eps=1e-5, temp_coef=coef,
                       temp_every=every, v_off=q_len + k_len, n_kv_heads=G * maps, head_dim=d, n_v_heads=G, v_dim=dv,
                       tok_seq=ints(seq), slots=ints([1, 2, 3]), page_table=table, k_cache=kc, v_cache=vc)
    got = out.float().cpu().numpy()
    tol = 2e-5 if dtype == "float32" else 2.0 ** -8
    err = np.abs(got - want) / np.maximum(1.0, np.abs(want))
    assert np.isfinite(got).all() and err.max() < tol, f"column {int(err.max(axis=0).argmax())} off by {err.max():.3e}"
    tb = table.cpu().numpy()
    for r in (0, n // 2, n - 1):  # what the pages hold is what the row holds
        page, at = int(tb[seq[r] + 1, pos[r] // 64]), int(pos[r] % 64)
        assert torch.equal(kc[page, :, at].reshape(-1), out[r, q_len:q_len + k_len])
        assert torch.equal(vc[page, :, at].reshape(-1), out[r, q_len + k_len:q_len + k_len + v_len])
    assert torch.isnan(kc).any() and int((~torch.isnan(kc[:, 0, :, 0])).sum()) == n  # and nothing else was written


ATT_SHAPES = [  # query heads, key heads, key width, value width, window, key heads per value head, sink
    (4, 2, 16, 24, 0, 1, "zero"), (12, 4, 8, 16, 0, 2, None), (3, 1, 24, 7, 64, 1, "learned"), (6, 2, 10, 12, 0, 2, None),
    (16, 8, 16, 32, 0, 2, None), (4, 1, 32, 16, 0, 1, "zero"), (4, 1, 64, 48, 70, 1, "learned"), (2, 1, 56, 40, 150, 1, "learned"),
    (8, 2, 128, 128, 0, 1, "zero"), (16, 4, 64, 128, 0, 2, None), (8, 1, 256, 192, 129, 1, "learned"), (5, 5, 6, 6, 1, 1, "zero"),
    (6, 6, 48, 48, 33, 1, None), (32, 8, 32, 64, 0, 2, "learned"),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", ATT_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_attention_with_a_sink_and_shared_values_over_the_pages(cuda_device, dtype, shape):
    """Whole prompts, pieces behind cached tokens and single tokens (keys dealt out over several blocks or not), on
    the general kernel and, where the sizes fit it, on the tensor-core kernel for runs of tokens, with results in
    the compute type and in float32: the same rows as the plain softmax, with a sink that holds a good part of the
    weight, with one key planted just inside and one just outside the window of the last token of the longest
    sequence, and (without a window) one planted at the very first position, all with scores far above the rest
    and values that dwarf the others."""
    from bitnet_c_b200.csrc import ops
    H, G, d, dv, window, share, sink_kind = shape
    rng = np.random.default_rng(sum(x if isinstance(x, int) else len(str(x)) for x in shape))
    t = DT[dtype]
    lens = [200, 70, 5]
    T = sum(lens)
    Gv = G // share
    scale = 1.5 / np.sqrt(d)
    q, k = bf(rng.standard_normal((T, H, d))), bf(rng.standard_normal((T, G, d)))
    v = bf(rng.standard_normal((T, Gv, dv)))
    sink = {None: None, "zero": np.zeros(H), "learned": rng.standard_normal(H) * 2 + 3}[sink_kind]
    last = lens[0] - 1
    per = H // G
    if window > 1:
        for dist, val in ((window - 1, 40.0), (window, -1000.0)):  # inside: seen whole; outside: must not be seen
            if last - dist >= 0:
                k[last - dist] = bf(q[last].reshape(G, per, d)[:, 0] * 3.0)
                v[last - dist] = val
    elif window == 0:
        k[0] = bf(q[last].reshape(G, per, d)[:, 0] * 3.0)  # the farthest key there is
        v[0] = 40.0
    want = np.zeros((T, H * dv))
    at = 0
    for n in lens:
        for h in range(H):
            g = h // per
            want[at:at + n, h * dv:(h + 1) * dv] = pn.attend(q[at:at + n, h], k[at:at + n, g], v[at:at + n, g // share], scale, window,
                                                              None if sink is None else float(np.float32(sink[h])))
        at += n
    kc, vc, table = _paged(lens, G, d, Gv, dv, t, k, v)
    sk = dev(sink) if sink is not None else None
    tol = 2e-5 if dtype == "float32" else 2.0 ** -7
    starts = np.concatenate([[0], np.cumsum(lens)])
    for what, new in (("whole", lens), ("pieces", [66, 3, 5]), ("pieces of 17", [17, 17, 1]), ("single", [1, 1, 1])):
        rows = np.concatenate([np.arange(starts[s] + lens[s] - c, starts[s] + lens[s]) for s, c in enumerate(new)])
        pos = np.concatenate([np.arange(lens[s] - c, lens[s]) for s, c in enumerate(new)])
        seq = np.concatenate([np.full(c, s) for s, c in enumerate(new)])
        qd = dev(q.reshape(T, -1)[rows], t)
        ref = want[rows]

        def check(out, how):
            got = out.float().cpu().numpy()
            err = np.abs(got - ref).max(axis=1) / np.maximum(1.0, np.abs(ref).max(axis=1))
            assert np.isfinite(got).all() and err.max() < tol, \
                f"{what}, {how}: row {int(np.argmax(err))} (position {pos[int(np.argmax(err))]}) off by {err.max():.3e}"

        for max_keys in ((0, 100000) if what == "single" else (0,)):
            for wide in (False, True):
                out = torch.full((len(rows), H * dv), float("nan"), dtype=torch.float32 if wide else t, device="cuda")
                ops.attention_general(qd, qd.shape[1], out, len(rows), H, G, d, scale, window, ints(seq), ints(pos), ints([1, 2, 3]),
                                      table, kc, vc, sink=sk, v_share=share, max_keys=max_keys)
                check(out, f"general kernel, max_keys {max_keys}, float32 out {wide}")
        if dtype != "bfloat16" or d % 16 or dv % 16 or d > 256 or dv > 256:
            continue
        tiles = [(s_, r) for s_, c_ in enumerate(new) for r in range(0, c_, 64)]
        for wide in (False, True):
            out = torch.full((len(rows), H * dv), float("nan"), dtype=torch.float32 if wide else t, device="cuda")
            ops.attention_prefill(qd, qd.shape[1], out, H, G, d, scale, window, ints(s_ for s_, _ in tiles), ints(r for _, r in tiles),
                                  ints(np.concatenate([[0], np.cumsum(new)])), ints(l - c_ for l, c_ in zip(lens, new)), ints([1, 2, 3]),
                                  table, kc, vc, precise=True, sink=sk, v_share=share)
            check(out, f"runs of tokens, float32 out {wide}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_maps_combined_gates_on_rows_experts_by_table_and_the_rotation_of_halves(cuda_device, dtype):
    from bitnet_c_b200.csrc import ops
    t = DT[dtype]
    rng = np.random.default_rng(3)
    tol = 2e-5 if dtype == "float32" else 2.0 ** -7
    # a1 - lambda a2 over maps laid out [group][map][head in group], unit norm, factor
    for H, G, dv, lam, post in ((6, 2, 16, 0.7, 0.65), (3, 1, 12, -0.4, 0.2), (8, 8, 40, 1.3, 0.5), (4, 1, 128, 0.8, 0.4)):
        n, per = 37, H // G
        maps = rng.standard_normal((n, G, 2, per, dv)).astype(np.float32)
        o = maps[:, :, 0].astype(np.float64) - np.float32(lam) * maps[:, :, 1]
        want = (pn.rms(o, 1e-5) * post).reshape(n, H * dv)
        out = torch.full((n, H * dv), float("nan"), dtype=t, device="cuda")
        ops.diff_combine(dev(maps.reshape(n, -1)), out, H, per, dv, lam, 1e-5, post)
        assert np.abs(out.float().cpu().numpy() - want).max() < tol * 4
    # an output gate on every number, on views into wider rows
    x, g = bf(rng.standard_normal((19, 50))), bf(2 * rng.standard_normal((19, 70)))
    xd, gd = dev(x, t), dev(g, t)
    ops.gate_rows(xd[:, 3:45], gd[:, 11:53])
    want = x.copy()
    want[:, 3:45] *= pn.sigmoid(g[:, 11:53])
    assert np.abs(xd.float().cpu().numpy() - want).max() < tol * 4
    # experts by token id
    table = np.stack([rng.permutation(7)[:3] for _ in range(20)]).astype(np.int32)
    toks = rng.integers(0, 20, size=33)
    ids, wts = ops.moe_table_route(ints(toks), torch.from_numpy(table).cuda(), 3, 7)
    assert np.array_equal(ids.cpu().numpy(), table[toks]) and torch.all(wts == np.float32(1.0 / 3.0))
    ids, wts = ops.moe_table_route(ints(toks), torch.from_numpy(table).cuda(), 2, 7)  # fewer than the table's columns
    assert np.array_equal(ids.cpu().numpy(), table[toks][:, :2]) and torch.all(wts == 0.5)
    # rotation of number i with number i + dims / 2, cos and sin times a magnitude, inside wider heads
    for dims, base, sc in ((8, 10000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}), (6, 500.0, None), (64, 1e6, {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0})):
        n, Hq, plain_part = 23, 3, 10
        f, mag = pn.yarn_frequencies(dims, base, sc)
        pos = rng.integers(0, 3000, size=n)
        x = bf(rng.standard_normal((n, Hq, plain_part + dims)))
        want = x.copy()
        a = pos[:, None].astype(np.float64) * f.astype(np.float32)[None, :].astype(np.float64)
        want[:, :, plain_part:] = pn.rotate_half(x[:, :, plain_part:], pos, dims, base, sc)
        xd = dev(x.reshape(n, -1), t)
        ops.rotary_pairs_append(xd, dev(f), ints(pos), q_off=0, n_q_heads=Hq, q_head_stride=plain_part + dims, q_rot_off=plain_part,
                                split_halves=True, magnitude=mag)
        err = np.abs(xd.float().cpu().numpy().reshape(want.shape) - want).max()
        assert err < (2e-3 if dtype == "float32" else 3e-2), f"dims {dims}: {err:.3e}"  # angles of thousands of radians in float32


# ---- whole models --------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, cfg in nc.CASES.items():
        w = nc.draw_weights(cfg, seed=21)
        out[name] = (nc.write_folder(str(tmp_path_factory.mktemp("netanex") / name), cfg, w), w)
    return out


_ROUNDED = {}


def _plain_rounded(cfg, w, tokens):
    key = (json.dumps(cfg, sort_keys=True), id(w), tuple(tokens))
    if key not in _ROUNDED:
        _ROUNDED[key] = pn.forward(tokens, w, cfg, r=pn.to_bf16)
    return _ROUNDED[key]


def _check(got, cfg, w, reqs, plain, dtype, what):
    """float32: every position within 1e-4 of the plain logits (relative to the largest).  bfloat16: the bound of a
    request is three times what rounding the stored activations does to the plain statement, taken at the request's
    80th percentile of positions; at most a fifth of a request's positions may lie beyond it, none beyond three
    times the largest gap."""
    for r, per_pos in got.items():
        assert all(np.isfinite(row).all() for row in per_pos.values()), f"{what}: request {r}"
    if dtype == "float32":
        return compare(got, plain, lambda ref: TOL_F32 * max(1.0, float(np.abs(ref).max())), what)
    for r, per_pos in got.items():
        gap = np.abs(plain[r] - _plain_rounded(cfg, w, reqs[r])).max(axis=1)[sorted(per_pos)]
        bound = BF16_GAP_FACTOR * float(np.percentile(gap, 80))
        assert bound < 0.1 * float(np.abs(plain[r]).max()), "the test model is too rough for bfloat16"
        err = np.array([np.abs(row.astype(np.float64) - plain[r][p]).max() for p, row in sorted(per_pos.items())])
        assert err.max() <= BF16_GAP_FACTOR * float(gap.max()), f"{what}: request {r}: position {sorted(per_pos)[int(err.argmax())]}"
        beyond = int((err > bound).sum())
        assert beyond <= max(1, len(err) // 5), (f"{what}: request {r}: {beyond} of {len(err)} positions beyond {bound:.3e}; "
                                                 f"first at {sorted(per_pos)[int(np.argmax(err > bound))]}")


def _poison(cache):
    """Pages that nobody holds may contain anything."""
    for g in cache.groups:
        g.k.fill_(float("nan"))
        if g.v is not None:
            g.v.fill_(float("inf"))


@pytest.mark.parametrize("case", sorted(nc.CASES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_models_step_like_the_plain_statement_however_the_tokens_are_cut(folders, cuda_device, case, dtype):
    cfg = nc.CASES[case]
    d, w = folders[case]
    V = cfg["vocab"]
    reqs = {"a": random_tokens(1, 210, V), "b": random_tokens(2, 3, V), "c": random_tokens(3, 77, V), "d": random_tokens(4, 131, V)}
    plain = {r: pn.forward(t, w, cfg) for r, t in reqs.items()}
    model = bn.load_model(d, dtype=dtype)
    cache = model.new_cache(max_tokens=64 * 12, max_seqs=4)
    _poison(cache)
    schedules = (
        ("whole", trace_whole(reqs)),
        ("every token alone", trace_tail({"c": reqs["c"], "b": reqs["b"]}, 1000)),
        ("150 tokens decoded one by one", trace_tail({"a": reqs["a"]}, 150)),
        ("pieces down to two tokens", trace_chunks(reqs, pieces=(2, 1, 5, 64, 33))),
        ("pieces of a page and around it", trace_chunks({"a": reqs["a"], "d": reqs["d"]}, pieces=(63, 1, 64, 65), stagger=2)),
        ("unequal batches, slots and pages used again",
         trace_batches([{"a": (reqs["a"], 40), "b": (reqs["b"], 2), "c": (reqs["c"], 9)},
                        {"d": (reqs["d"], 70), "b": (reqs["b"], 1)}, {"c": (reqs["c"], 76), "a": (reqs["a"], 3)}])),
    )
    for what, steps in schedules:
        _check(replay(model, cache, steps), cfg, w, reqs, plain, dtype, f"case {case}, {what}, {dtype}")
        assert cache.slots.n_free == cache.slots.n_slots
    model.check_kernels()


def test_the_stream_after_every_layer_is_the_plain_statements(folders, cuda_device):
    for case in sorted(nc.CASES):
        cfg = nc.CASES[case]
        d, w = folders[case]
        toks = random_tokens(9, 90, cfg["vocab"])
        want = []
        pn.forward(toks, w, cfg, taps=want)
        model = bn.load_model(d, dtype="float32")
        diag = model.diagnostics = bn.Diagnostics(dump_tag="lout", keep=True, out=io.StringIO())
        cache = model.new_cache(max_tokens=256, max_seqs=1)
        slot = cache.open()
        model.step(cache, [bn.SeqStep(slot, toks, [len(toks) - 1])])
        cache.close(slot)
        for i, ref in enumerate(want):
            for pos in (0, 1, 40, 89):
                (got,) = [r["values"] for r in diag.records if (r["tag"], r["layer"], r["pos"]) == ("lout", i, pos)]
                assert np.abs(got - ref[pos]).max() < 1e-4 * max(1.0, np.abs(ref[pos]).max()), f"case {case}, after layer {i}, position {pos}"


@pytest.mark.parametrize("case", ["A", "C"])
def test_a_request_alone_and_in_a_batch_give_the_same_logits(folders, cuda_device, case):
    cfg = nc.CASES[case]
    d, _w = folders[case]
    V = cfg["vocab"]
    reqs = {"a": random_tokens(11, 100, V), "b": random_tokens(12, 7, V), "c": random_tokens(13, 160, V)}
    model = bn.load_model(d, dtype="float32")
    cache = model.new_cache(max_tokens=64 * 10, max_seqs=3)
    alone = replay(model, cache, trace_whole(reqs))
    together = replay(model, cache, trace_batches([{r: (t, min(12, len(t) - 1)) for r, t in reqs.items()}]))
    for r in reqs:
        for p, row in together[r].items():
            assert np.abs(row - alone[r][p]).max() < 1e-5 * max(1.0, np.abs(row).max()), f"request {r}, position {p}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_and_long_decoding_far_past_every_window(folders, cuda_device, dtype):
    cfg = nc.CASE_C
    d, w = folders["C"]
    toks = random_tokens(17, 1400, cfg["vocab"])
    plain = {"x": pn.forward(toks, w, cfg)}
    model = bn.load_model(d, dtype=dtype)
    cache = model.new_cache(max_tokens=1536, max_seqs=1)
    _poison(cache)
    steps = trace_tail({"x": toks}, 300)
    # of the prompt, logits at the edges of pages and windows and at its end only, to keep the test quick
    steps[0]["entries"][0]["want"] = [0, 63, 64, 69, 70, 71, 149, 150, 151, 1023, 1024, 1099]
    got = replay(model, cache, steps)
    _check(got, cfg, w, {"x": toks}, plain, dtype, f"1,100 tokens and 300 more one by one, {dtype}")
    # the windowed planes gave their pages back as the sequence grew
    assert cache.slots.n_free == cache.slots.n_slots


EDGES = {
    "one head, one expert, no window": [
        {"type": "attention_2", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.7},
         "mlp": {"kind": "moe", "router": {"experts": 1, "top": 1}, "expert": {"ff": 8}}},
        {"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.7, "diff": 0.0}, "mlp": None},
        {"type": "latent_attention", "mixer": {"heads": 1, "dim": 8, "rot_dim": 2, "vdim": 8, "kv_rank": 8, "scale": 0.6,
                                               "rot": {"base": 10.0, "dims": 2}}, "mlp": None}],
    "windows of one and two positions": [
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 8, "kv_rank": 12, "scale": 0.6,
                                               "mask": {"size": 1}, "rot": {"base": 100.0, "dims": 4}},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 8}}},
        {"type": "latent_attention", "mixer": {"heads": 4, "dim": 4, "rot_dim": 8, "vdim": 4, "kv_rank": 24, "scale": 0.6,
                                               "mask": {"size": 2}, "rot": {"base": 100.0, "dims": 8,
                                                                            "scaling": {"factor": 1.0, "original": 16, "fast": 2.0, "slow": 1.0}}},
         "mlp": None}],
    "one layer's weights for every layer": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 8, "vdim": 4, "scale": 0.6, "diff": 0.9,
                                        "q_temp": {"coef": 2.0, "every": 3}},
         "mlp": {"kind": "moe", "router": {"experts": 40, "top": 1}, "expert": {"ff": 8}}}] + [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 8, "vdim": 4, "scale": 0.6, "diff": 0.9,
                                        "q_temp": {"coef": 2.0, "every": 3}},
         "mlp": {"kind": "moe", "router": {"experts": 40, "top": 1}, "expert": {"ff": 8}}, "weights_of": 0}] * 3,
    "shared weights under constants of their own": [
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 8, "vdim": 8, "kv_rank": 16, "scale": 0.5,
                                               "mask": {"size": 40}, "rot": {"base": 100.0, "dims": 8}},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 8}}},
        {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 8, "vdim": 8, "kv_rank": 16, "scale": 0.3,
                                               "mask": {"size": 7}, "rot": {"base": 100.0, "dims": 4}},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 2}, "expert": {"ff": 8}}, "weights_of": 0},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.6, "diff": 0.3}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.6, "diff": 0.7,
                                        "q_temp": {"coef": 1.0, "every": 9}}, "mlp": None, "weights_of": 2}],
    "all experts for every token": [
        {"type": "attention_2", "mixer": {"heads": 8, "kv_heads": 1, "dim": 4, "vdim": 12, "scale": 0.9},
         "mlp": {"kind": "moe", "router": {"experts": 6, "top": 6}, "expert": {"ff": 12}}}],
}


@pytest.mark.parametrize("kind", sorted(EDGES))
def test_models_at_the_edges_of_what_the_configuration_allows(tmp_path, cuda_device, kind):
    cfg = {"architecture": "Netanex", "vocab": 53, "width": 32, "norm": {"eps": 1e-6}, "layers": EDGES[kind]}
    w = nc.draw_weights(cfg, seed=8)
    d = nc.write_folder(str(tmp_path / "m"), cfg, w)
    reqs = {"a": random_tokens(1, 140, 53), "b": random_tokens(2, 1, 53), "c": random_tokens(3, 66, 53)}
    plain = {r: pn.forward(t, w, cfg) for r, t in reqs.items()}
    for dtype in ("float32", "bfloat16"):
        model = bn.load_model(d, dtype=dtype)
        cache = model.new_cache(max_tokens=64 * 8, max_seqs=3)
        _poison(cache)
        for what, steps in (("whole", trace_whole(reqs)), ("pieces", trace_chunks(reqs, pieces=(2, 31, 1, 64))),
                            ("batch", trace_batches([{"a": (reqs["a"], 30), "b": (reqs["b"], 0), "c": (reqs["c"], 65)}]))):
            _check(replay(model, cache, steps), cfg, w, reqs, plain, dtype, f"{kind}, {what}, {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wider_model_with_heads_of_128_and_latent_rows_beyond_256(tmp_path, cuda_device, dtype):
    cfg = {"architecture": "Netanex", "vocab": 200, "width": 256, "norm": {"eps": 1e-6}, "layers": [
        {"type": "attention_2", "mixer": {"heads": 8, "kv_heads": 1, "dim": 128, "vdim": 64, "scale": 0.15},
         "mlp": {"kind": "moe", "router": {"experts": 4, "top": 2}, "expert": {"ff": 96}}},
        {"type": "latent_attention", "mixer": {"heads": 4, "dim": 64, "rot_dim": 64, "vdim": 128, "kv_rank": 320, "scale": 0.1,
                                               "mask": {"size": 100},
                                               "rot": {"base": 1e6, "dims": 64,
                                                       "scaling": {"factor": 16.0, "original": 256, "fast": 32.0, "slow": 1.0}}},
         "mlp": None},
        {"type": "attention", "mixer": {"heads": 8, "kv_heads": 8, "dim": 64, "vdim": 128, "scale": 0.2, "diff": 0.4,
                                        "q_temp": {"coef": 0.2, "every": 64}},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 1}, "expert": {"ff": 160}}}]}
    w = nc.draw_weights(cfg, seed=12)
    d = nc.write_folder(str(tmp_path / "m"), cfg, w)
    reqs = {"a": random_tokens(5, 260, 200), "b": random_tokens(6, 40, 200)}
    plain = {r: pn.forward(t, w, cfg) for r, t in reqs.items()}
    model = bn.load_model(d, dtype=dtype)
    cache = model.new_cache(max_tokens=64 * 8, max_seqs=2)
    _poison(cache)
    for what, steps in (("whole", trace_whole(reqs)), ("pieces", trace_chunks(reqs, pieces=(70, 1, 33))),
                        ("batch", trace_batches([{"a": (reqs["a"], 20), "b": (reqs["b"], 8)}]))):
        _check(replay(model, cache, steps), cfg, w, reqs, plain, dtype, f"wider model, {what}, {dtype}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point_and_the_replay_program(folders, cuda_device, tmp_path, dtype):
    cfg = nc.CASE_A
    d, w = folders["A"]
    V = cfg["vocab"]
    model = bn.load_model(d, dtype=dtype)
    prompts = [random_tokens(31, 50, V), random_tokens(32, 3, V), random_tokens(33, 120, V)]
    got = bn.generate(model, prompts, max_new_tokens=[70, 20, 24])
    for p, g in zip(prompts, got):
        assert len(g.tokens) in (70, 20, 24) and g.finish_reason == "length"
        seq = list(p) + g.tokens[:-1]
        ref = pn.forward(seq, w, cfg)[len(p) - 1:]
        if dtype == "float32":
            slack = 2 * TOL_F32 * max(1.0, float(np.abs(ref).max()))
        else:
            slack = 2 * BF16_GAP_FACTOR * float(np.abs(pn.forward(seq, w, cfg, r=pn.to_bf16)[len(p) - 1:] - ref).max())
        off = [i for i, t in enumerate(g.tokens) if ref[i, t] < ref[i].max() - slack]
        assert not off, f"tokens {off[:5]} of a prompt of {len(p)} are not the plain statement's"
    # a second call on the same model: slots and pages are used again
    again = bn.generate(model, prompts[::-1], max_new_tokens=[24, 20, 70])
    assert [g.tokens for g in again[::-1]] == [g.tokens for g in got]
    reqs = {"x": prompts[0] + got[0].tokens, "y": prompts[1]}
    steps = trace_tail(reqs, 6)
    out = str(tmp_path / "out")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", out,
                        "--max-tokens", "256"], input=steps_to_jsonl(steps), capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    plain = {k: pn.forward(t, w, cfg) for k, t in reqs.items()}
    _check(collect_trace_output(steps, out, V), cfg, w, reqs, plain, dtype, "through bin/trace_run")


def test_the_command_line_writes_a_random_model_of_the_design_and_generates_from_it(tmp_path, cuda_device):
    cfgp = tmp_path / "cfg.json"
    cfgp.write_text(json.dumps(nc.CASE_C))
    folder = tmp_path / "m"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "bitnet"), str(folder), "--random-weights", "--config", str(cfgp),
           "--weight-seed", "3", "--dtype", "float32", "--prompt-token-ids", "5,17,3,9,9,1", "--prompt-token-ids", "7",
           "-n", "9", "--repeat-penalty", "1.0", "--token-ids"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [[int(t) for t in l.split(",")] for l in p.stdout.splitlines() if l.strip()]
    assert [len(l) for l in lines] == [9, 9] and "Generation complete tokens=18" in p.stderr
