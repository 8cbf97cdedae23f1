"""The Mekevik design on the GPU against its plain statement (tests/plain_mekevik.py): every kernel it brought
alone, then whole models of small sizes (tests/mekevik_cases.py) through the step function, the cache, the
generation loop and the replay program."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import bitnet_c_b200 as bn
import mekevik_cases as mc
import plain_mekevik as pm
from helpers import (BF16_GAP_FACTOR, TOL_F32, collect_trace_output, compare, random_tokens, replay, steps_to_jsonl,
                     trace_batches, trace_chunks, trace_tail, trace_whole)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def _give_device_memory_back():
    """The models and caches of this module leave the allocator's pool when it is done."""
    yield
    import gc
    import torch as _torch
    gc.collect()
    if _torch.cuda.is_available():
        _torch.cuda.empty_cache()
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
bf = pm.to_bf16


def dev(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to("cuda", dtype)


def ints(a):
    return torch.tensor(list(a), dtype=torch.int32, device="cuda")


def _paged(lens, G, d, dv, t, k=None, v=None):
    """A paged cache for sequences of the given lengths in scattered pages (sequence s lives in slot s + 1);
    what nobody wrote is NaN and Inf.  With k, v ([sum(lens), G, d] and [.., G, dv]) the rows are written in."""
    pages = [(n + 63) // 64 for n in lens]
    order = np.random.default_rng(5).permutation(sum(pages) + 3)
    table = np.zeros((len(lens) + 2, max(pages)), dtype=np.int32)
    at = 0
    for s, p in enumerate(pages):
        table[s + 1, :p] = order[at:at + p]
        at += p
    kc = torch.full((sum(pages) + 3, G, 64, d), float("nan"), dtype=t, device="cuda")
    vc = torch.full((sum(pages) + 3, G, 64, dv), float("inf"), dtype=t, device="cuda")
    if k is not None:
        at = 0
        for s, n in enumerate(lens):
            for pos in range(n):
                page = int(table[s + 1, pos // 64])
                kc[page, :, pos % 64] = dev(k[at + pos], t)
                vc[page, :, pos % 64] = dev(v[at + pos], t)
            at += n
    return kc, vc, torch.from_numpy(table).cuda()


def _distance_table(rel, pb, bias_max):
    """The bias of every distance 0 .. bias_max by the plain bucket function, the heads' own biases added in."""
    B = rel.shape[0]
    return np.stack([rel[pm.distance_bucket(n, B, bias_max)] + pb for n in range(bias_max + 1)])


# ---- kernels alone -----------------------------------------------------------------------------------
ATT_SHAPES = [  # heads, key/value heads, key width, value width, window, bias buckets, bias_max
    (4, 2, 16, 24, 37, 16, 30), (6, 2, 8, 24, 64, 32, 50), (3, 3, 10, 12, 30, 10, 40), (8, 2, 32, 16, 150, 32, 120),
    (5, 1, 6, 7, 0, 20, 100), (2, 2, 64, 32, 1, 6, 20), (16, 4, 64, 64, 129, 32, 300), (4, 1, 128, 128, 65, 8, 70),
    (6, 2, 16, 48, 37, 16, 30), (8, 1, 16, 16, 100, 12, 90), (8, 8, 32, 32, 70, 32, 500), (24, 8, 80, 112, 0, 32, 64), (10, 2, 96, 16, 64, 4, 3),
    (16, 2, 128, 64, 90, 32, 200), (8, 8, 128, 128, 130, 16, 64), (32, 8, 64, 128, 200, 32, 128), (7, 1, 112, 48, 33, 6, 40),
    (8, 4, 32, 64, 77, 16, 100), (16, 8, 16, 16, 140, 32, 90), (12, 4, 48, 32, 0, 8, 30), (4, 4, 64, 16, 64, 32, 64),
    (6, 3, 16, 16, 50, 8, 40), (5, 5, 32, 16, 20, 8, 40), (12, 6, 16, 32, 90, 16, 70), (7, 7, 16, 16, 33, 6, 40),  # clusters of 3, 5, 6, 7 blocks
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", ATT_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_attention_without_a_softmax_over_the_pages(cuda_device, dtype, shape):
    """Whole prompts, pieces behind cached tokens, and single tokens (keys dealt out over several blocks or not),
    on the general kernel and, where the sizes fit it, on the tensor-core kernel for runs of tokens: the same
    rows as the plain weights, with one key planted just inside and one just outside the window of the
    last token of the longest sequence, both with scores far above the rest and values that dwarf the others."""
    from bitnet_c_b200.csrc import ops
    H, G, d, dv, window, B, bias_max = shape
    rng = np.random.default_rng(sum(shape))
    t = DT[dtype]
    lens = [200, 70, 5]
    T = sum(lens)
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": 1.0 / np.sqrt(d), "bias_max": bias_max, "mask": {"size": window}}
    w = {"rel": bf(rng.standard_normal((B, H))), "pb": bf(rng.standard_normal(H) - 1.5),
         "talk": bf(np.eye(H) * 0.6 + 0.4 * rng.standard_normal((H, H)))}
    q, k = bf(rng.standard_normal((T, H, d))), bf(rng.standard_normal((T, G, d)))
    v, gate = bf(rng.standard_normal((T, G, dv))), bf(2 * rng.standard_normal((T, H * dv)))
    last = lens[0] - 1
    if window > 1:
        for dist, val in ((window - 1, 40.0), (window, -1000.0)):  # inside: seen whole; outside: must not be seen
            if last - dist >= 0:
                k[last - dist] = bf(q[last].reshape(G, H // G, d)[:, 0] * 8.0)
                v[last - dist] = val
    want = np.zeros((T, H * dv))
    at = 0
    for n in lens:
        a = pm.attention_weights(q[at:at + n], k[at:at + n], w, "", m)
        for h in range(H):
            want[at:at + n, h * dv:(h + 1) * dv] = a[h] @ v[at:at + n, h // (H // G)]
        at += n
    want *= pm.sigmoid(gate)
    kc, vc, table = _paged(lens, G, d, dv, t, k, v)
    rel = dev(_distance_table(w["rel"], w["pb"], bias_max))
    talk = dev(w["talk"])
    tol = 2e-5 if dtype == "float32" else 2.0 ** -7
    starts = np.concatenate([[0], np.cumsum(lens)])
    for what, new in (("whole", lens), ("pieces", [66, 3, 5]), ("pieces of 17", [17, 17, 1]), ("single", [1, 1, 1])):
        rows = np.concatenate([np.arange(starts[s] + lens[s] - c, starts[s] + lens[s]) for s, c in enumerate(new)])
        pos = np.concatenate([np.arange(lens[s] - c, lens[s]) for s, c in enumerate(new)])
        seq = np.concatenate([np.full(c, s) for s, c in enumerate(new)])
        qd, gd = dev(q.reshape(T, -1)[rows], t), dev(gate[rows], t)
        for max_keys in ((0, 100000) if what == "single" else (0,)):
            out = torch.full((len(rows), H * dv), float("nan"), dtype=t, device="cuda")
            ops.sigmoid_attention(qd, qd.shape[1], out, len(rows), H, G, d, m["scale"], window, ints(seq), ints(pos), ints([1, 2, 3]),
                                  table, kc, vc, rel=rel, mix=talk, gate=gd, gate_stride=gd.shape[1], max_keys=max_keys)
            got = out.float().cpu().numpy()
            ref = want[rows]
            err = np.abs(got - ref).max(axis=1) / np.maximum(1.0, np.abs(ref).max(axis=1))
            assert np.isfinite(got).all() and err.max() < tol, f"{what}: row {int(np.argmax(err))} (position {pos[int(np.argmax(err))]}) off by {err.max():.3e}"
        if dtype != "bfloat16" or not ops.sigmoid_attention_prefill_fits(H, G, d, dv):
            assert dtype != "bfloat16" or d % 16 or dv % 16, "these sizes should fit the kernel for runs of tokens"
            continue
        tiles = [(s_, r) for s_, c_ in enumerate(new) for r in range(0, c_, 64)]
        for splits in ((1, 2, 5) if what == "single" else (1,)):  # single tokens also with their pages dealt out over clusters
            out = torch.full((len(rows), H * dv), float("nan"), dtype=t, device="cuda")
            ops.sigmoid_attention_prefill(qd, qd.shape[1], out, H, G, d, m["scale"], window, ints(s_ for s_, _ in tiles),
                                          None if splits > 1 else ints(r for _, r in tiles), ints(np.concatenate([[0], np.cumsum(new)])),
                                          ints(l - c_ for l, c_ in zip(lens, new)), ints([1, 2, 3]), table, kc, vc, rel=rel, mix=talk, gate=gd,
                                          gate_stride=gd.shape[1], splits=splits)
            got = out.float().cpu().numpy()
            err = np.abs(got - want[rows]).max(axis=1) / np.maximum(1.0, np.abs(want[rows]).max(axis=1))
            assert np.isfinite(got).all() and err.max() < tol, \
                f"{what}, runs of tokens, {splits} splits: row {int(np.argmax(err))} (position {pos[int(np.argmax(err))]}) off by {err.max():.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_plain_heads_without_mixing_bias_or_gate_run_on_the_same_kernel(cuda_device, dtype):
    """Every option of the mixer's kernel is a parameter: without a mixing matrix, a bias table or a gate the rows
    are sums of logistic weights times values."""
    from bitnet_c_b200.csrc import ops
    H, G, d, dv, n = 4, 2, 16, 16, 90
    rng = np.random.default_rng(3)
    t = DT[dtype]
    q, k, v = bf(rng.standard_normal((n, H, d))), bf(rng.standard_normal((n, G, d))), bf(rng.standard_normal((n, G, dv)))
    kc, vc, table = _paged([n], G, d, dv, t, k, v)
    out = torch.empty((n, H * dv), dtype=t, device="cuda")
    qd = dev(q.reshape(n, -1), t)
    ops.sigmoid_attention(qd, H * d, out, n, H, G, d, 0.3, 20, ints([0] * n), ints(range(n)), ints([1]), table, kc, vc)
    i, j = np.arange(n)[:, None], np.arange(n)[None, :]
    seen = (i >= j) & (i - j < 20)
    for h in range(H):
        a = np.where(seen, pm.sigmoid(q[:, h] @ k[:, h // 2].T * 0.3), 0.0)
        ref = a @ v[:, h // 2]
        got = out[:, h * dv:(h + 1) * dv].float().cpu().numpy()
        assert np.abs(got - ref).max() < (2e-5 if dtype == "float32" else 2.0 ** -7) * np.abs(ref).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 16, 24), (3, 3, 10, 12), (5, 1, 6, 7), (8, 2, 32, 16)])
def test_norms_over_whole_projections_the_blend_and_the_cache_in_one_launch(cuda_device, dtype, H, G, d, dv):
    from bitnet_c_b200.csrc import ops
    rng = np.random.default_rng(H * 10 + d)
    t = DT[dtype]
    lens, new = [70, 5, 130], [3, 5, 66]
    T = sum(new)
    pos = np.concatenate([np.arange(n - c, n) for n, c in zip(lens, new)])
    seq = np.concatenate([np.full(c, i) for i, c in enumerate(new)])
    nq, nk, nv = H * d, G * d, G * dv
    row = nq + nk + nv + 5
    x = bf(rng.standard_normal((T, row)) * 3)
    wq, wk = bf(1 + 0.3 * rng.standard_normal(nq)), bf(1 + 0.3 * rng.standard_normal(nk))
    other = bf(rng.standard_normal((T, nv + 3)))
    for lam in (None, 0.3125):
        xd = dev(x, t)
        kc, vc, table = _paged(lens, G, d, dv, t)
        ops.slice_norm_append(xd, nq, dev(wq, t), nq, dev(wk, t), nq + nk, G, d, dv, 1e-5,
                              v_other=None if lam is None else dev(other, t)[:, :nv], blend=lam or 0.0, tok_seq=ints(seq), tok_pos=ints(pos),
                              slots=ints([1, 2, 3]), page_table=table, k_cache=kc, v_cache=vc)
        r = bf if dtype == "bfloat16" else (lambda a: a)
        qn, kn = pm.rms_norm(x[:, :nq], wq, 1e-5), pm.rms_norm(x[:, nq:nq + nk], wk, 1e-5)
        vn = x[:, nq + nk:nq + nk + nv] if lam is None else (1 - lam) * x[:, nq + nk:nq + nk + nv] + lam * other[:, :nv]
        got = xd.float().cpu().numpy()
        tol = 2e-6 if dtype == "float32" else 2.0 ** -7
        assert np.abs(got[:, :nq] - qn).max() < tol * np.abs(qn).max() and np.abs(got[:, nq:nq + nk] - kn).max() < tol * np.abs(kn).max()
        assert np.array_equal(got[:, nq + nk + nv:], x[:, nq + nk + nv:])  # what lies behind the slices stays
        for i in range(T):
            page = int(table[seq[i] + 1, pos[i] // 64])
            assert np.abs(kc[page, :, pos[i] % 64].float().cpu().numpy().ravel() - kn[i]).max() < tol * np.abs(kn).max()
            assert np.abs(vc[page, :, pos[i] % 64].float().cpu().numpy().ravel() - r(vn[i])).max() < tol * np.abs(vn).max()
        assert int(torch.isfinite(kc.float()).sum()) == T * nk  # nothing else was written


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_clamped_unit_and_the_routers_softmax_scores(cuda_device, dtype):
    from bitnet_c_b200.csrc import ops
    rng = np.random.default_rng(8)
    t = DT[dtype]
    n, inter = 9, 21
    h = bf(rng.standard_normal((n, 2 * inter)) * 3)
    out = torch.empty((n, inter), dtype=t, device="cuda")
    ops.glu_limited(dev(h, t), out, 1.25, 1.702)
    g, u = np.minimum(h[:, :inter], 1.25), np.clip(h[:, inter:], -1.25, 1.25)
    ref = g * pm.sigmoid(1.702 * g) * (u + 1)
    assert np.abs(out.float().cpu().numpy() - ref).max() < (2e-6 if dtype == "float32" else 2.0 ** -7) * np.abs(ref).max()
    # the experts' unit on rows of [gate | up], number by number and in 16-byte pieces
    for inter2 in (21, 24, 200):
        h2 = bf(rng.standard_normal((n, 2 * inter2)) * 3)
        out2 = torch.empty((n, inter2), dtype=t, device="cuda")
        ops.glu_halves(dev(h2, t), out2, ops.ACTIVATIONS["silu"])
        ref2 = pm.silu(h2[:, :inter2]) * h2[:, inter2:]
        assert np.abs(out2.float().cpu().numpy() - ref2).max() < (2e-6 if dtype == "float32" else 2.0 ** -7) * np.abs(ref2).max()
    # experts: all of them chosen, one of one, two of five; the weights are the chosen scores over their sum
    for E, top, scale in ((3, 3, 1.5), (1, 1, 2.0), (5, 2, 0.7), (40, 4, 1.0)):
        x, wr = bf(rng.standard_normal((n, 32))), bf(rng.standard_normal((E, 32)))
        ids, wts = ops.moe_route(dev(x, t), dev(wr, t), top, True, softmax=True, weight_scale=scale, sum_eps=1e-20)
        want_ids, want_w = pm.router(x, {"router": wr}, "", {"router": {"top": top, "scale": scale}})
        assert np.array_equal(np.sort(ids.cpu().numpy(), axis=1), np.sort(want_ids, axis=1))
        order_g, order_w = np.argsort(ids.cpu().numpy(), axis=1), np.argsort(want_ids, axis=1)
        assert np.abs(np.take_along_axis(wts.cpu().numpy(), order_g, 1) - np.take_along_axis(want_w, order_w, 1)).max() < 1e-5 * scale


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("width", [50, 192, 1030])
def test_the_sum_of_the_deltas_and_the_next_blocks_two_norms_in_one_pass(cuda_device, dtype, width):
    from bitnet_c_b200.csrc import ops
    rng = np.random.default_rng(width)
    t = DT[dtype]
    n = 7
    x, a, b = rng.standard_normal((n, width)) * 2, bf(rng.standard_normal((n, width))), rng.standard_normal((n, width))
    w1, w2 = bf(1 + 0.3 * rng.standard_normal(width)), bf(1 + 0.3 * rng.standard_normal(width))
    tol = 2e-6 if dtype == "float32" else 2.0 ** -7
    for second, with_b in ((True, True), (False, True), (True, False)):
        xd = dev(x)
        h1, h2 = ops.residual_add_norms(xd, dev(a, t), dev(b) if with_b else None, dev(w1, t), dev(w2, t) if second else None, 1e-5, t)
        want = x.astype(np.float32).astype(np.float64) + (a + (b.astype(np.float32) if with_b else 0.0))
        assert np.abs(xd.cpu().numpy() - want).max() < 1e-6 * np.abs(want).max()
        assert np.abs(h1.float().cpu().numpy() - pm.rms_norm(want, w1, 1e-5)).max() < tol * 4
        assert (h2 is None) == (not second)
        if second:
            assert np.abs(h2.float().cpu().numpy() - pm.rms_norm(want, w2, 1e-5)).max() < tol * 4


# ---- whole models ------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfg, buckets) in mc.CASES.items():
        w = mc.draw_weights(cfg, buckets, seed=21)
        out[name] = (mc.write_folder(str(tmp_path_factory.mktemp("mekevik") / name), cfg, w), w)
    return out


_ROUNDED = {}
CLOSE = {"float32": 2e-4, "bfloat16": 0.05}  # router margins below these may fall either way in that number format


def _plain_rounded(cfg, w, tokens):
    """The plain statement with bfloat16 storage, and per position the smallest margin of any router."""
    key = (json.dumps(cfg, sort_keys=True), tuple(tokens))
    if key not in _ROUNDED:
        margins = []
        rounded = pm.forward(cfg, w, tokens, round_fn=pm.to_bf16)
        pm.forward(cfg, w, tokens, margins_out=margins)
        _ROUNDED[key] = (rounded, np.min(margins, axis=0) if margins else np.full(len(tokens), np.inf))
    return _ROUNDED[key]


def _check(got, cfg, w, reqs, plain, dtype, what, rough_ok=False):
    """float32: every position within 1e-4 of the plain logits (relative to the largest).  bfloat16: the bound
    of a request is three times what rounding the stored activations does to the plain statement, taken at the
    request's 80th percentile of positions; at most a fifth of a request's positions may lie beyond it, none
    beyond three times the largest gap.  A position at which a router's choice is a close call (the last chosen
    expert's logit within ``CLOSE`` of the first one left out) is only looked at for non-finite numbers: among
    thousands of positions some always are.  ``rough_ok``: a request whose bound would exceed a tenth of its largest
    logit is only looked at for non-finite numbers."""
    sure = {}
    for r, per_pos in got.items():
        margin = _plain_rounded(cfg, w, reqs[r])[1]
        assert all(np.isfinite(row).all() for row in per_pos.values()), f"{what}: request {r}"
        sure[r] = {p: row for p, row in per_pos.items() if margin[p] >= CLOSE[dtype]}
        assert len(sure[r]) >= 0.9 * len(per_pos) - 1, "too many close calls: the test model's routers are too flat"
    if dtype == "float32":
        return compare(sure, plain, lambda ref: TOL_F32 * max(1.0, float(np.abs(ref).max())), what)
    for r, per_pos in sure.items():
        if not per_pos:
            continue
        gap = np.abs(plain[r] - _plain_rounded(cfg, w, reqs[r])[0]).max(axis=1)[sorted(per_pos)]  # of the positions that are looked at
        bound = BF16_GAP_FACTOR * float(np.percentile(gap, 80))
        if rough_ok and bound >= 0.1 * float(np.abs(plain[r]).max()):
            continue
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
    for s in cache.states.values():
        s.fill_(float("nan"))


@pytest.mark.parametrize("case", sorted(mc.CASES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_models_step_like_the_plain_statement_however_the_tokens_are_cut(folders, cuda_device, case, dtype):
    cfg = mc.CASES[case][0]
    d, w = folders[case]
    V = cfg["vocab"]
    reqs = {"a": random_tokens(1, 210, V), "b": random_tokens(2, 3, V), "c": random_tokens(3, 77, V), "d": random_tokens(4, 131, V)}
    plain = {r: pm.forward(cfg, w, t) for r, t in reqs.items()}
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
    """Layer by layer in float32: the residual stream after each block, through the step's diagnostic taps."""
    cfg = mc.CASES["A"][0]
    d, w = folders["A"]
    toks = random_tokens(9, 90, cfg["vocab"])
    want = []
    pm.forward(cfg, w, toks, layers_out=want)
    import io
    model = bn.load_model(d, dtype="float32")
    diag = model.diagnostics = bn.Diagnostics(dump_tag="lout", keep=True, out=io.StringIO())
    cache = model.new_cache(max_tokens=256, max_seqs=1)
    slot = cache.open()
    model.step(cache, [bn.SeqStep(slot, toks, [len(toks) - 1])])
    cache.close(slot)
    for i, ref in enumerate(want):
        for pos in (0, 1, 40, 89):
            (got,) = [r["values"] for r in diag.records if (r["tag"], r["layer"], r["pos"]) == ("lout", i, pos)]
            assert np.abs(got - ref[pos]).max() < 1e-4 * max(1.0, np.abs(ref[pos]).max()), f"after layer {i}, position {pos}"


@pytest.mark.parametrize("case", ["A", "C"])
def test_a_request_alone_and_in_a_batch_give_the_same_logits(folders, cuda_device, case):
    """Beyond rounding nothing of the batch around a request reaches it: in float32 the same numbers to 1e-5."""
    cfg = mc.CASES[case][0]
    d, _w = folders[case]
    V = cfg["vocab"]
    reqs = {"a": random_tokens(11, 140, V), "b": random_tokens(12, 66, V), "c": random_tokens(13, 5, V)}
    model = bn.load_model(d, dtype="float32")
    cache = model.new_cache(max_tokens=64 * 10, max_seqs=3)
    alone = replay(model, cache, trace_tail(reqs, 8))
    _poison(cache)
    together = replay(model, cache, trace_batches([{r: (t, min(8, len(t) - 1)) for r, t in reqs.items()}]))
    for r in reqs:
        for p, row in together[r].items():
            assert np.abs(row - alone[r][p]).max() < 1e-5 * max(1.0, np.abs(row).max()), (r, p)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_long_prompt_and_long_decoding_far_past_every_window(folders, cuda_device, dtype):
    """1,100 tokens in one step and 300 more one by one: the pages of every window are given back and taken again
    many times over, distances run far past the last bucket of every bias table."""
    cfg = mc.CASES["C"][0]
    d, w = folders["C"]
    toks = random_tokens(7, 1400, cfg["vocab"])
    reqs = {"x": toks}
    plain = {"x": pm.forward(cfg, w, toks)}
    model = bn.load_model(d, dtype=dtype)
    cache = model.new_cache(max_tokens=64 * 24, max_seqs=2)
    _poison(cache)
    got = replay(model, cache, trace_tail(reqs, 300))
    if dtype == "float32":
        compare(got, plain, lambda ref: 3 * TOL_F32 * max(1.0, float(np.abs(ref).max())), "long")
    else:
        _check(got, cfg, w, reqs, plain, dtype, "long, bfloat16")
    assert all(not h for g in cache.groups for h in g.held.values())


EDGE_LAYERS = {
    # one head on one key/value head, a mixing matrix of one number, key and value rows of one 16-byte piece
    "one head": [{"type": "attention", "mixer": {"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.7, "bias_max": 5,
                                                 "mask": {"size": 3}, "v_mix": True}, "mlp": None}] * 2,
    # nothing blends; no feed-forward anywhere; no mask
    "bare": [{"type": "attention", "mixer": {"heads": 4, "kv_heads": 4, "dim": 12, "vdim": 20, "scale": 0.5, "bias_max": 64},
              "mlp": None}] * 3,
    # only the last two layers blend; a window of two; every expert chosen by every token, and experts far more than tokens use
    "late blend": [{"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 8, "scale": 0.5, "bias_max": 33,
                                                   "mask": {"size": 2}, "v_mix": False},
                    "mlp": {"kind": "moe", "router": {"experts": 2, "top": 2, "scale": 1.0}, "expert": {"ff": 12}}},
                   {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 24, "scale": 0.5, "bias_max": 33,
                                                   "mask": {"size": 128}, "v_mix": True},
                    "mlp": {"kind": "moe", "router": {"experts": 40, "top": 1, "scale": 0.5}, "expert": {"ff": 8}}},
                   {"type": "attention", "mixer": {"heads": 6, "kv_heads": 3, "dim": 8, "vdim": 8, "scale": 0.5, "bias_max": 200,
                                                   "mask": {"size": 65}, "v_mix": True},
                    "mlp": {"kind": "dense", "ff": 24, "limit": 0.5}}],
}


@pytest.mark.parametrize("kind", sorted(EDGE_LAYERS))
def test_models_at_the_edges_of_what_the_configuration_allows(tmp_path, cuda_device, kind):
    cfg = {"architecture": "Mekevik", "vocab": 200, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.5},
           "logit_scale": 2.0, "layers": copy.deepcopy(EDGE_LAYERS[kind])}
    buckets = {i: (2, 4, 6, 12)[i % 4] for i in range(len(cfg["layers"]))}
    w = mc.draw_weights(cfg, buckets, seed=3)
    folder = mc.write_folder(str(tmp_path / "m"), cfg, w)
    reqs = {"a": random_tokens(1, 150, 200), "b": random_tokens(2, 70, 200), "c": random_tokens(3, 1, 200)}
    plain = {r: pm.forward(cfg, w, t) for r, t in reqs.items()}
    for dtype in ("float32", "bfloat16"):
        model = bn.load_model(folder, dtype=dtype)
        cache = model.new_cache(max_tokens=64 * 8, max_seqs=3)
        _poison(cache)
        for what, steps in (("whole", trace_whole(reqs)), ("last 30 one by one", trace_tail(reqs, 30)),
                            ("an unequal batch", trace_batches([{"a": (reqs["a"], 20), "b": (reqs["b"], 30), "c": (reqs["c"], 0)}]))):
            _check(replay(model, cache, steps), cfg, w, reqs, plain, dtype, f"{kind}, {what}, {dtype}", rough_ok=True)
        model.check_kernels()


WIDE = {
    # heads of 128 numbers; eight query heads on a key/value head, then eight key/value heads with one query head each;
    # a window that is no multiple of a page
    "architecture": "Mekevik", "vocab": 1500, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0}, "logit_scale": 0.5,
    "layers": [
        {"type": "attention", "mixer": {"heads": 8, "kv_heads": 1, "dim": 128, "vdim": 64, "scale": 0.09, "bias_max": 100,
                                        "mask": {"size": 150}, "v_mix": True},
         "mlp": {"kind": "moe", "router": {"experts": 8, "top": 2, "scale": 2.0}, "expert": {"ff": 48}}},
        {"type": "attention", "mixer": {"heads": 8, "kv_heads": 8, "dim": 32, "vdim": 8, "scale": 0.18, "bias_max": 300,
                                        "mask": {"size": 100}, "v_mix": True},
         "mlp": {"kind": "dense", "ff": 320, "limit": 4.0}},
        {"type": "attention", "mixer": {"heads": 16, "kv_heads": 4, "dim": 64, "vdim": 128, "scale": 0.125, "bias_max": 64,
                                        "v_mix": False},
         "mlp": {"kind": "moe", "router": {"experts": 3, "top": 1, "scale": 1.0}, "expert": {"ff": 200}}},
    ],
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_wider_model_with_heads_of_128_and_eight_heads_either_way(tmp_path, cuda_device, dtype):
    cfg = WIDE
    w = mc.draw_weights(cfg, {0: 32, 1: 64, 2: 8}, seed=2)
    folder = mc.write_folder(str(tmp_path / "m"), cfg, w)
    V = cfg["vocab"]
    reqs = {"a": random_tokens(1, 330, V), "b": random_tokens(2, 40, V), "c": random_tokens(3, 17, V)}
    plain = {r: pm.forward(cfg, w, t) for r, t in reqs.items()}
    model = bn.load_model(folder, dtype=dtype)
    cache = model.new_cache(max_tokens=64 * 12, max_seqs=3)
    _poison(cache)
    for what, steps in (("whole", trace_whole(reqs)), ("last 40 one by one", trace_tail(reqs, 40)),
                        ("pieces", trace_chunks(reqs, pieces=(16, 1, 100, 3))),
                        ("an unequal batch", trace_batches([{"a": (reqs["a"], 30), "b": (reqs["b"], 30), "c": (reqs["c"], 5)}]))):
        _check(replay(model, cache, steps), cfg, w, reqs, plain, dtype, f"wide, {what}, {dtype}")
    model.check_kernels()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_entry_point_and_the_replay_program(folders, cuda_device, tmp_path, dtype):
    cfg = mc.CASES["A"][0]
    d, w = folders["A"]
    V = cfg["vocab"]
    model = bn.load_model(d, dtype=dtype)
    prompts = [random_tokens(31, 50, V), random_tokens(32, 3, V), random_tokens(33, 120, V)]
    got = bn.generate(model, prompts, max_new_tokens=[70, 20, 24])
    for p, g in zip(prompts, got):
        assert len(g.tokens) in (70, 20, 24) and g.finish_reason == "length"
        seq = list(p) + g.tokens[:-1]
        ref = pm.forward(cfg, w, seq)[len(p) - 1:]
        if dtype == "float32":
            slack = 2 * TOL_F32 * max(1.0, float(np.abs(ref).max()))
        else:
            slack = 2 * BF16_GAP_FACTOR * float(np.abs(pm.forward(cfg, w, seq, round_fn=pm.to_bf16)[len(p) - 1:] - ref).max())
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
    plain = {k: pm.forward(cfg, w, t) for k, t in reqs.items()}
    _check(collect_trace_output(steps, out, V), cfg, w, reqs, plain, dtype, "through bin/trace_run")


def test_the_command_line_writes_a_random_model_of_the_design_and_generates_from_it(tmp_path, cuda_device):
    cfgp = tmp_path / "cfg.json"
    cfgp.write_text(json.dumps(mc.CASE_C))
    folder = tmp_path / "m"
    cmd = [sys.executable, os.path.join(ROOT, "bin", "bitnet"), str(folder), "--random-weights", "--config", str(cfgp),
           "--weight-seed", "3", "--dtype", "float32", "--prompt-token-ids", "5,17,3,9,9,1", "--prompt-token-ids", "7",
           "-n", "9", "--repeat-penalty", "1.0", "--token-ids"]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [[int(t) for t in l.split(",")] for l in p.stdout.splitlines() if l.strip()]
    assert [len(l) for l in lines] == [9, 9] and "Generation complete tokens=18" in p.stderr
