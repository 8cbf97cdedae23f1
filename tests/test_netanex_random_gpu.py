"""Netanex configurations drawn at random by fixed seeds from all that its config.json allows (numbers of layers
and their kinds in any order, layers that run with an earlier layer's weights, head counts and sizes with key and
value widths apart, rotated parts of any even width, windows below and above a cache page or absent, frequency
tables with and without the blend, factors on the queries with steps of any width or none, experts of which a
token takes one, some or all, layers without a feed-forward), each stepped whole, token by token, in pieces and in
unequal batches against the plain statement, in both number formats."""
import copy

import numpy as np
import pytest

import bitnet_c_b200 as bn
import netanex_cases as nc
import plain_netanex as pn
from helpers import TOL_F32, random_tokens, replay, trace_batches, trace_chunks, trace_tail, trace_whole
from test_netanex_gpu import _poison, _plain_rounded

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


def draw_config(seed: int):
    rng = np.random.default_rng(seed)
    pick = lambda xs: xs[int(rng.integers(len(xs)))]
    width = pick([32, 40, 48, 64, 72, 96, 128])
    vocab = int(rng.integers(50, 300))
    layers = []
    for i in range(int(rng.integers(1, 7))):
        own = [j for j, l in enumerate(layers) if l.get("weights_of") is None]
        if own and rng.random() < 0.3:
            j = pick(own)
            layers.append({**copy.deepcopy(layers[j]), "weights_of": j})
            continue
        kind = pick(["attention", "attention_2", "latent_attention"])
        if kind == "latent_attention":
            dr = pick([2, 4, 6, 8, 16, 32])
            m = {"heads": pick([1, 2, 3, 4, 6]), "dim": pick([4, 8, 12, 16, 32]), "rot_dim": dr, "vdim": pick([4, 8, 12, 16, 32]),
                 "kv_rank": pick([8, 12, 24, 40, 48, 72]), "scale": float(rng.uniform(0.1, 0.5)),
                 "rot": {"base": float(pick([100.0, 1e4, 1e6])), "dims": dr}}
            if rng.random() < 0.7:
                m["rot"]["scaling"] = {"factor": float(pick([1.5, 2.0, 4.0, 32.0])), "original": int(pick([16, 64, 512, 4096])),
                                       "fast": float(pick([4.0, 16.0, 32.0])), "slow": float(pick([0.5, 1.0, 2.0]))}
            if rng.random() < 0.85:
                m["mask"] = {"size": int(rng.integers(1, 200))}
        else:
            g = pick([1, 2, 3, 4])
            m = {"heads": g * pick([1, 2, 3, 4]), "kv_heads": g, "dim": pick([4, 8, 16, 20, 32, 64]), "vdim": pick([4, 8, 12, 16, 32, 48]),
                 "scale": float(rng.uniform(0.15, 0.8))}
            if kind == "attention":
                m["diff"] = float(pick([0.0, 0.2, 0.5, 0.8]))
                if rng.random() < 0.8:
                    m["q_temp"] = {"coef": float(pick([0.1, 0.5, 1.0])), "every": int(pick([1, 2, 7, 32, 64, 100, 1000]))}
        mlp = None
        if rng.random() < 0.75:
            e = pick([1, 2, 3, 5, 8, 16])
            mlp = {"kind": "moe", "router": {"experts": e, "top": int(rng.integers(1, min(e, 4) + 1))}, "expert": {"ff": pick([8, 12, 24, 40])}}
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    return {"architecture": "Netanex", "vocab": vocab, "width": width, "norm": {"eps": pick([1e-5, 1e-6])}, "layers": layers}


@pytest.mark.parametrize("seed", range(12))
def test_a_configuration_drawn_at_random_steps_like_the_plain_statement(tmp_path, cuda_device, seed):
    cfg = draw_config(4000 + seed)
    w = nc.draw_weights(cfg, seed=seed)
    folder = nc.write_folder(str(tmp_path / "m"), cfg, w)
    V = cfg["vocab"]
    reqs = {"a": random_tokens(seed, 230, V), "b": random_tokens(seed + 50, 1, V), "c": random_tokens(seed + 99, 70, V)}
    plain = {r: pn.forward(t, w, cfg) for r, t in reqs.items()}
    # how much single-precision rounding may move a position shows when the plain statement runs with weights
    # moved by 1e-7 of their size; float32 is allowed 30 times that on top of its bound
    rng = np.random.default_rng(seed)
    moved = {k: (a if a.dtype == np.int32 else a * (1.0 + 1e-7 * rng.standard_normal(a.shape))) for k, a in w.items()}
    slack = {r: 30.0 * np.abs(pn.forward(t, moved, cfg) - plain[r]).max(axis=1) for r, t in reqs.items()}
    for dtype in ("float32", "bfloat16") if seed % 2 == 0 else ("float32",):
        model = bn.load_model(folder, dtype=dtype)
        cache = model.new_cache(max_tokens=64 * 10, max_seqs=3)
        _poison(cache)
        for what, steps in (("whole", trace_whole(reqs)), ("last 25 one by one", trace_tail(reqs, 25)),
                            ("pieces", trace_chunks(reqs, pieces=(3, 64, 17, 1))),
                            ("an unequal batch", trace_batches([{"a": (reqs["a"], 12), "c": (reqs["c"], 30), "b": (reqs["b"], 0)}]))):
            got = replay(model, cache, steps)
            for r, per_pos in got.items():
                assert all(np.isfinite(row).all() for row in per_pos.values()), f"seed {seed}: {what}: request {r}"
                if dtype == "bfloat16":
                    # a model drawn at random may be rough: the bound follows what rounding the stored activations does
                    # to the plain statement, place by place (three times the request's largest gap, a fifth of the
                    # positions beyond three times its 80th percentile)
                    gap = np.abs(plain[r] - _plain_rounded(cfg, w, reqs[r])).max(axis=1)[sorted(per_pos)]
                    err = np.array([np.abs(row.astype(np.float64) - plain[r][p]).max() for p, row in sorted(per_pos.items())])
                    assert err.max() <= 3.0 * gap.max() + 1e-3, f"seed {seed}: {what}, {dtype}: request {r}: position {sorted(per_pos)[int(err.argmax())]}"
                    assert int((err > 3.0 * np.percentile(gap, 80) + 1e-3).sum()) <= max(1, len(err) // 5), f"seed {seed}: {what}, {dtype}: request {r}"
                    continue
                for p, row in sorted(per_pos.items()):
                    err = float(np.abs(row.astype(np.float64) - plain[r][p]).max())
                    assert err <= TOL_F32 * max(1.0, float(np.abs(plain[r]).max())) + slack[r][p], \
                        f"seed {seed}: {what}: request {r} position {p}: max |diff| {err:.3e}"
        model.check_kernels()
