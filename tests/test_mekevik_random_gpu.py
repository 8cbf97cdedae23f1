"""Mekevik configurations drawn at random by fixed seeds from all that its config.json allows (numbers of
layers, head counts and sizes with key and value widths apart, windows below and above a cache page or absent,
bias tables of few and many rows, blending in any subset of the layers, dense units, experts of which a token
takes one, some or all, layers without a feed-forward), each stepped whole, token by token, in pieces and in
unequal batches against the plain statement, in both number formats."""
import numpy as np
import pytest

import bitnet_c_b200 as bn
import mekevik_cases as mc
import plain_mekevik as pm
from helpers import TOL_F32, random_tokens, replay, trace_batches, trace_chunks, trace_tail, trace_whole
from test_mekevik_gpu import _check, _poison

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
    blend_width = pick([16, 24, 32, 48])  # layers that blend hold as many value numbers per token as their source
    layers, buckets = [], {}
    for i in range(int(rng.integers(1, 7))):
        g = pick([1, 2, 3, 4])
        m = {"heads": g * pick([1, 2, 3, 4]), "kv_heads": g, "dim": pick([4, 8, 16, 20, 32, 64]), "vdim": pick([4, 8, 12, 16, 32, 48]),
             "scale": float(rng.uniform(0.2, 1.0)), "v_mix": bool(rng.random() < 0.6)}
        if m["v_mix"]:
            if blend_width % g:
                m["v_mix"] = False
            else:
                m["vdim"] = blend_width // g
        if rng.random() < 0.85:
            m["mask"] = {"size": int(rng.integers(1, 200))}
        buckets[i] = pick([2, 4, 8, 16, 32, 33])
        m["bias_max"] = buckets[i] // 2 + int(rng.integers(1, 300))
        kind = pick(["dense", "moe", "moe", None])
        if kind == "dense":
            mlp = {"kind": "dense", "ff": pick([8, 12, 24, 40, 64, 100]), "limit": float(pick([0.5, 1.0, 2.0, 7.0]))}
        elif kind == "moe":
            e = pick([1, 2, 3, 5, 8, 16])
            mlp = {"kind": "moe", "router": {"experts": e, "top": int(rng.integers(1, min(e, 4) + 1)), "scale": float(pick([0.5, 1.0, 2.5]))},
                   "expert": {"ff": pick([8, 12, 24, 40])}}
        else:
            mlp = None
        layers.append({"type": "attention", "mixer": m, "mlp": mlp})
    cfg = {"architecture": "Mekevik", "vocab": int(rng.integers(50, 300)), "width": width, "norm": {"eps": pick([1e-5, 1e-6])},
           "embedding": {"scale": float(pick([1.0, 2.0, 5.5]))}, "logit_scale": float(pick([0.25, 1.0, 3.0])), "layers": layers}
    return cfg, buckets


@pytest.mark.parametrize("seed", range(12))
def test_a_configuration_drawn_at_random_steps_like_the_plain_statement(tmp_path, cuda_device, seed):
    cfg, buckets = draw_config(3000 + seed)
    w = mc.draw_weights(cfg, buckets, seed=seed)
    folder = mc.write_folder(str(tmp_path / "m"), cfg, w)
    V = cfg["vocab"]
    reqs = {"a": random_tokens(seed, 230, V), "b": random_tokens(seed + 50, 1, V), "c": random_tokens(seed + 99, 70, V)}
    plain = {r: pm.forward(cfg, w, t) for r, t in reqs.items()}
    # how much single-precision rounding may move a position shows when the plain statement runs with weights
    # moved by 1e-7 of their size; float32 is allowed 30 times that on top of its bound
    rng = np.random.default_rng(seed)
    moved = {k: a * (1.0 + 1e-7 * rng.standard_normal(a.shape)) for k, a in w.items()}
    slack = {r: 30.0 * np.abs(pm.forward(cfg, moved, t) - plain[r]).max(axis=1) for r, t in reqs.items()}
    for dtype in ("float32", "bfloat16") if seed % 2 == 0 else ("float32",):
        model = bn.load_model(folder, dtype=dtype)
        cache = model.new_cache(max_tokens=64 * 10, max_seqs=3)
        _poison(cache)
        for what, steps in (("whole", trace_whole(reqs)), ("last 25 one by one", trace_tail(reqs, 25)),
                            ("pieces", trace_chunks(reqs, pieces=(3, 64, 17, 1))),
                            ("an unequal batch", trace_batches([{"a": (reqs["a"], 12), "c": (reqs["c"], 30), "b": (reqs["b"], 0)}]))):
            got = replay(model, cache, steps)
            if dtype == "bfloat16":
                _check(got, cfg, w, reqs, plain, dtype, f"seed {seed}: {what}, {dtype}", rough_ok=True)
                continue
            for r, per_pos in got.items():
                for p, row in sorted(per_pos.items()):
                    err = float(np.abs(row.astype(np.float64) - plain[r][p]).max())
                    assert err <= TOL_F32 * max(1.0, float(np.abs(plain[r]).max())) + slack[r][p], \
                        f"seed {seed}: {what}: request {r} position {p}: max |diff| {err:.3e}"
        model.check_kernels()
