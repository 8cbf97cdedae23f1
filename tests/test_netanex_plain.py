"""The plain statement of the Netanex design (tests/plain_netanex.py) against closed forms, the faults it must
show, and the host side of the library for this design (configuration, parameter names, frequency table, cache
planes, random weights): everything here runs without a GPU."""
import copy
import json
import math

import numpy as np
import pytest

import netanex_cases as nc
import plain_netanex as pn
from helpers import random_tokens


# ---- the plain mechanisms against closed forms -----------------------------------------------------------
def test_a_window_sees_itself_and_the_positions_before_it():
    assert pn.visible(10, 10, 4) and pn.visible(10, 7, 4) and not pn.visible(10, 6, 4) and not pn.visible(10, 11, 4)
    assert pn.visible(10, 0, 0) and not pn.visible(3, 4, 0)
    assert pn.visible(5, 5, 1) and not pn.visible(5, 4, 1)


def test_a_sink_takes_weight_and_gives_nothing_back():
    s = np.array([0.3, -1.0, 2.0])
    plain = np.exp(s) / np.exp(s).sum()
    assert np.allclose(pn.softmax_with_sink(s, None), plain)
    w0 = pn.softmax_with_sink(s, 0.0)
    assert np.allclose(w0, np.exp(s) / (1.0 + np.exp(s).sum())) and w0.sum() < 1.0
    w = pn.softmax_with_sink(s, 50.0)  # a sink above every score
    assert np.allclose(w, np.exp(s - 50.0) / (1.0 + np.exp(s - 50.0).sum())) and w.sum() < 1e-18
    assert np.allclose(pn.softmax_with_sink(s, -1e9), plain)
    q, k, v = np.ones((1, 2)), np.ones((1, 2)), np.array([[3.0, -1.0]])
    assert np.allclose(pn.attend(q, k, v, 0.0, 0, 0.0), v / 2.0)  # one key with score 0 against a sink of 0


def test_the_query_factor_grows_by_steps_with_the_logarithm():
    f = [pn.query_temperature(p, 0.5, 4) for p in range(13)]
    assert f[0] == f[2] == 1.0 and f[3] == f[6] == 1.0 + 0.5 * math.log(2) and f[7] == 1.0 + 0.5 * math.log(3)
    assert f[11] == 1.0 + 0.5 * math.log(4) and pn.query_temperature(0, 0.3, 1) == 1.0 + 0.3 * math.log(2)


def test_blended_frequencies_keep_the_fast_end_and_divide_the_slow_end():
    f0 = 10000.0 ** (-2.0 * np.arange(16) / 32)
    f, mag = pn.yarn_frequencies(32, 10000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0})
    lo = math.floor(32 * math.log(64 / (2 * math.pi * 8.0)) / (2 * math.log(10000.0)))
    hi = math.ceil(32 * math.log(64 / (2 * math.pi * 2.0)) / (2 * math.log(10000.0)))
    assert np.allclose(f[: max(lo, 0) + 1], f0[: max(lo, 0) + 1]) and np.allclose(f[hi:], f0[hi:] / 4.0)
    assert all(f0[i] / 4.0 < f[i] < f0[i] for i in range(max(lo, 0) + 1, hi))
    assert mag == 0.1 * math.log(4.0) + 1.0
    g, one = pn.yarn_frequencies(32, 10000.0, None)
    assert np.allclose(g, f0) and one == 1.0


def test_rotated_scores_depend_on_the_distance_only_and_pair_the_halves():
    rng = np.random.default_rng(0)
    q, k = rng.standard_normal((1, 8)), rng.standard_normal((1, 8))
    sc = {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}
    dots = [float(pn.rotate_half(q, np.array([p + 5]), 8, 100.0, sc)[0] @ pn.rotate_half(k, np.array([p]), 8, 100.0, sc)[0]) for p in (0, 9, 200)]
    assert np.allclose(dots, dots[0])
    x = np.zeros((1, 8))
    x[0, 1] = 1.0
    y = pn.rotate_half(x, np.array([3]), 8, 100.0, None)[0]
    a = 3 * 100.0 ** (-2.0 / 8)
    assert np.allclose(y[[1, 5]], [math.cos(a), math.sin(a)]) and np.allclose(np.delete(y, [1, 5]), 0.0)
    z = pn.rotate_half(np.ones((1, 10)), np.array([3]), 4, 100.0, None)[0]  # numbers beyond the rotated ones pass
    assert np.allclose(z[4:], 1.0)


def test_the_second_maps_factor_and_the_experts_of_a_token():
    w = {"lq1": np.array([1.0, 2.0]), "lk1": np.array([0.5, 0.25]), "lq2": np.array([1.0, 0.0]), "lk2": np.array([-1.0, 9.0])}
    assert math.isclose(pn.differential_lambda(w, "", 0.3), math.exp(1.0) - math.exp(-1.0) + 0.3)
    assert [pn.kv_head_of(h, 6, 2) for h in range(6)] == [0, 0, 0, 1, 1, 1]
    rng = np.random.default_rng(1)
    W = {f"e{e}.{n}": rng.standard_normal((3, 4) if n != "down" else (4, 3)) for e in range(3) for n in ("gate", "up", "down")}
    W["table"] = np.array([[2, 0], [1, 2]], dtype=np.int32)
    h = rng.standard_normal((2, 4))
    got = pn.experts_by_table(h, [1, 0], W, "", {"router": {"top": 2}})
    want0 = (pn.expert(h[:1], W, "e1.") + pn.expert(h[:1], W, "e2.")) / 2
    want1 = (pn.expert(h[1:], W, "e2.") + pn.expert(h[1:], W, "e0.")) / 2
    assert np.allclose(got, np.concatenate([want0, want1]))


def test_a_layer_that_names_another_runs_with_that_layers_tensors():
    cfg = nc.CASE_A
    w = nc.draw_weights(cfg, 3)
    assert pn.layer_prefix(cfg, 3) == "l2." and pn.layer_prefix(cfg, 4) == "l1." and pn.layer_prefix(cfg, 5) == "l5."
    assert not any(n.startswith(("l3.", "l4.")) for n in w)
    taps = []
    pn.forward(random_tokens(1, 9, cfg["vocab"]), w, cfg, taps=taps)
    assert len(taps) == 6


# ---- faults must show --------------------------------------------------------------------------------------
def _faults(cfg):
    """(name, changed configuration, function that changes the weights) for every constant and tensor kind."""
    out = []

    def cfg_fault(name, i, path, fn):
        c = copy.deepcopy(cfg)
        for j, layer in enumerate(c["layers"]):  # a layer that shares weights shares the constants
            if j == i or layer.get("weights_of") == i:
                node = layer["mixer"]
                for key in path[:-1]:
                    node = node[key]
                node[path[-1]] = fn(node[path[-1]])
        out.append((f"layer {i}: {name}", c, None))

    def w_fault(name, tensor, fn):
        out.append((name, cfg, lambda w: {**w, tensor: fn(w[tensor])}))

    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        m, p = layer["mixer"], f"l{i}."
        cfg_fault("scale", i, ("scale",), lambda v: v * 2.0)
        if layer["type"] == "latent_attention":
            if m["mask"]["size"] <= 64:  # one key among more than that is too little to show with random weights
                cfg_fault("window one shorter", i, ("mask", "size"), lambda v: v - 1)
                cfg_fault("window one longer", i, ("mask", "size"), lambda v: v + 1)
            else:
                cfg_fault("window halved", i, ("mask", "size"), lambda v: v // 2)
            cfg_fault("rotary base", i, ("rot", "base"), lambda v: v * 10)
            if m["rot"].get("scaling"):
                cfg_fault("frequency factor", i, ("rot", "scaling", "factor"), lambda v: v * 2)
                cfg_fault("scaling taken off", i, ("rot", "scaling"), lambda v: None)
            w_fault(f"layer {i}: sinks far below every score", p + "mix.sink", lambda a: a - 60.0)
            w_fault(f"layer {i}: sinks of zero", p + "mix.sink", lambda a: a * 0.0)
            w_fault(f"layer {i}: gate off", p + "mix.g", lambda a: a * 0.0)
            w_fault(f"layer {i}: the latent's gain dropped", p + "mix.dkv.norm", lambda a: a * 0.0 + 1.0)
            w_fault(f"layer {i}: heads of the unrotated keys swapped", p + "mix.uk", lambda a: a[::-1].copy())
        else:
            w_fault(f"layer {i}: query bias off", p + "mix.q.b", lambda a: a * 0.0)
            w_fault(f"layer {i}: value bias off", p + "mix.v.b", lambda a: a * 0.0)
            w_fault(f"layer {i}: query gain dropped", p + "mix.q.norm", lambda a: a * 0.0 + 1.0)
        if layer["type"] == "attention":
            cfg_fault("diff", i, ("diff",), lambda v: v * 0.5)
            cfg_fault("no factor on the queries", i, ("q_temp", "coef"), lambda v: 0.0)
            cfg_fault("factor steps eight times as wide", i, ("q_temp", "every"), lambda v: v * 8)
            w_fault(f"layer {i}: the factor's vectors off", p + "mix.lq1", lambda a: a * 0.0)
            w_fault(f"layer {i}: output bias off", p + "mix.o.b", lambda a: a * 0.0)
            w_fault(f"layer {i}: maps swapped in the keys", p + "mix.k",
                    lambda a, d=m["dim"]: a.reshape(-1, 2, d, a.shape[1])[:, ::-1].reshape(a.shape).copy())
        if layer["type"] == "attention_2":
            w_fault(f"layer {i}: gate off", p + "mix.g", lambda a: a * 0.0)
            if m["heads"] * m["dim"] > m["dim"]:
                w_fault(f"layer {i}: the whole-projection gain rolled by a head", p + "mix.q.norm", lambda a, d=m["dim"]: np.roll(a, d))
        w_fault(f"layer {i}: first norm's gain taken as the factor itself", p + "norm1", lambda a: a - 1.0)
        w_fault(f"layer {i}: norm after the mixer left out", p + "norm1b", lambda a: a * 0.0 + 3.0)
        if layer.get("mlp") and layer["mlp"]["router"]["experts"] > layer["mlp"]["router"]["top"]:
            E = layer["mlp"]["router"]["experts"]
            w_fault(f"layer {i}: table shifted by an expert", p + "mlp.table", lambda a, E=E: ((a + 1) % E).astype(np.int32))
    out.append(("eps", {**copy.deepcopy(cfg), "norm": {"eps": 0.05}}, None))
    w_fault("embedding norm left out", "embed.norm", lambda a: a * 0.0)
    w_fault("final norm's gain taken as the factor itself", "final.norm", lambda a: a - 1.0)
    return out


@pytest.mark.parametrize("case", sorted(nc.CASES))
def test_every_constant_and_tensor_kind_moves_the_logits(case):
    """Every fault moves the logits by more than the GPU tests let a bfloat16 engine differ (tests/test_netanex_gpu.py:
    no position beyond three times the largest gap that rounding the stored activations opens, at most a fifth of
    the positions beyond three times the gap's 80th percentile)."""
    cfg = nc.CASES[case]
    w = nc.draw_weights(cfg, 21)
    toks = random_tokens(5, 200, cfg["vocab"])
    ref = pn.forward(toks, w, cfg)
    gap = np.abs(pn.forward(toks, w, cfg, r=pn.to_bf16) - ref).max(axis=1)
    faults = _faults(cfg)
    assert len(faults) >= 25
    for name, c, change in faults:
        err = np.abs(pn.forward(toks, change(w) if change else w, c) - ref).max(axis=1)
        caught = err.max() > 3.0 * gap.max() or int((err > 3.0 * np.percentile(gap, 80)).sum()) > len(toks) // 5
        assert caught, f"case {case}: {name} moves the logits by no more than rounding may"


def test_a_sink_of_zero_differs_from_no_sink():
    rng = np.random.default_rng(2)
    q, k, v = rng.standard_normal((12, 6)), rng.standard_normal((12, 6)), rng.standard_normal((12, 5))
    with_sink, without = pn.attend(q, k, v, 0.7, 0, 0.0), pn.attend(q, k, v, 0.7, 0, None)
    assert np.abs(with_sink - without).max() > 1e-2
    assert np.allclose(without, _plain_softmax(q, k, v, 0.7, 0)) and np.allclose(pn.attend(q, k, v, 0.7, 4, None), _plain_softmax(q, k, v, 0.7, 4))


def _plain_softmax(q, k, v, scale, window):
    T = q.shape[0]
    out = np.zeros((T, v.shape[1]))
    for i in range(T):
        js = [j for j in range(T) if pn.visible(i, j, window)]
        s = (k[js] @ q[i]) * scale
        e = np.exp(s - s.max())
        out[i] = (e / e.sum()) @ v[js]
    return out


# ---- the library's host side ---------------------------------------------------------------------------
def test_the_configuration_becomes_blocks_a_schedule_and_the_designs_tensor_names():
    from bitnet_c_b200.config import architecture_of
    from bitnet_c_b200.engine.model import parameter_table
    for name, cfg in nc.CASES.items():
        arch = architecture_of(cfg)
        assert arch.name == "Netanex"
        spec = arch.to_spec(arch.read_config(cfg))
        own = [i for i, l in enumerate(cfg["layers"]) if l.get("weights_of") is None]
        assert len(spec.blocks) == len(own) and len(spec.schedule) == len(cfg["layers"])
        for i, (layer, e) in enumerate(zip(cfg["layers"], spec.schedule)):
            src = layer.get("weights_of")
            assert e.block == own.index(i if src is None else src) and e.cache_of is None  # weights shared, caches not
        table = parameter_table(spec)
        names = {arch.tensor_name(p): tuple(s.shape) for p, s in table.items()}
        assert names == {n: tuple(s) for n, s in nc.tensor_shapes(cfg).items()}, name
        assert all(s.integer == (arch.tensor_name(p).endswith(".table")) for p, s in table.items())
        assert spec.tie_embeddings and spec.embedding_norm.one_plus and spec.final_norm.one_plus


def test_a_layer_on_anothers_weights_may_have_constants_of_its_own():
    from bitnet_c_b200.config import architecture_of
    from bitnet_c_b200.engine.model import parameter_table
    cfg = copy.deepcopy(nc.CASE_A)
    cfg["layers"][3]["mixer"]["mask"]["size"] = 5  # the same tensors under another window
    cfg["layers"][4]["mixer"]["diff"] = 0.1
    arch = architecture_of(cfg)
    spec = arch.to_spec(arch.read_config(cfg))
    assert len(spec.blocks) == 6 and [e.block for e in spec.schedule] == [0, 1, 2, 3, 4, 5]
    assert [b.label for b in spec.blocks] == ["0", "1", "2", "2@3", "1@4", "5"]
    assert spec.blocks[3].mixer.window == 5 and spec.blocks[2].mixer.window == 37 and spec.blocks[4].mixer.diff == 0.1
    table = parameter_table(spec)
    names = {arch.tensor_name(p) for p in table}
    assert names == set(nc.tensor_shapes(nc.CASE_A))  # no tensor more than the owners have
    assert arch.tensor_name("blocks.2@3.mixer.sink") == "l2.mix.sink" and arch.tensor_name("blocks.1@4.ffn.table") == "l1.mlp.table"


def test_mixers_carry_every_constant_of_the_configuration():
    from bitnet_c_b200.config import architecture_of
    arch = architecture_of(nc.CASE_A)
    spec = arch.to_spec(arch.read_config(nc.CASE_A))
    whole, two, latent = spec.blocks[0].mixer, spec.blocks[1].mixer, spec.blocks[2].mixer
    assert (whole.qk_norm, whole.sink, whole.head_gate, whole.maps, whole.proj_bias, whole.out_bias) == ("whole", "zero", True, 1, True, False)
    assert (two.qk_norm, two.sink, two.maps, two.diff, two.temp_coef, two.temp_every, two.out_bias) == ("head", "none", 2, 0.35, 0.8, 16, True)
    assert (latent.q_rank, latent.sink, latent.element_gate, latent.head_gate, latent.window) == (0, True, True, False, 37)
    assert (latent.position.pairing, latent.position.factor, latent.position.fast, latent.position.slow) == ("halves", 4.0, 8.0, 2.0)
    assert spec.blocks[2].ffn is None and spec.blocks[0].ffn.scores == "table" and spec.blocks[0].ffn.table_rows == 97
    assert spec.blocks[1].ffn.top == 3 and not spec.blocks[1].ffn.weight_on_input
    assert spec.blocks[0].mixer_norm.eps == 1e-5 and latent.norm_eps == 1e-5


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][0].update(type="attention_3"), "type"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "multiple"),
    (lambda c: c["layers"][2]["mixer"].update(rot_dim=6), "rot"),
    (lambda c: c["layers"][3].update(weights_of=4), "weights_of"),
    (lambda c: c["layers"][4].update(type="attention_2"), "another kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mixer"].pop("diff"), "diff"),
    (lambda c: c["norm"].update(eps=0), "eps"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
])
def test_configurations_that_cannot_be_built_are_refused_by_name(change, message):
    from bitnet_c_b200.config import ConfigError, architecture_of
    cfg = copy.deepcopy(nc.CASE_A)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        architecture_of(cfg).read_config(cfg)


def test_the_librarys_frequency_table_is_the_plain_one():
    from bitnet_c_b200.config import RotaryBlendSpec
    from bitnet_c_b200.parts.position import blended_frequencies
    for dims, base, sc in ((8, 10000.0, {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 2.0}), (6, 500.0, None),
                           (64, 1e6, {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}),
                           (16, 1000.0, {"factor": 8.0, "original": 32, "fast": 4.0, "slow": 1.0})):
        spec = RotaryBlendSpec(dims=dims, base=base, **({k: float(v) for k, v in sc.items()} if sc else {}))
        f, mag = blended_frequencies(spec)
        want, want_mag = pn.yarn_frequencies(dims, base, sc)
        assert f.dtype == np.float32 and np.array_equal(f, want.astype(np.float32)) and math.isclose(mag, want_mag)


def test_cache_planes_of_the_design_keep_a_window_and_fewer_value_heads():
    from bitnet_c_b200.config import architecture_of
    from bitnet_c_b200.engine import Model
    arch = architecture_of(nc.CASE_A)
    model = Model(arch.to_spec(arch.read_config(nc.CASE_A)), dtype="float32", device=None)
    cache = model.new_cache(max_tokens=64 * 8, max_seqs=2, allocate=False)
    reqs = [g.request for g in cache.groups]
    two = [r for r in reqs if r.v_heads]
    assert len(two) == 1 and (two[0].n_kv_heads, two[0].n_v_heads, two[0].head_dim, two[0].v_dim) == (4, 2, 8, 16)
    latent = [g for g in cache.groups if g.request.values_in_keys]
    assert len(latent) == 1 and latent[0].request.window == 37 and latent[0].request.head_dim == 48 and len(latent[0].entries) == 2
    assert sum(len(g.entries) for g in cache.groups) == 6  # a plane for every run, also for runs that share weights
    s = cache.open()
    cache.reserve(s, 300)
    cache.advance(s, 300)
    assert len(latent[0].held[s]) == 1 and all(len(g.held[s]) == 5 for g in cache.groups if g is not latent[0])
    cache.close(s)
    cache.check()
    assert all(g.pool.n_free == g.pool.n_pages for g in cache.groups)


def test_random_weights_of_the_design_have_tables_of_different_experts(tmp_path):
    import bitnet_c_b200 as bn
    from bitnet_c_b200.weights.safetensors_io import SafetensorsFile
    folder = bn.write_random_model(str(tmp_path / "m"), nc.CASE_C, seed=5)
    f = SafetensorsFile(str(tmp_path / "m" / "model.safetensors"))
    try:
        assert set(f.names()) == set(nc.tensor_shapes(nc.CASE_C))
        t = f.read("l2.mlp.table").numpy()
        assert t.shape == (150, 3) and t.min() >= 0 and t.max() < 4 and all(len(set(row)) == 3 for row in t)
        assert abs(float(f.read("l0.norm1").float().mean())) < 0.1  # gains are kept as offsets from one
    finally:
        f.close()
    assert json.load(open(tmp_path / "m" / "config.json"))["architecture"] == "Netanex"
