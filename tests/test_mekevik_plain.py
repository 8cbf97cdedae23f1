"""The plain statement of the Mekevik design checks itself on small facts, the test models are sharp enough to
show faults, and the library's host side (configuration, parameter table, cache planes) is checked without a GPU."""
import copy
import math

import numpy as np
import pytest

import mekevik_cases as mc
import plain_mekevik as pm
from helpers import random_tokens


def test_distance_buckets_are_exact_below_half_and_logarithmic_beyond():
    B, D = 32, 120
    b = [pm.distance_bucket(n, B, D) for n in range(400)]
    assert b[:16] == list(range(16))  # below half the table a distance is its own bucket
    assert b[16] == 16 and b[D] == B - 1  # the last bucket starts at D at the latest
    assert all(x <= y for x, y in zip(b, b[1:])) and max(b) == B - 1 and b[399] == B - 1
    # an edge where the logarithm says it is: bucket 16 + k begins at 16 * (D / 16) ** (k / 16)
    for k in range(1, 16):
        edge = 16 * (D / 16) ** (k / 16)
        n = math.ceil(edge - 1e-9)
        assert pm.distance_bucket(n, B, D) >= 16 + k > pm.distance_bucket(n - 1, B, D) or n - 1 < 16
    # tables with an odd number of rows and with two rows
    assert [pm.distance_bucket(n, 5, 9) for n in range(12)][:2] == [0, 1]
    assert [pm.distance_bucket(n, 2, 3) for n in range(5)] == [0, 1, 1, 1, 1]


def test_a_window_holds_the_token_itself_and_the_ones_before_it():
    assert pm.visible(10, 10, 1) and not pm.visible(10, 9, 1)
    assert pm.visible(10, 4, 7) and not pm.visible(10, 3, 7) and not pm.visible(10, 11, 7)
    assert pm.visible(500, 0, 0)  # no mask: every earlier key


def test_weights_are_not_normalised_and_heads_are_mixed_after_the_logistic_function():
    rng = np.random.default_rng(0)
    T, H, G, d = 9, 4, 2, 8
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": 4, "scale": 0.5, "bias_max": 20, "mask": {"size": 5}}
    q, k = rng.standard_normal((T, H, d)), rng.standard_normal((T, G, d))
    w = {"rel": rng.standard_normal((8, H)), "pb": rng.standard_normal(H), "talk": rng.standard_normal((H, H))}
    a = pm.attention_weights(q, k, w, "", m)
    for h in range(H):
        for i in range(T):
            for j in range(T):
                want = 0.0
                for g in range(H):
                    if 0 <= i - j < 5:
                        s = q[i, g] @ k[j, g // 2] * 0.5 + w["rel"][pm.distance_bucket(i - j, 8, 20), g] + w["pb"][g]
                        want += w["talk"][h, g] / (1.0 + math.exp(-s))
                assert abs(a[h, i, j] - want) < 1e-12
    # with the identity as mixing matrix every weight lies in (0, 1) and rows do not sum to one
    w["talk"] = np.eye(H)
    a = pm.attention_weights(q, k, w, "", m)
    assert (a >= 0).all() and (a < 1).all() and abs(a[0, 8].sum() - 1.0) > 1e-3


def test_values_are_blended_number_by_number_and_the_first_layer_is_the_source():
    rng = np.random.default_rng(1)
    h = rng.standard_normal((5, 6))
    m = {"kv_heads": 2, "vdim": 3}
    w = {"v": rng.standard_normal((6, 6)), "vmix": np.asarray(0.25)}
    first = rng.standard_normal((5, 3, 2))  # other heads, the same count of numbers per token
    v = pm.attention_values(h, w, "", m, first)
    assert np.allclose(v.reshape(5, 6), 0.75 * (h @ w["v"].T) + 0.25 * first.reshape(5, 6))
    assert np.allclose(pm.attention_values(h, w, "", m, None).reshape(5, 6), h @ w["v"].T)


def test_the_dense_unit_clamps_the_gate_from_above_and_the_other_half_on_both_sides():
    w = {"gate": np.array([[1.0], [1.0], [1.0]]), "up": np.array([[1.0], [-1.0], [0.0]]), "down": np.eye(3)}
    y = pm.dense_ffn(np.array([[10.0], [-10.0]]), w, "", {"limit": 2.0})
    s = lambda z: 1.0 / (1.0 + math.exp(-1.702 * z))  # noqa: E731
    assert np.allclose(y[0], [2 * s(2) * 3.0, 2 * s(2) * -1.0, 2 * s(2) * 1.0])
    assert np.allclose(y[1], [-10 * s(-10) * -1.0, -10 * s(-10) * 3.0, -10 * s(-10) * 1.0])


def test_router_weights_are_softmax_scores_of_the_chosen_over_their_sum_times_the_scale():
    rng = np.random.default_rng(2)
    h = rng.standard_normal((7, 5))
    w = {"router": rng.standard_normal((6, 5))}
    ids, wt = pm.router(h, w, "", {"router": {"experts": 6, "top": 2, "scale": 1.5}})
    z = h @ w["router"].T
    for t in range(7):
        order = np.argsort(-z[t])
        assert list(ids[t]) == list(order[:2])
        e = np.exp(z[t][order[:2]])
        assert np.allclose(wt[t], 1.5 * e / e.sum())
    ids, wt = pm.router(h, w, "", {"router": {"experts": 6, "top": 6, "scale": 0.5}})
    assert np.allclose(wt.sum(1), 0.5)


@pytest.mark.parametrize("case", sorted(mc.CASES))
def test_faults_in_the_mechanisms_move_the_logits_of_the_test_models(case):
    """The models of the engine tests are sharp enough: each of these faults moves some logit by far more than
    the engine's float32 tolerance, so a test that passes excludes them."""
    cfg, buckets = mc.CASES[case]
    w = mc.draw_weights(cfg, buckets, seed=5)
    toks = random_tokens(4, 170, cfg["vocab"])
    ref = pm.forward(cfg, w, toks)
    assert 0.5 < np.abs(ref).max() < 500.0

    def moved(change_cfg=None, change_w=None):
        c, ww = copy.deepcopy(cfg), dict(w)
        if change_cfg:
            change_cfg(c)
        if change_w:
            change_w(ww)
        return float(np.abs(pm.forward(c, ww, toks) - ref).max())

    blending = [i for i, l in enumerate(cfg["layers"]) if l["mixer"].get("v_mix")]
    for i, l in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", l["mixer"]
        size = (m.get("mask") or {}).get("size", 0)
        if 1 < size < 170:
            assert moved(lambda c: c["layers"][i]["mixer"]["mask"].update(size=size + 1)) > 1e-3, f"mask of layer {i}"
            assert moved(lambda c: c["layers"][i]["mixer"]["mask"].update(size=size - 1)) > 1e-3, f"mask of layer {i}"
        assert moved(lambda c: c["layers"][i]["mixer"].update(scale=m["scale"] * 1.1)) > 1e-3, f"scale of layer {i}"
        if size != 1:
            assert moved(lambda c: c["layers"][i]["mixer"].update(bias_max=m["bias_max"] + 7)) > 1e-4, f"bias reach of layer {i}"
            assert moved(change_w=lambda ww: ww.update({p + "rel": np.roll(w[p + "rel"], 1, axis=0)})) > 1e-3, f"bias of layer {i}"
        assert moved(change_w=lambda ww: ww.update({p + "pb": w[p + "pb"] + 0.5})) > 1e-3, f"head bias of layer {i}"
        assert moved(change_w=lambda ww: ww.update({p + "talk": w[p + "talk"].T.copy()})) > 1e-3 or m["heads"] == 1, f"mixing of layer {i}"
        assert moved(change_w=lambda ww: ww.update({p + "g": np.zeros_like(w[p + "g"])})) > 1e-3, f"gate of layer {i}"
        assert moved(change_w=lambda ww: ww.update({p + "q.norm": np.ones_like(w[p + "q.norm"])})) > 1e-3, f"query norm of layer {i}"
        if i in blending[1:]:
            assert moved(change_w=lambda ww: ww.update({p + "vmix": np.asarray(0.0)})) > 1e-3, f"blend of layer {i}"
        if i == blending[0]:  # the source's own weight is not read
            assert moved(change_w=lambda ww: ww.update({p + "vmix": np.asarray(0.9)})) == 0.0
        mlp = l.get("mlp")
        if mlp and mlp["kind"] == "dense":
            assert moved(lambda c: c["layers"][i]["mlp"].update(limit=mlp["limit"] * 0.5)) > 1e-3, f"limit of layer {i}"
        if mlp and mlp["kind"] == "moe":
            assert moved(lambda c: c["layers"][i]["mlp"]["router"].update(scale=mlp["router"]["scale"] * 1.2)) > 1e-3, f"router scale of layer {i}"
            if mlp["router"]["top"] < mlp["router"]["experts"]:
                assert moved(lambda c: c["layers"][i]["mlp"]["router"].update(top=mlp["router"]["top"] + 1)) > 1e-3, f"top of layer {i}"
    assert moved(lambda c: c["norm"].update(eps=0.5)) > 1e-3
    assert moved(lambda c: c["embedding"].update(scale=cfg["embedding"]["scale"] * 1.5)) > 1e-3
    assert moved(lambda c: c.update(logit_scale=cfg["logit_scale"] * 1.1)) > 1e-3


# ---- the library's host side ---------------------------------------------------------------------
def test_the_configuration_is_read_key_by_key_and_builds_the_parameter_table_of_the_design():
    import bitnet_c_b200 as bn
    from bitnet_c_b200.config import ConfigError, architecture_of
    from bitnet_c_b200.engine.model import parameter_table
    assert "Mekevik" in bn.known_architectures()
    for cfg_dict, buckets in mc.CASES.values():
        shapes = mc.tensor_shapes(cfg_dict, buckets)
        arch = architecture_of(cfg_dict)
        cfg = arch.read_config(arch.complete_config(cfg_dict, shapes))
        spec = arch.to_spec(cfg)
        table = {}
        for p, s in parameter_table(spec).items():
            if not s.optional or arch.tensor_name(p) in shapes:
                table.setdefault(arch.tensor_name(p), set()).add(tuple(s.shape))
        assert {n: next(iter(v)) for n, v in table.items()} == shapes and all(len(v) == 1 for v in table.values())
        assert arch.read_config(arch.config_to_dict(cfg)) == cfg
    arch = architecture_of(mc.CASE_A)
    spec = arch.to_spec(arch.read_config(arch.complete_config(mc.CASE_A, mc.tensor_shapes(mc.CASE_A, mc.BUCKETS_A))))
    m0, m1, m2, m3 = (b.mixer for b in spec.blocks)
    assert (m0.kind, m0.window, m0.bias_buckets, m0.bias_max_distance, m0.value_mix) == ("sigmoid_attention", 37, 16, 30, "source")
    assert (m1.value_mix, m2.value_mix, m3.value_mix, m3.window, m1.scale) == ("blend", "none", "blend", 1, 0.7)
    f0, f1, f2 = spec.blocks[0].ffn, spec.blocks[1].ffn, spec.blocks[2].ffn
    assert (f0.kind, f0.limit, f0.slope, f0.intermediate) == ("limited_mlp", 1.5, 1.702, 40) and f2 is None
    assert (f1.kind, f1.n_experts, f1.top, f1.scores, f1.weight_scale, f1.renormalise, f1.activation) == ("moe", 5, 2, "softmax", 0.7, True, "silu")
    assert spec.embedding_scale == 2.0 and spec.head.scale == 0.5 and not spec.tie_embeddings
    specB = arch.to_spec(arch.read_config(arch.complete_config(mc.CASE_B, mc.tensor_shapes(mc.CASE_B, mc.BUCKETS_B))))
    assert [b.mixer.value_mix for b in specB.blocks] == ["none", "source", "blend"] and specB.blocks[2].mixer.window == 0
    for bad, what in ((lambda c: c["layers"][0].update(type="conv"), "type"),
                      (lambda c: c["layers"][1]["mixer"].pop("scale"), "scale"),
                      (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "kv_heads"),
                      (lambda c: c["layers"][1]["mixer"].update(vdim=8), "v_mix"),
                      (lambda c: c["layers"][0]["mixer"].update(bias_max=3), "bias_max"),
                      (lambda c: c["layers"][0]["mlp"].update(kind="conv"), "kind"),
                      (lambda c: c["layers"][0]["mlp"].update(limit=0), "limit"),
                      (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "top"),
                      (lambda c: c["norm"].pop("eps"), "eps"),
                      (lambda c: c.pop("logit_scale"), "logit_scale")):
        c = copy.deepcopy(mc.CASE_A)
        bad(c)
        with pytest.raises(ConfigError, match=what):
            arch.read_config(arch.complete_config(c, mc.tensor_shapes(mc.CASE_A, mc.BUCKETS_A)))


def test_the_distance_table_of_the_mixer_follows_the_plain_buckets():
    from bitnet_c_b200.parts.sigmoid_attention import bias_buckets
    for B, D in ((32, 120), (16, 30), (6, 20), (4, 12), (2, 3), (20, 100), (8, 9), (5, 9)):
        got = bias_buckets(B, D).tolist()
        assert got == [pm.distance_bucket(n, B, D) for n in range(D + 1)] and got[-1] == B - 1
        assert all(pm.distance_bucket(n, B, D) == B - 1 for n in (D + 1, 3 * D, 100000))


def test_windowed_planes_give_back_the_pages_that_no_later_token_sees():
    from bitnet_c_b200.cache import Cache
    from bitnet_c_b200.parts import KvRequest
    c = Cache([KvRequest(2, 16, window=37, v_head_dim=24), KvRequest(2, 8, window=64, v_head_dim=24)], [None, None], [None, None],
              64 * 12, 1 << 20, None, None, allocate=False)
    s = c.open()
    c.reserve(s, 300)
    c.advance(s, 300)
    # the next token, at 300, sees 264..300 under the window of 37 and 237..300 under the window of 64
    assert sorted(c.groups[0].held[s]) == [4] and sorted(c.groups[1].held[s]) == [3, 4]
    c.close(s)
    c.check()
