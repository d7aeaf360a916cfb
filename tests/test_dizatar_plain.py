"""The plain Dizatar statement against loop-level formulas, and the
configuration, run order and tensor list of the packaged model (no GPU)."""
import json
import math

import numpy as np
import pytest
import torch

import dizatar_cases as C
import plain_dizatar as P


def test_rotation_pairs_i_with_i_plus_half():
    rng = np.random.default_rng(0)
    dims, n, base = 6, 9, 37.0
    v = torch.tensor(rng.normal(size=(4, 2, n)))
    pos = torch.tensor([0, 3, 11, 500])
    out = P.rotate_half_pairs(v, pos, dims, base)
    for t in range(4):
        for h in range(2):
            for i in range(dims // 2):
                a = float(pos[t]) * base ** (-2.0 * i / dims)
                u, w = float(v[t, h, i]), float(v[t, h, i + dims // 2])
                assert abs(float(out[t, h, i]) - (u * math.cos(a) - w * math.sin(a))) < 1e-12
                assert abs(float(out[t, h, i + dims // 2]) - (w * math.cos(a) + u * math.sin(a))) < 1e-12
            assert torch.equal(out[t, h, dims:], v[t, h, dims:])
    assert torch.allclose(out[0], v[0])                     # position 0 rotates nothing


def test_router_chooses_by_corrected_score_and_weighs_by_score():
    h = torch.eye(4, dtype=torch.float64)[:1]               # one token, picks column 0 of the router
    router = torch.tensor([[2.0], [1.0], [0.0], [-1.0]], dtype=torch.float64).repeat(1, 4)
    s = torch.softmax(torch.tensor([2.0, 1.0, 0.0, -1.0], dtype=torch.float64), 0)
    ids, w = P.route(h, router, torch.zeros(4, dtype=torch.float64), 2)
    assert ids.tolist() == [[0, 1]] and torch.allclose(w[0], s[:2] / s[:2].sum())
    # a correction moves the choice to outputs 3 and 2; the weights stay the uncorrected scores
    ids, w = P.route(h, router, torch.tensor([0.0, 0.0, 1.0, 2.0], dtype=torch.float64), 2)
    assert ids.tolist() == [[3, 2]] and torch.allclose(w[0], torch.stack([s[3], s[2]]) / (s[3] + s[2]))


def test_identity_experts_return_their_input():
    rng = np.random.default_rng(1)
    W, F = 6, 4
    h = torch.tensor(rng.normal(size=(5, W)))
    w = {"router": torch.zeros(3, W, dtype=torch.float64), "correction": torch.tensor([0.0, 5.0, 4.0], dtype=torch.float64),
         "e0.gate": torch.tensor(rng.normal(size=(F, W))), "e0.up": torch.tensor(rng.normal(size=(F, W))),
         "e0.down": torch.tensor(rng.normal(size=(W, F)))}
    p = dict(router=dict(experts=1, identity=2, top=2), shared=None)
    assert torch.allclose(P.expert_mixture(h, w, p), h)     # both choices are identity experts with weight 1/2
    w["correction"] = torch.tensor([9.0, 5.0, 0.0], dtype=torch.float64)
    ref = 0.5 * h + 0.5 * P.gated_expert(h, w["e0.gate"], w["e0.up"], w["e0.down"])
    assert torch.allclose(P.expert_mixture(h, w, p), ref)


def test_attention_against_loops():
    rng = np.random.default_rng(2)
    p = C.mixer(2, 4, 6, 3, 5, base=9.0, scale=0.37)
    W, T, H, dn, dr, dv, R = 7, 6, 2, 4, 6, 3, 5
    w = {"q": rng.normal(size=(H * (dn + dr), W)), "dkv": rng.normal(size=(R + dr, W)), "dkv.norm": rng.normal(size=R),
         "uk": rng.normal(size=(H * dn, R)), "uv": rng.normal(size=(H * dv, R)), "o": rng.normal(size=(W, H * dv))}
    h = rng.normal(size=(T, W))
    eps = 1e-3
    got = P.latent_attention(torch.tensor(h), {k: torch.tensor(v) for k, v in w.items()}, p, eps).numpy()

    def rot(v, pos):
        out = v.copy()
        for i in range(dr // 2):
            a = pos * 9.0 ** (-2.0 * i / dr)
            out[i] = v[i] * math.cos(a) - v[i + dr // 2] * math.sin(a)
            out[i + dr // 2] = v[i + dr // 2] * math.cos(a) + v[i] * math.sin(a)
        return out

    lat, krot = [], []
    for t in range(T):
        d = w["dkv"] @ h[t]
        c = d[:R] / math.sqrt((d[:R] ** 2).mean() + eps) * w["dkv.norm"]
        lat.append(c)
        krot.append(rot(d[R:], t))
    for t in range(T):
        q = (w["q"] @ h[t]).reshape(H, dn + dr)
        heads = []
        for hd in range(H):
            qr = rot(q[hd, dn:], t)
            s = np.array([(q[hd, :dn] @ (w["uk"][hd * dn:(hd + 1) * dn] @ lat[j]) + qr @ krot[j]) * 0.37
                          for j in range(t + 1)])
            a = np.exp(s - s.max())
            a /= a.sum()
            heads.append(sum(a[j] * (w["uv"][hd * dv:(hd + 1) * dv] @ lat[j]) for j in range(t + 1)))
        assert np.allclose(got[t], w["o"] @ np.concatenate(heads), atol=1e-10)


def test_run_order_of_the_plain_model_and_of_the_package():
    from railgun_b200.config.dizatar import DizatarConfig
    from railgun_b200.models.dizatar import dizatar_model_spec
    for name, (cfg, _, _) in C.CASES.items():
        order = P.layer_order(cfg)
        spec = dizatar_model_spec(DizatarConfig.from_dict(cfg))
        sched = spec.run_order()
        assert [e.layer for e in sched] == [i for i, _ in order]
        assert [e.before >= 0 for e in sched] == [s for _, s in order]
        assert sorted(e.cache for e in sched) == list(range(len(sched)))        # a cache of its own for every run
    assert [i for i, _ in P.layer_order(C.CASE_P)] == [0, 1, 0, 1, 0, 1, 2]
    assert [s for _, s in P.layer_order(C.CASE_P)] == [True, False, True, False, True, False, False]
    assert [i for i, _ in P.layer_order(C.CASE_N)] == [0, 1]
    # an empty span: every layer once, nothing fed in again, the matrix still belongs to the model
    empty = {**C.CASE_P, "loop": dict(start=1, stop=1, times=3)}
    spec = dizatar_model_spec(DizatarConfig.from_dict(empty))
    assert [(e.layer, e.before) for e in spec.run_order()] == [(0, -1), (1, -1), (2, -1)]
    assert [i for i, s in P.layer_order(empty)] == [0, 1, 2] and not any(s for _, s in P.layer_order(empty))
    from railgun_b200.parts.model import expected_tensors
    assert "loop.in" in expected_tensors(spec)


def test_configuration_round_trip_and_errors():
    from railgun_b200.config.base import ConfigError
    from railgun_b200.config.dizatar import DizatarConfig
    from railgun_b200.config.registry import architecture_name, architecture_of
    for cfg, _, _ in C.CASES.values():
        c = DizatarConfig.from_dict(cfg)
        again = DizatarConfig.from_dict(json.loads(json.dumps(c.to_dict())))
        assert again == c
    assert architecture_of(architecture_name(C.CASE_P)).name == "Dizatar"
    c = DizatarConfig.from_dict(C.CASE_P)
    assert c.layers[1].mlp is None and c.layers[2].mlp.shared_ff is None and c.layers[0].mlp.identity == 2
    assert c.loop.times == 3 and DizatarConfig.from_dict(C.CASE_N).loop is None
    for breakage in (dict(width=None), dict(layers=[]), dict(loop=dict(start=2, stop=1, times=1)),
                     dict(loop=dict(start=0, stop=9, times=1)), dict(norm=None)):
        bad = {k: v for k, v in {**C.CASE_P, **breakage}.items() if v is not None}
        with pytest.raises(ConfigError):
            DizatarConfig.from_dict(bad)
    bad = json.loads(json.dumps(C.CASE_P))
    bad["layers"][0]["type"] = "something_else"
    with pytest.raises(ConfigError):
        DizatarConfig.from_dict(bad)
    bad = json.loads(json.dumps(C.CASE_P))
    bad["layers"][0]["mlp"]["router"]["top"] = 8
    with pytest.raises(ConfigError):
        DizatarConfig.from_dict(bad)


def test_tensor_list_and_random_model_folder():
    from railgun_b200.config.dizatar import DizatarConfig
    from railgun_b200.models.dizatar import dizatar_model_spec
    from railgun_b200.parts.model import expected_tensors
    from railgun_b200.weights.loader import WeightError, load_weights
    exp = expected_tensors(dizatar_model_spec(DizatarConfig.from_dict(C.CASE_P)))
    shapes = {k: tuple(v.shape) for k, v in exp.items()}
    assert shapes["embed"] == (211, 48) and shapes["head"] == (211, 48) and shapes["loop.in"] == (48, 96)
    assert shapes["l0.mix.q"] == (3 * 24, 48) and shapes["l0.mix.dkv"] == (48, 48) and shapes["l0.mix.dkv.norm"] == (40,)
    assert shapes["l0.mix.uk"] == (48, 40) and shapes["l0.mix.uv"] == (72, 40) and shapes["l0.mix.o"] == (48, 72)
    assert shapes["l0.mlp.router"] == (7, 48) and shapes["l0.mlp.correction"] == (7,)
    assert shapes["l0.mlp.e4.down"] == (48, 24) and shapes["l0.mlp.shared.gate"] == (16, 48)
    assert "l0.mlp.e5.gate" not in shapes and "l2.mlp.shared.up" not in shapes
    assert not any(k.startswith("l1.mlp") or k.startswith("l1.norm2") or k == "l1.ls2" for k in shapes)
    assert {"l1.norm1", "l1.norm1b", "l1.ls1", "final.norm"} <= set(shapes)
    assert "loop.in" not in expected_tensors(dizatar_model_spec(DizatarConfig.from_dict(C.CASE_N)))
    d = C.model_dir("P")
    loaded = load_weights(d, exp)
    assert set(loaded) == set(exp) and all(tuple(loaded[k].shape) == shapes[k] for k in exp)
    plain = C.plain_model("P")
    assert set(plain.tensors) == set(exp)
    assert torch.equal(plain.tensors["l2.mix.uk"].to(torch.bfloat16), loaded["l2.mix.uk"])
    with pytest.raises(WeightError):
        load_weights(d, {k: v for k, v in exp.items() if k != "l0.ls1"})


def test_plain_model_is_causal_and_the_cap_holds():
    plain = C.plain_model("P")
    toks = C.prompts(211, [20], seed=4)[0]
    a = plain.forward(toks)
    b = plain.forward(toks[:12] + [(t + 1) % 211 for t in toks[12:]])
    assert np.array_equal(a[:12], b[:12]) and not np.allclose(a[12:], b[12:])
    assert np.abs(a).max() < 8.0
