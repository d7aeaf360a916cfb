"""The plain statement of Rupulix against loop-level formulas, and the
package's configuration, run order and tensor list for the design (no GPU)."""
import json
import math

import numpy as np
import pytest

import plain_rupulix as P
import rupulix_cases as C


def test_rotation_layouts_pair_the_right_numbers():
    rng = np.random.default_rng(0)
    x = rng.normal(size=(5, 2, 12))
    pos = np.array([0, 1, 7, 300, 4000])
    for layout in ("half", "interleaved"):
        for dims in (0, 4, 12):
            got = P.rotate(x, pos, dims, 50.0, layout)
            for t in range(5):
                for h in range(2):
                    ref = x[t, h].copy()
                    for i in range(dims // 2):
                        a = pos[t] * 50.0 ** (-2.0 * i / dims)
                        lo, hi = (i, i + dims // 2) if layout == "half" else (2 * i, 2 * i + 1)
                        u, v = x[t, h, lo], x[t, h, hi]
                        ref[lo], ref[hi] = u * math.cos(a) - v * math.sin(a), v * math.cos(a) + u * math.sin(a)
                    assert np.allclose(got[t, h], ref, atol=1e-12)
    # a rotation keeps q . k a function of the distance only
    q, k = rng.normal(size=(1, 1, 8)), rng.normal(size=(1, 1, 8))
    d1 = (P.rotate(q, [9], 8, 10.0, "interleaved") * P.rotate(k, [4], 8, 10.0, "interleaved")).sum()
    d2 = (P.rotate(q, [105], 8, 10.0, "interleaved") * P.rotate(k, [100], 8, 10.0, "interleaved")).sum()
    assert abs(d1 - d2) < 1e-9


def test_window_and_sink():
    m = P.visible(6, 3)
    assert [int(m[5, j]) for j in range(6)] == [0, 0, 0, 1, 1, 1] and m[0, 0] and not m[2, 3]
    assert P.visible(4, 0)[3].all() and P.visible(4, 1).sum() == 4
    s = np.array([[[0.0, 0.0], [1.0, 2.0]]])
    p = P.softmax_rows(s, P.visible(2, 0)[None], sink=np.array([math.log(3.0)]))
    assert np.allclose(p[0, 0], [1.0 / 4.0, 0.0])                          # e^0 / (e^0 + 3)
    assert np.allclose(p[0, 1].sum(), (math.e + math.e ** 2) / (math.e + math.e ** 2 + 3.0))
    assert np.allclose(P.softmax_rows(s, P.visible(2, 0)[None])[0, 1].sum(), 1.0)


def test_latent_attention_against_loops():
    cfg = C.CASE_H
    w = {k: v.astype(np.float64) for k, v in C.random_tensors(cfg, 1).items()}
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    rng = np.random.default_rng(2)
    T = 14
    h = rng.normal(size=(T, cfg["width"]))
    got = P.latent_attention(h, w, "l0.mix.", m, eps)
    H, dn, dr, dv, R, win = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["mask"]["size"]
    heads = np.zeros((T, H * dv))
    lat, kr = [], []
    for t in range(T):
        down = w["l0.mix.dkv"] @ h[t]
        c = down[:R] / math.sqrt((down[:R] ** 2).mean() + eps) * w["l0.mix.dkv.norm"]
        lat.append(c)
        kr.append(P.rotate(down[None, None, R:], [t], dr, m["rot"]["base"], "interleaved")[0, 0])
    for t in range(T):
        q = (w["l0.mix.q"] @ h[t]).reshape(H, dn + dr)
        for hd in range(H):
            qr = P.rotate(q[None, None, hd, dn:], [t], dr, m["rot"]["base"], "interleaved")[0, 0]
            js = [j for j in range(T) if 0 <= t - j < win]
            sc = [m["scale"] * (q[hd, :dn] @ (w["l0.mix.uk"][hd * dn:(hd + 1) * dn] @ lat[j]) + qr @ kr[j]) for j in js]
            e = np.exp(sc)
            den = e.sum() + math.exp(w["l0.mix.sink"][hd])
            heads[t, hd * dv:(hd + 1) * dv] = sum(e[i] / den * (w["l0.mix.uv"][hd * dv:(hd + 1) * dv] @ lat[j])
                                                  for i, j in enumerate(js))
    assert np.allclose(got, heads @ w["l0.mix.o"].T, atol=1e-10)


def test_talking_attention_and_recurrence_against_loops():
    cfg = C.CASE_H
    w = {k: v.astype(np.float64) for k, v in C.random_tensors(cfg, 4).items()}
    eps = cfg["norm"]["eps"]
    rng = np.random.default_rng(5)
    T = 11
    h = rng.normal(size=(T, cfg["width"]))
    a = cfg["layers"][1]["mixer"]["left"]
    p = "l1.mix.left."
    H, G, d, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    unit = lambda v: v / math.sqrt((v ** 2).mean() + eps)
    q = np.stack([[P.rotate((unit((w[p + "q"] @ h[t])[g * d:(g + 1) * d]) * w[p + "q.norm"])[None, None], [t],
                            a["rot"]["dims"], a["rot"]["base"], "half")[0, 0] for g in range(H)] for t in range(T)])
    k = np.stack([[P.rotate((unit((w[p + "k"] @ h[t])[g * d:(g + 1) * d]) * w[p + "k.norm"])[None, None], [t],
                            a["rot"]["dims"], a["rot"]["base"], "half")[0, 0] for g in range(G)] for t in range(T)])
    v = np.stack([(w[p + "v"] @ h[t]).reshape(G, dv) for t in range(T)])
    out = np.zeros((T, H * dv))
    for t in range(T):
        raw = np.array([[a["scale"] * q[t, g] @ k[j, g // (H // G)] for j in range(t + 1)] for g in range(H)])
        mixed = w[p + "talk"] @ raw
        for hd in range(H):
            e = np.exp(mixed[hd] - mixed[hd].max())
            out[t, hd * dv:(hd + 1) * dv] = (e / e.sum()) @ v[:t + 1, hd // (H // G)]
    assert np.allclose(P.talking_attention(h, w, p, a, eps), out @ w[p + "o"].T, atol=1e-10)

    r = cfg["layers"][1]["mixer"]["right"]
    p = "l1.mix.right."
    Cw, B, K = r["width"], r["blocks"], r["conv"]
    bs = Cw // B
    xin = [w[p + "x"] @ h[t] + w[p + "x.b"] for t in range(T)]
    S, outs = np.zeros(Cw), []
    for t in range(T):
        u = w[p + "conv.b"] + sum(w[p + "conv"][:, K - 1 - j] * xin[t - j] for j in range(K) if t - j >= 0)
        gr = np.concatenate([w[p + "ra"][b] @ u[b * bs:(b + 1) * bs] + w[p + "ra.b"][b] for b in range(B)])
        gi = np.concatenate([w[p + "ri"][b] @ u[b * bs:(b + 1) * bs] + w[p + "ri.b"][b] for b in range(B)])
        aa = np.exp(-8.0 * (1 / (1 + np.exp(-gr))) * np.log1p(np.exp(w[p + "lam"])))
        S = aa * S + np.sqrt(1 - aa ** 2) * (1 / (1 + np.exp(-gi))) * u
        z = w[p + "y"] @ h[t] + w[p + "y.b"]
        outs.append(S * 0.5 * z * (1 + np.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))))
    assert np.allclose(P.gated_recurrence(h, w, p, r), np.stack(outs) @ w[p + "o"].T, atol=1e-10)


def test_hyper_connections_against_loops_and_plain_residual():
    rng = np.random.default_rng(7)
    S, T, W = 3, 4, 6
    xs = rng.normal(size=(S, T, W))
    w = {"h.in": rng.normal(size=S), "h.out": rng.normal(size=S), "h.mix": rng.normal(size=(S, S))}
    nw = rng.normal(size=W)
    fn = lambda z: z * 2.0 + 1.0
    got = P.hyper_step(xs, w, "h", nw, 1e-5, fn)
    u = sum(w["h.in"][s] * xs[s] for s in range(S))
    y = fn(P.rms_norm(u, nw, 1e-5))
    for t in range(S):
        assert np.allclose(got[t], sum(w["h.mix"][s, t] * xs[s] for s in range(S)) + w["h.out"][t] * y)
    # one copy with in = out = mix = 1 is the plain residual addition
    one = {"h.in": np.ones(1), "h.out": np.ones(1), "h.mix": np.ones((1, 1))}
    assert np.allclose(P.hyper_step(xs[:1], one, "h", nw, 1e-5, fn)[0], xs[0] + fn(P.rms_norm(xs[0], nw, 1e-5)))


def test_run_order_and_causality():
    assert P.run_order(dict(layers=[0] * 4, loop=dict(start=1, stop=3, times=2))) == [0, 1, 2, 1, 2, 3]
    assert P.run_order(dict(layers=[0] * 3)) == [0, 1, 2]
    assert P.run_order(dict(layers=[0] * 2, loop=dict(start=0, stop=2, times=3))) == [0, 1] * 3
    for name in ("H", "J"):
        cfg = C.CASES[name][0]
        w = {k: v.astype(np.float64) for k, v in C.random_tensors(cfg, 3).items()}
        ids = C.prompts(cfg["vocab"], [20], seed=1)[0]
        full, kept = P.forward(cfg, w, ids, keep_layers=True)
        assert kept.shape == (len(P.run_order(cfg)), 20, cfg["width"])
        assert np.allclose(P.forward(cfg, w, ids[:13]), full[:13], atol=1e-9)       # later tokens change nothing earlier


@pytest.mark.parametrize("name", sorted(C.CASES))
def test_configuration_round_trip_run_order_and_tensor_list(name):
    from railgun_b200.config.registry import architecture_of
    from railgun_b200.config.rupulix import RupulixConfig
    from railgun_b200.parts.model import expected_tensors
    raw = C.CASES[name][0]
    cfg = RupulixConfig.from_dict(raw)
    assert RupulixConfig.from_dict(json.loads(json.dumps(cfg.to_dict()))).to_dict() == cfg.to_dict()
    for key in ("width", "vocab", "logit_scale", "layers"):
        assert cfg.to_dict()[key] == raw[key]
    arch = architecture_of("Rupulix")
    spec = arch.model_spec(cfg)
    assert [e.layer for e in spec.run_order()] == P.run_order(raw)
    assert len({e.cache for e in spec.run_order()}) == len(spec.run_order())         # every pass its own cache
    expected = expected_tensors(spec)
    made = C.random_tensors(raw, 0)
    assert set(expected) == set(made)
    for k, ts in expected.items():
        assert tuple(ts.shape) == made[k].shape, k
    assert all(L.arrangement == ("hyper" if raw.get("streams") else "prenorm") for L in spec.layers)


def test_configuration_errors():
    from railgun_b200.config.base import ConfigError
    from railgun_b200.config.rupulix import RupulixConfig
    import copy
    good = C.CASE_H
    for path, value in ((("layers", 0, "type"), "convolution"), (("layers", 1, "mixer", "left", "kv_heads"), 3),
                        (("layers", 1, "mixer", "right", "blocks"), 5), (("loop", "stop"), 9),
                        (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 0, "mlp", "kind"), "moe"),
                        (("streams",), 0), (("norm",), None)):
        bad = copy.deepcopy(good)
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError):
            RupulixConfig.from_dict(bad)


def test_random_weights_mode_writes_a_loadable_folder(tmp_path):
    from railgun_b200.config.registry import load_config
    from railgun_b200.config.rupulix import RupulixConfig
    from railgun_b200.parts.model import expected_tensors
    from railgun_b200.weights.loader import load_weights
    from railgun_b200.weights.random_init import write_random_model
    write_random_model(RupulixConfig.from_dict(C.CASE_T), 1, tmp_path)
    arch, cfg = load_config(tmp_path)
    assert arch.name == "Rupulix"
    t = load_weights(tmp_path, expected_tensors(arch.model_spec(cfg)))
    assert abs(float(t["l1.hc1.mix"].float().diagonal().mean()) - 1.0) < 0.1       # mixing matrices start near the identity
    assert P.forward(C.CASE_T, P.read_safetensors(tmp_path / "model.safetensors"), [1, 2, 3]).shape == (3, 90)
