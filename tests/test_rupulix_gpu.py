"""Rupulix on the GPU against the plain statement: each mechanism alone, then
the model through the step function in several cuts and both precisions, then
generation through the engine, its scheduler and the command line."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import helpers
import plain_rupulix as P
import rupulix_cases as C

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = torch.device("cuda:0")
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
# bfloat16: the weights here are several times larger than a trained model's, and a few positions per hundred reach
# 3.7e-2 of the largest logit by rounding alone, the same in every cut; a lost key or state is caught by the
# tests of the mechanisms alone, where it changes a row by its whole size
TOL = {"float32": 3e-5, "bfloat16": 6e-2}


def rel(got, ref):
    got = got.double().cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got, dtype=np.float64)
    ref = ref.double().cpu().numpy() if isinstance(ref, torch.Tensor) else np.asarray(ref, dtype=np.float64)
    return np.abs(got - ref).max() / np.abs(ref).max()


def dev(x, dtype=None):
    t = torch.as_tensor(x)
    return t.to(DEV, dtype=dtype) if dtype is not None else t.to(DEV)


# ---- hyper-connections alone ------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("S,W,T", [(1, 24, 3), (2, 64, 5), (3, 100, 9), (4, 256, 300), (8, 40, 2), (2, 128, 700), (3, 36, 513)])
def test_hyper_step_alone(S, W, T, dtype):
    """The start (all copies the same), an update fused with the next read, and the fold into one stream."""
    from railgun_b200 import ops
    rng = np.random.default_rng(S * W)
    x0 = rng.normal(size=(T, W)).astype(np.float32)
    w = {f"{n}.{k}": rng.normal(size=shape).astype(np.float32) for n in ("a", "b")
         for k, shape in (("in", (S,)), ("out", (S,)), ("mix", (S, S)))}
    nw = rng.uniform(0.5, 1.5, size=W).astype(np.float32)
    y = torch.tensor(rng.normal(size=(T, W)), dtype=TORCH[dtype])
    copies = torch.empty((T, S, W), dtype=torch.float32, device=DEV)
    h = ops.hyper_step(copies, dev(x0), None, None, None, dev(w["a.in"]), dev(nw), 1e-5, TORCH[dtype])
    xs = np.stack([x0.astype(np.float64)] * S)
    assert np.array_equal(copies.cpu().numpy(), np.transpose(xs, (1, 0, 2)).astype(np.float32))
    ref_h = P.rms_norm(np.einsum("s,stw->tw", w["a.in"].astype(np.float64), xs), nw, 1e-5)
    assert rel(h, ref_h) < (1e-6 if dtype == "float32" else 5e-3)
    # the update by branch a's output, read by branch b
    h2 = ops.hyper_step(copies, None, y.to(DEV), dev(w["a.mix"]), dev(w["a.out"]), dev(w["b.in"]), dev(nw), 1e-5,
                        TORCH[dtype])
    wd = {k: v.astype(np.float64) for k, v in w.items()}
    xs2 = np.einsum("st,sjw->tjw", wd["a.mix"], xs) + wd["a.out"][:, None, None] * y.double().numpy()[None]
    assert rel(copies.transpose(0, 1), xs2) < 1e-6
    assert rel(h2, P.rms_norm(np.einsum("s,stw->tw", wd["b.in"], xs2), nw, 1e-5)) < (2e-6 if dtype == "float32" else 5e-3)
    # the fold: the plain sum of the updated copies, 32-bit
    total = ops.hyper_step(copies, None, y.to(DEV), dev(w["b.mix"]), dev(w["b.out"]), None, None, 0.0, torch.float32)
    xs3 = np.einsum("st,sjw->tjw", wd["b.mix"], xs2) + wd["b.out"][:, None, None] * y.double().numpy()[None]
    assert total.dtype == torch.float32 and rel(total, xs3.sum(0)) < 2e-6


# ---- attention kernels alone, over hand-made rows -----------------------------------------------------

def paged(rows, page, seed):
    """Rows [n, D] of one request scattered over shuffled pages: (cache [pages, page, D], block table [1, blocks])."""
    n, D = rows.shape
    blocks = -(-n // page)
    rng = np.random.default_rng(seed)
    ids = rng.permutation(blocks + 5)[:blocks]
    cache = torch.full((blocks + 5, page, D), 1e4, dtype=rows.dtype)        # a row read from a wrong place is far off
    for j in range(n):
        cache[ids[j // page], j % page] = rows[j]
    return cache, torch.tensor(ids, dtype=torch.int32)[None]


def plain_talking_rows(q, k, v, talk, scale, window):
    """q [H, d] of the request's last token over keys k [n, G, d] and values v [n, G, dv]."""
    H, G = q.shape[0], k.shape[1]
    n = k.shape[0]
    lo = max(0, n - window) if window else 0
    grp = torch.arange(H) // (H // G)
    s = torch.einsum("hd,jhd->hj", q, k[lo:, grp]) * scale
    if talk is not None:
        s = talk @ s
    return torch.einsum("hj,jhd->hd", torch.softmax(s, dim=-1), v[lo:, grp])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv,page,window", [(4, 2, 16, 8, 8, 0), (6, 3, 48, 80, 16, 0), (8, 8, 32, 32, 4, 0),
                                                  (5, 1, 24, 40, 16, 0), (16, 4, 64, 128, 32, 0), (2, 1, 16, 16, 16, 37),
                                                  (12, 2, 16, 64, 16, 100)])
def test_talking_attention_kernel_alone(H, G, d, dv, page, window, dtype):
    """The last query is made to point at one key (far back, at page borders, just inside and just outside the
    window, the first token): a key that is lost or taken from the neighbouring place changes the row by its
    whole size.  The mixing matrix is far from the identity."""
    from railgun_b200 import ops
    n = 333
    rng = np.random.default_rng(H * d + window)
    keys_at = [0, 1, page - 1, page, n - 2 * page, n - page - 1, 150, n - 2, n - 1]
    if window:
        keys_at += [n - window, n - window - 1, n - window + 1]
    talk = torch.tensor(np.eye(H) + rng.normal(0, 0.3, size=(H, H)), dtype=torch.float32)
    for key in keys_at:
        k = torch.tensor(rng.normal(size=(n, G, d)), dtype=TORCH[dtype]).double()
        v = torch.tensor(rng.normal(size=(n, G, dv)), dtype=TORCH[dtype]).double()
        q = torch.tensor(rng.normal(size=(H, d)), dtype=TORCH[dtype]).double()
        q[0] = (k[key, 0] * 4.0).to(TORCH[dtype]).double()                  # head 0 looks for that key
        ref = plain_talking_rows(q, k, v, talk.double(), d ** -0.5, window)
        rows = torch.cat([v.reshape(n, G * dv), k.reshape(n, G * d)], dim=1).to(TORCH[dtype])        # values, then keys
        cache, table = paged(rows, page, key)
        # the last token as a single token, and as the end of a portion of 70 (whose earlier queries are random)
        for portion in (1, 70):
            qs = torch.tensor(rng.normal(size=(portion, H, d)), dtype=TORCH[dtype])
            qs[-1] = q.to(TORCH[dtype])
            positions = torch.arange(n - portion, n, dtype=torch.int32)
            got = ops.talking_attention_general(dev(qs), dev(cache), dev(talk), dev(table),
                                                dev(torch.zeros(portion, dtype=torch.int32)), dev(positions), G, dv,
                                                window, d ** -0.5, out_scale=0.5)
            assert rel(got[-1].view(H, dv), ref * 0.5) < (2e-5 if dtype == "float32" else 2e-2), f"key {key}"
            if dtype == "bfloat16" and dv % 2 == 0 and ops.latent_attention_mma_ok(torch.bfloat16, H, G * dv, G * (d + dv)):
                # the tensor-core form: the mixing inside the queries, every head over the rows [values | keys]
                hpg = H // G
                mixed = torch.zeros((portion, H, G * (d + dv)), dtype=torch.float64)
                for c in range(G):
                    mixed[:, :, G * dv + c * d:G * dv + (c + 1) * d] = d ** -0.5 * torch.einsum(
                        "hg,tgd->thd", talk.double()[:, c * hpg:(c + 1) * hpg], qs.double()[:, c * hpg:(c + 1) * hpg])
                qa = dev(mixed.to(torch.bfloat16))
                for splits in ((1,) if portion > 1 else (1, 2, 5)):
                    wide = torch.zeros((portion, H * dv + 24), dtype=torch.bfloat16, device=DEV)
                    tiles = dev(torch.tensor([[0, 64, 0], [64, portion - 64, 0]], dtype=torch.int32)) if portion > 1 else None
                    ops.latent_attention_mma(qa, wide[:, 8:8 + H * dv], dev(cache), dev(table), tiles, None,
                                             2 if portion > 1 else 1,
                                             dev(torch.zeros(portion, dtype=torch.int32)), dev(positions), G * dv, window,
                                             1.0, splits, select=(dv, hpg), out_scale=0.5, score_from=G * dv)
                    assert rel(wide[-1, 8:8 + H * dv].view(H, dv), ref * 0.5) < 3e-2, f"key {key}, tensor cores, {splits} shares"
                    assert float(wide[:, :8].abs().max()) == 0.0 and float(wide[:, 8 + H * dv:].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv,dims", [(4, 2, 16, 8, 8), (6, 3, 48, 80, 48), (3, 1, 24, 40, 0), (2, 2, 64, 16, 32)])
def test_talking_prepare_alone(H, G, d, dv, dims, dtype):
    """Norm per head, rotation of part of the head in pairs (i, i + dims/2), and the cache row."""
    from railgun_b200 import ops
    from railgun_b200.parts.latent_attention import rotary_frequencies
    T, page = 9, 4
    rng = np.random.default_rng(d)
    qkv = torch.tensor(rng.normal(size=(T, (H + G) * d + G * dv)), dtype=TORCH[dtype])
    qn, kn = rng.uniform(0.5, 2, size=d), rng.uniform(0.5, 2, size=d)
    pos = np.array([0, 1, 2, 3, 500, 501, 70000, 5, 6])
    slots = torch.tensor([5, 4, -1, 7, 0, 1, 2, 11, 3], dtype=torch.int32)
    cache = torch.zeros((3, page, G * (d + dv)), dtype=TORCH[dtype], device=DEV)
    q_out = torch.empty((T, H, d), dtype=TORCH[dtype], device=DEV)
    ops.talking_prepare(dev(qkv), q_out, cache, dev(qn, torch.float32), dev(kn, torch.float32), 1e-5,
                        rotary_frequencies(dims, 300.0).to(DEV), dims, dev(pos.astype(np.int32)), dev(slots), H, G, d, dv)
    x = qkv.double().numpy()
    q_ref = P.rotate(P.rms_norm(x[:, :H * d].reshape(T, H, d), qn, 1e-5), pos, dims, 300.0, "half")
    k_ref = P.rotate(P.rms_norm(x[:, H * d:(H + G) * d].reshape(T, G, d), kn, 1e-5), pos, dims, 300.0, "half")
    tol = 2e-6 if dtype == "float32" else 8e-3
    assert rel(q_out, q_ref) < tol
    flat = cache.view(-1, G * (d + dv)).cpu()
    for t in range(T):
        if slots[t] >= 0:
            assert rel(flat[slots[t], G * dv:], k_ref[t].reshape(-1)) < tol
            assert torch.equal(flat[slots[t], :G * dv], qkv[t, (H + G) * d:])
    assert float(flat[8].abs().max()) == 0.0 and float(flat[6].abs().max()) == 0.0          # untouched rows
    # the queries of the tensor-core form: zeros, then per key/value head the mixed and scaled queries of its heads
    talk = rng.normal(size=(H, H))
    qa = torch.empty((T, H, G * (d + dv)), dtype=TORCH[dtype], device=DEV)
    ops.talking_prepare(dev(qkv), None, None, dev(qn, torch.float32), dev(kn, torch.float32), 1e-5,
                        rotary_frequencies(dims, 300.0).to(DEV), dims, dev(pos.astype(np.int32)), None, H, G, d, dv,
                        qa=qa, talk=dev(talk, torch.float32), scale=0.3)
    hpg = H // G
    ref = np.zeros((T, H, G * (d + dv)))
    for c in range(G):
        ref[:, :, G * dv + c * d:G * dv + (c + 1) * d] = 0.3 * np.einsum(
            "hg,tgd->thd", talk.astype(np.float32)[:, c * hpg:(c + 1) * hpg], q_ref[:, c * hpg:(c + 1) * hpg])
    assert rel(qa, ref) < tol and float(qa[:, :, :G * dv].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,R,dr,page,window", [(3, 40, 8, 8, 9), (8, 64, 16, 16, 37), (4, 16, 16, 4, 0),
                                                (16, 128, 32, 16, 50), (3, 96, 32, 32, 200)])
def test_latent_attention_with_sink_and_window_alone(H, R, dr, page, window, dtype):
    """The sink alone decides a head when it is large, and does nothing when it is very negative; keys just inside
    and just outside the window, at page borders and far back, for single tokens and the ends of portions."""
    from railgun_b200 import ops
    n, D = 300, R + dr
    rng = np.random.default_rng(R + window)
    keys_at = [0, page, n - page - 1, 123, n - 1]
    if window:
        keys_at += [n - window, n - window - 1, n - window + 1]
    for key in keys_at:
        rows = torch.tensor(rng.normal(size=(n, D)), dtype=TORCH[dtype])
        qa = torch.tensor(rng.normal(size=(H, D)), dtype=TORCH[dtype])
        qa[0] = rows[key] * 3.0
        sink = torch.tensor(rng.normal(0, 2, size=H), dtype=torch.float32)
        sink[1], sink[-1] = 60.0, -60.0
        lo = max(0, n - window) if window else 0
        s = (qa.double() @ rows.double()[lo:].T) * 0.2
        e = torch.exp(s - s.max(dim=1, keepdim=True).values)
        den = e.sum(1, keepdim=True) + torch.exp(sink.double()[:, None] - s.max(dim=1, keepdim=True).values)
        ref = (e / den) @ rows.double()[lo:, :R]
        cache, table = paged(rows, page, key)
        for portion in (1, 33):
            qs = torch.tensor(rng.normal(size=(portion, H, D)), dtype=TORCH[dtype])
            qs[-1] = qa
            positions = torch.arange(n - portion, n, dtype=torch.int32)
            got = ops.latent_attention_general(dev(qs), dev(cache), dev(table), dev(torch.zeros(portion, dtype=torch.int32)),
                                               dev(positions), R, window, 0.2, dev(sink))
            err = np.abs(got[-1].double().cpu().numpy() - ref.numpy()).max() / float(rows[:, :R].double().abs().max())
            assert err < (2e-5 if dtype == "float32" else 2e-2), f"key {key}"
            assert float(got[-1, 1].abs().max()) < 1e-6                                    # all weight on the sink
            if dtype == "bfloat16" and ops.latent_attention_mma_ok(torch.bfloat16, H, R, D):
                for splits in ((1,) if portion > 1 else (1, 3)):
                    out = torch.empty((portion, H, R), dtype=torch.bfloat16, device=DEV)
                    tiles = dev(torch.tensor([[0, portion, 0]], dtype=torch.int32)) if portion > 1 else None
                    ops.latent_attention_mma(dev(qs), out, dev(cache), dev(table), tiles, None, 1,
                                             dev(torch.zeros(portion, dtype=torch.int32)), dev(positions), R, window, 0.2,
                                             splits, sink=dev(sink))
                    err = np.abs(out[-1].double().cpu().numpy() - ref.numpy()).max() / float(rows[:, :R].double().abs().max())
                    assert err < 3e-2, f"key {key}, tensor cores, {splits} shares"
                    assert float(out[-1, 1].abs().max()) < 1e-6


# ---- mixers alone, through the cache and the state ----------------------------------------------------

def feed_part(runner, part, view, h, cuts, rid=1):
    """Rows ``h`` [T, W] through one mixer in steps that end at ``cuts``."""
    from railgun_b200.engine.batch import StepEntry, build_step_batch
    outs, start = [], 0
    for end in list(cuts) + [h.shape[0]]:
        if end <= start:
            continue
        entries = [StepEntry(rid, [0] * (end - start), [])]
        batch = build_step_batch(entries, runner.alloc, runner.page_sizes, runner.model.vocab_size,
                                 runner.model.spec.max_position, runner.device, runner.err_flag)
        outs.append(part.forward(h[start:end].contiguous(), batch, view).float())
        runner._commit(entries, batch)
        start = end
    runner.check_device_errors()
    runner.end([rid])
    return torch.cat(outs)


CUTS = ((), (1,), (2, 4, 145), (9, 25, 147, 148, 149), tuple(range(1, 150, 7)))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("H", 1), ("H", 2), ("J", 0), ("J", 2), ("L", 0), ("T", 1)])
def test_parallel_mixer_and_its_branches_alone(name, layer, dtype):
    """The talking-heads attention alone, the recurrence alone (state and convolution tail carried over cuts
    down to one token; a slot that another request used before), and both side by side.  One far row is scaled
    so that its value stands out."""
    from railgun_b200.engine.runner import ModelRunner
    cfg, _, page = C.CASES[name]
    plain = C.plain_model(name)
    m, eps, W = cfg["layers"][layer]["mixer"], cfg["norm"]["eps"], cfg["width"]
    runner = ModelRunner(C.model_dir(name), dtype=dtype, page_size=page, max_tokens=256, max_requests=2)
    cache_id = [e.cache for e in runner.model.order if e.layer == layer][0]
    mixer, view = runner.model.layers[layer].mixer, runner.views.view(cache_id)
    rng = np.random.default_rng(layer)
    h = torch.tensor(rng.normal(size=(150, W)), dtype=torch.float32).to(TORCH[dtype])
    h[3] *= 8.0
    hd = h.double().numpy()
    p = f"l{layer}.mix."
    refs = [(mixer.parts[0], view.parts[0], P.talking_attention(hd, plain.w, p + "left.", m["left"], eps)),
            (mixer.parts[1], view.parts[1], P.gated_recurrence(hd, plain.w, p + "right.", m["right"])),
            (mixer, view, P.parallel_mixer(hd, plain.w, p, m, eps))]
    junk = torch.tensor(rng.normal(size=(11, W)) * 5, dtype=torch.float32).to(TORCH[dtype]).to(DEV)
    for part, v, ref in refs:
        for cuts in CUTS:
            feed_part(runner, part, v, junk, (4,), rid=7)                  # leaves pages and the slot dirty
            got = feed_part(runner, part, v, h.to(DEV), cuts)
            assert rel(got, ref) < TOL[dtype], f"{type(part).__name__}, cuts {cuts}"
    runner.alloc.check()


def test_recurrence_remembers_far_tokens_through_many_single_steps():
    """Decays a hair below one: the first token's input is still most of the state after 400 single-token steps."""
    from railgun_b200.engine.runner import ModelRunner
    import tempfile

    def slow(t):
        for k in t:
            if k.endswith("right.lam"):
                t[k][:] = -9.0
    d = C.write_model(C.CASE_T, 4, tempfile.mkdtemp(prefix="rg_rupulix_slow_"), change=slow)
    plain = C.Plain(d)
    cfg = C.CASE_T
    runner = ModelRunner(d, dtype="float32", page_size=16, max_tokens=512, max_requests=2)
    mixer, view = runner.model.layers[1].mixer.parts[1], runner.views.view(1).parts[1]
    rng = np.random.default_rng(0)
    h = torch.tensor(rng.normal(size=(400, cfg["width"])) * 0.05, dtype=torch.float32)
    h[0] *= 400.0
    ref = P.gated_recurrence(h.double().numpy(), plain.w, "l1.mix.right.", cfg["layers"][1]["mixer"]["right"])
    without = P.gated_recurrence(h[1:].double().numpy(), plain.w, "l1.mix.right.", cfg["layers"][1]["mixer"]["right"])
    assert np.abs(ref[-1] - without[-1]).max() > 0.3 * np.abs(ref[-1]).max()              # the first token matters
    got = feed_part(runner, mixer, view, h.to(DEV), tuple(range(1, 400)))
    assert rel(got, ref) < 3e-5 and rel(got[-1], ref[-1]) < 3e-5


def test_convolution_continues_from_the_state_and_splits_u_into_two_halves():
    """The convolution of two requests side by side (one new, one that continues from its slot's tail), and u as
    two bfloat16 numbers whose sum is u to 2^-16: what the gates' tensor-core products are fed."""
    from types import SimpleNamespace
    from railgun_b200 import ops
    rng = np.random.default_rng(3)
    C, K, B, n0, n1 = 48, 4, 3, 5, 7
    proj = torch.tensor(rng.normal(size=(n0 + n1, 2 * C)), dtype=torch.bfloat16)
    xb, cb = rng.normal(size=C) * 0.3, rng.normal(size=C) * 0.3
    taps = rng.normal(size=(C, K))
    state = torch.tensor(rng.normal(size=(3, K, C)), dtype=torch.float32)
    batch = SimpleNamespace(cu_seqlens=dev(torch.tensor([0, n0, n0 + n1], dtype=torch.int32)),
                            req_of_token=dev(torch.tensor([0] * n0 + [1] * n1, dtype=torch.int32)),
                            start_pos=dev(torch.tensor([0, 9], dtype=torch.int32)),
                            state_slots=dev(torch.tensor([2, 1], dtype=torch.int32)))
    u, halves = ops.recurrent_conv(dev(proj), C, dev(xb, torch.float32), dev(taps, torch.float32), dev(cb, torch.float32),
                                   dev(state), batch, halves_blocks=B)
    xin = proj.double().numpy()[:, C:] + xb
    ref0 = P.causal_conv(xin[:n0], taps, cb)                                              # starts from zeros
    ref1 = P.causal_conv(np.concatenate([state[1, :K - 1].double().numpy(), xin[n0:]]), taps, cb)[K - 1:]
    assert rel(u, np.concatenate([ref0, ref1])) < 2e-6
    both = halves.float().view(n0 + n1, B, 2, C // B)
    assert rel((both[:, :, 0] + both[:, :, 1]).reshape(n0 + n1, C), u) < 2e-5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("H", 0), ("K", 0), ("K", 2), ("L", 1), ("T", 0), ("J", 1)])
def test_latent_mixer_alone(name, layer, dtype):
    from railgun_b200.engine.runner import ModelRunner
    cfg, _, page = C.CASES[name]
    plain = C.plain_model(name)
    runner = ModelRunner(C.model_dir(name), dtype=dtype, page_size=page, max_tokens=256, max_requests=2)
    cache_id = [e.cache for e in runner.model.order if e.layer == layer][0]
    rng = np.random.default_rng(layer)
    h = torch.tensor(rng.normal(size=(150, cfg["width"])), dtype=torch.float32).to(TORCH[dtype])
    ref = P.latent_attention(h.double().numpy(), plain.w, f"l{layer}.mix.", cfg["layers"][layer]["mixer"], cfg["norm"]["eps"])
    for cuts in CUTS:
        got = feed_part(runner, runner.model.layers[layer].mixer, runner.views.view(cache_id), h.to(DEV), cuts)
        assert rel(got, ref) < TOL[dtype], f"cuts {cuts}"
    runner.alloc.check()


@pytest.mark.parametrize("dtype", DTYPES)
def test_dense_feed_forward_alone(dtype):
    from railgun_b200 import ops
    from railgun_b200.engine.runner import ModelRunner
    runner = ModelRunner(C.model_dir("H"), dtype=dtype, page_size=8, max_tokens=64, max_requests=1)
    plain = C.plain_model("H")
    rng = np.random.default_rng(1)
    for T in (1, 5, 70):
        h = torch.tensor(rng.normal(size=(T, 64)), dtype=torch.float32).to(TORCH[dtype])
        got = runner.model.layers[0].ffn.forward(h.to(DEV), None)
        assert rel(got, P.feed_forward(h.double().numpy(), plain.w, "l0.")) < TOL[dtype]
    z = torch.linspace(-4, 4, 1003, dtype=torch.float32)
    for kind, fn in (("relu2", lambda v: np.maximum(v, 0) ** 2), ("relu", lambda v: np.maximum(v, 0)),
                     ("gelu_tanh", P.gelu_tanh), ("silu", lambda v: v * P.sigmoid(v))):
        assert rel(ops.activation(z.to(DEV), kind, in_place=False), fn(z.double().numpy())) < 1e-6


# ---- the model through the step function --------------------------------------------------------------

LENGTHS = {"H": [5, 17, 33, 70, 100, 131, 64, 48], "J": [1, 2, 9, 40, 90, 3], "K": [1, 2, 9, 40, 3],
           "L": [300, 392, 129, 257, 64, 395], "T": [3, 90, 150, 64, 33]}
PORTIONS = {"L": (130, 2, 64, 7, 128, 3, 65, 2, 33, 129)}
MIXED = {"L": (5, 1, 2, 70, 1, 1, 3, 140, 1, 2, 128, 17)}
_oracle: dict = {}


def oracle(name):
    if name not in _oracle:
        cfg = C.CASES[name][0]
        reqs = {f"r{i}": p for i, p in enumerate(C.prompts(cfg["vocab"], LENGTHS[name], seed=21))}
        plain = C.plain_model(name)
        _oracle[name] = (reqs, {k: plain.forward(v) for k, v in reqs.items()})
    return _oracle[name]


def make_trace(mode, reqs, name):
    if mode == "whole":
        return helpers.trace_whole(reqs)
    if mode == "tail":
        return helpers.trace_tail_decode(reqs, 32)
    if mode == "every_token":
        return helpers.trace_tail_decode(reqs, 10 ** 6)
    if mode == "portions":
        return helpers.trace_portions(reqs, **({"sizes": PORTIONS[name]} if name in PORTIONS else {}))
    if mode == "mixed":
        return helpers.trace_mixed(reqs, max_live=4, seed=5, **({"sizes": MIXED[name]} if name in MIXED else {}))
    raise ValueError(mode)


def replay(name, dtype, steps, out_dir, page=None, **more):
    from railgun_b200.engine.runner import ModelRunner
    from railgun_b200.replay import Replayer
    runner = ModelRunner(C.model_dir(name), dtype=dtype, page_size=page or C.CASES[name][2],
                         max_tokens=helpers.peak_tokens(steps, 64), max_requests=4, **more)
    rp = Replayer(runner, out_dir)
    for s in steps:
        rp.feed(s)
    runner.check_device_errors()
    runner.alloc.check()
    assert runner.alloc.num_requests() == 0
    return helpers.collect(steps, out_dir, C.CASES[name][0]["vocab"])


def compare(rows, reqs, logits, dtype, what):
    worst = 0.0
    for name, toks in reqs.items():
        ref = logits[name]
        scale = np.abs(ref).max()
        for p in range(len(toks)):
            err = np.abs(rows[(name, p)] - ref[p]).max() / scale
            assert err <= TOL[dtype], (f"{what}: request {name} (length {len(toks)}) first differs at position {p}: "
                                       f"relative error {err:.3e}")
            worst = max(worst, err)
    return worst


@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", sorted(C.CASES))
def test_replay_matches_plain(name, dtype, mode, tmp_path):
    """Whole prompts; the last 32 tokens one by one; portions down to two tokens, cut inside pages and windows;
    up to four live requests in a pool so small that pages and slots are used again."""
    reqs, logits = oracle(name)
    rows = replay(name, dtype, make_trace(mode, reqs, name), tmp_path)
    print(f"{name} {dtype} {mode}: worst relative error {compare(rows, reqs, logits, dtype, f'{name} {dtype} {mode}'):.3e}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["H", "T"])
def test_every_token_decoded_alone_matches_whole_prompts(name, dtype, tmp_path):
    """Token-by-token decoding from the first token on (up to 150 single steps through the decode graphs: the
    windows pass over decoded tokens) against the plain logits of the whole prompt, and with graphs off."""
    reqs, logits = oracle(name)
    few = dict(list(reqs.items())[2:5])
    steps = make_trace("every_token", few, name)
    compare(replay(name, dtype, steps, tmp_path / "g"), few, logits, dtype, "decoded")
    compare(replay(name, dtype, steps, tmp_path / "e", use_graphs=False), few, logits, dtype, "decoded, no graphs")


@pytest.mark.parametrize("page", [2, 64])
def test_other_page_sizes(page, tmp_path):
    reqs, logits = oracle("H")
    for mode in ("portions", "mixed"):
        steps = make_trace(mode, reqs, "H")
        compare(replay("H", "float32", steps, tmp_path / mode, page=page), reqs, logits, "float32", f"page {page}")


def test_batch_of_unequal_requests_equals_each_alone(tmp_path):
    """One step with four prompts of unequal length beside one another, then single tokens of all four in one
    step: the rows equal those of each request run alone."""
    reqs, logits = oracle("H")
    names = list(reqs)[:4]
    together = [{"step": 0, "entries": [{"id": n, "tokens": reqs[n][:-1], "want": list(range(len(reqs[n]) - 1))}
                                         for n in names], "end": []},
                {"step": 1, "entries": [{"id": n, "tokens": reqs[n][-1:], "want": [0]} for n in names], "end": names}]
    alone, k = [], 0
    for n in names:
        alone.append({"step": k, "entries": [{"id": n, "tokens": reqs[n][:-1], "want": list(range(len(reqs[n]) - 1))}],
                      "end": []})
        alone.append({"step": k + 1, "entries": [{"id": n, "tokens": reqs[n][-1:], "want": [0]}], "end": [n]})
        k += 2
    for dtype in DTYPES:
        a = replay("H", dtype, together, tmp_path / f"t{dtype}")
        b = replay("H", dtype, alone, tmp_path / f"a{dtype}")
        compare(a, {n: reqs[n] for n in names}, logits, dtype, "together")
        for key in a:
            assert np.abs(a[key] - b[key]).max() <= (2e-5 if dtype == "float32" else 0.25) * np.abs(b[key]).max(), key


# ---- generation through the engine and the command line -----------------------------------------------

def greedy_consistent(plain, prompt, out, tol):
    """How many generated tokens are the plain model's choice given the tokens before them (teacher-forced), up
    to ``tol`` of the largest absolute logit."""
    logits = plain.forward(list(prompt) + list(out))
    return sum(int(logits[len(prompt) - 1 + i][t] >= logits[len(prompt) - 1 + i].max() - tol * np.abs(logits).max())
               for i, t in enumerate(out))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["H", "J"])
def test_greedy_generation_through_the_engine(name, dtype):
    """Prompts of one token and more, prefilled in portions by the scheduler beside decoding requests."""
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    cfg, _, page = C.CASES[name]
    prompts = C.prompts(cfg["vocab"], [1, 2, 9, 40, 63, 100], seed=2)
    plain = C.plain_model(name)
    eng = Engine(C.model_dir(name), dtype=dtype, block_size=page, num_gpu_blocks=1024 // page, max_num_seqs=4,
                 max_num_batched_tokens=64, max_prefill_chunk=24, max_model_len=256)
    outs = eng.generate(prompts, SamplingParams(max_new_tokens=10))
    good = 0
    for p, o in zip(prompts, outs):
        assert o.finish_reason == "max_tokens" and len(o.token_ids) == 10
        good += greedy_consistent(plain, p, o.token_ids, 1e-4 if dtype == "float32" else 6e-2)
        if dtype == "float32":
            assert o.token_ids == plain.greedy(p, 10)
    assert good == 60
    assert eng.stats()["num_free_blocks"] == 1024 // page and not eng.has_unfinished()


def test_long_decoding_through_the_engine():
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    cfg, _, page = C.CASES["K"]
    plain = C.plain_model("K")
    prompt = C.prompts(cfg["vocab"], [3], seed=8)[0]
    eng = Engine(C.model_dir("K"), dtype="float32", block_size=page, num_gpu_blocks=100, max_num_seqs=2,
                 max_model_len=400)
    out = eng.generate([prompt], SamplingParams(max_new_tokens=300))[0]
    assert len(out.token_ids) == 300
    assert greedy_consistent(plain, prompt, out.token_ids, 1e-4) == 300


def test_command_line_and_trace_runner(tmp_path):
    d = C.model_dir("T")
    plain = C.plain_model("T")
    prompt = [7, 80, 3, 55]
    res = subprocess.run([sys.executable, "-m", "railgun_b200", "generate", "-m", str(d), "--prompt-ids",
                          ",".join(map(str, prompt)), "--max-tokens", "6", "--dtype", "f32", "--block-size", "8"],
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l and l[0].isdigit()][0]
    assert [int(t) for t in line.split(",")] == plain.greedy(prompt, 6)
    toks = C.prompts(90, [30], seed=6)[0]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:19], "want": [0, 18]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[19:21], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[21:], "want": [8]}], "end": ["a"]}]
    res = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(d), "--dtype", "float32", "--out",
                          str(tmp_path), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = plain.forward(toks)
    got0 = np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(2, 90)
    got2 = np.fromfile(tmp_path / "2.f32", dtype="<f4").reshape(1, 90)
    assert not (tmp_path / "1.f32").exists()
    scale = np.abs(ref).max()
    assert np.abs(got0 - ref[[0, 18]]).max() < 1e-4 * scale and np.abs(got2[0] - ref[29]).max() < 1e-4 * scale
