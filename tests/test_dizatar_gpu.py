"""Dizatar on the GPU against the plain statement: each mechanism alone, then
the model through the step function in four cuts and both precisions, then
generation through the engine, its scheduler and the command line."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import dizatar_cases as C
import helpers
import plain_dizatar as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DEV = torch.device("cuda:0")
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 3e-5, "bfloat16": 3e-2}
# the mixer alone is fed rows scaled by 12: scores in the hundreds, which bfloat16 operands round by several
# tenths; a lost key there changes the row by its whole size
TOL_MIXER = {"float32": 3e-5, "bfloat16": 0.1}
# In bfloat16 the residual stream differs from the plain one by rounding, and a router whose choice is within
# a few percent of a tie may then choose another expert: such positions (``route_margin`` below this) are held to
# a loose bound only.  The 32-bit runs hold every position to the tight one.
CLEAR_MARGIN = 0.08


def rel(got, ref):
    got = got.double().cpu().numpy() if isinstance(got, torch.Tensor) else np.asarray(got, dtype=np.float64)
    ref = ref.double().numpy() if isinstance(ref, torch.Tensor) else np.asarray(ref, dtype=np.float64)
    return np.abs(got - ref).max() / np.abs(ref).max()


def bank_of(tensors, dtype):
    from railgun_b200.parts.model import TensorBank
    return TensorBank({k: v.to(torch.float32).to(dtype) for k, v in tensors.items()}, DEV)


def env_of(dtype, width):
    from railgun_b200.parts.spec import BuildEnv
    return BuildEnv(device=DEV, dtype=dtype, hidden_size=width, max_position=1 << 20)


def rounded(tensors, dtype):
    return {k: v.to(torch.float32).to(dtype).double() for k, v in tensors.items()}


# ---- the mixer alone ----------------------------------------------------------------------------------

def feed_mixer(runner, layer, cache_id, h, cuts, rid=1):
    """Rows ``h`` [T, W] through one layer's mixer in steps that end at ``cuts``."""
    from railgun_b200.engine.batch import StepEntry, build_step_batch
    mix = runner.model.layers[layer].mixer
    outs, start = [], 0
    for end in list(cuts) + [h.shape[0]]:
        if end <= start:
            continue
        entries = [StepEntry(rid, [0] * (end - start), [])]
        batch = build_step_batch(entries, runner.alloc, runner.page_sizes, runner.model.vocab_size,
                                 runner.model.spec.max_position, runner.device, runner.err_flag)
        outs.append(mix.forward(h[start:end].contiguous(), batch, runner.views.view(cache_id)).float())
        runner._commit(entries, batch)
        start = end
    runner.check_device_errors()
    runner.end([rid])
    return torch.cat(outs)


def mixer_weights(name, layer):
    plain = C.plain_model(name)
    return P.sub({k: v.double() for k, v in plain.tensors.items()}, f"l{layer}.mix."), plain.cfg


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("P", 0), ("P", 2), ("Q", 0), ("N", 0), ("M", 0)])
def test_mixer_alone_with_one_key_that_stands_out(name, layer, dtype):
    """Random rows with one key (at a page's first or last place, the very first token, far back) and the last
    query scaled so that this pair's score dominates: a key that is lost, or read from the neighbouring place,
    changes the result by far more than rounding.  Whole in one step, in portions cut inside pages, and with the
    last tokens as single steps."""
    from railgun_b200.engine.runner import ModelRunner
    cfg, _, page = C.CASES[name]
    w, _ = mixer_weights(name, layer)
    p = cfg["layers"][layer]["mixer"]
    T, W = 150, cfg["width"]
    runner = ModelRunner(C.model_dir(name), dtype=dtype, page_size=page, max_tokens=256, max_requests=2)
    cache_id = [e.cache for e in runner.model.order if e.layer == layer][0]
    rng = np.random.default_rng(layer)
    stood_out = 0
    for key in (0, 1, page - 1, page, 3 * page - 1, 3 * page, T - 2 * page, T - page - 1, 37, T - 2):
        base = torch.tensor(rng.normal(size=(T, W)), dtype=torch.float32).to(TORCH[dtype])
        best = None
        for sign in (1.0, -1.0):
            h = base.clone()
            h[key] *= 12.0 * sign
            h[T - 1] *= 12.0
            ref, att = P.latent_attention(h.double(), w, p, cfg["norm"]["eps"], return_weights=True)
            peak = float(att[:, T - 1, key].max())
            if best is None or peak > best[0]:
                best = (peak, h, ref)
        peak, h, ref = best
        stood_out += peak > 0.5
        hd = h.to(DEV)
        for cuts in ((), (key + 1, T - 3, T - 2, T - 1), (page + 3, 2 * page + 5, T - 1), (2, 4, T - 5)):
            got = feed_mixer(runner, layer, cache_id, hd, cuts)
            assert rel(got, ref) < TOL_MIXER[dtype], f"key {key}, cuts {cuts}"
            assert rel(got[T - 1], ref[T - 1]) < TOL_MIXER[dtype], f"last row, key {key}, cuts {cuts}"
    assert stood_out >= 6
    runner.alloc.check()


# ---- router, experts, norms -----------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("N,top,W", [(7, 2, 40), (18, 5, 200), (3, 3, 24), (40, 6, 72), (2, 1, 16)])
def test_router_alone(N, top, W, dtype):
    from railgun_b200 import ops
    rng = np.random.default_rng(N)
    x = torch.tensor(rng.normal(size=(33, W)), dtype=torch.float32).to(TORCH[dtype])
    router = torch.tensor(rng.normal(size=(N, W)) * 0.3, dtype=torch.float32)
    corr = torch.tensor(rng.normal(size=N) * 0.2, dtype=torch.float32)
    ids, wts = ops.moe_route(x.to(DEV), router.to(DEV), corr.to(DEV), top)
    scores = torch.softmax(x.double() @ router.double().T, -1)
    choice = scores + corr.double()
    ref_ids, ref_w = P.route(x.double(), router.double(), corr.double(), top)
    order = torch.sort(choice, dim=-1, descending=True).values
    clear = (order[:, :-1] - order[:, 1:]).min(dim=-1).values > 1e-5 if N > 1 else torch.ones(33, dtype=torch.bool)
    assert int(clear.sum()) > 20
    assert torch.equal(ids.cpu()[clear].long(), ref_ids[clear])
    assert torch.allclose(wts.cpu().double()[clear], ref_w[clear], atol=2e-6)
    assert torch.allclose(wts.sum(-1).cpu(), torch.ones(33), atol=1e-5)


def mixture_tensors(rng, W, E, ident, F, shared):
    t = {"l.mlp.router": torch.tensor(rng.normal(size=(E + ident, W)) * 0.3),
         "l.mlp.correction": torch.tensor(rng.normal(size=E + ident) * 0.1)}
    for e in range(E):
        t[f"l.mlp.e{e}.gate"] = torch.tensor(rng.normal(size=(F, W)) * 0.2)
        t[f"l.mlp.e{e}.up"] = torch.tensor(rng.normal(size=(F, W)) * 0.2)
        t[f"l.mlp.e{e}.down"] = torch.tensor(rng.normal(size=(W, F)) * 0.2)
    if shared:
        t["l.mlp.shared.gate"] = torch.tensor(rng.normal(size=(shared, W)) * 0.2)
        t["l.mlp.shared.up"] = torch.tensor(rng.normal(size=(shared, W)) * 0.2)
        t["l.mlp.shared.down"] = torch.tensor(rng.normal(size=(W, shared)) * 0.2)
    return t


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W,E,ident,top,F,shared,T", [
    (40, 5, 2, 3, 24, 16, 50), (64, 8, 0, 2, 48, None, 200), (32, 1, 3, 2, 16, 32, 9), (128, 16, 4, 4, 64, 64, 700),
    (48, 3, 1, 4, 72, 8, 1), (256, 10, 3, 5, 80, 112, 65)])
def test_expert_mixture_alone(W, E, ident, top, F, shared, T, dtype):
    """The feed-forward part against the plain mixture; the correction is set so that identity experts are
    chosen for many tokens, and every expert gets rows (some none, with few tokens)."""
    from railgun_b200.parts.registry import FEED_FORWARDS
    rng = np.random.default_rng(W + T)
    t = mixture_tensors(rng, W, E, ident, F, shared)
    if ident:
        t["l.mlp.correction"][E:] += 0.05
    p = dict(hidden_size=W, experts=E, identity=ident, top=top, expert_size=F, shared_size=shared, base="mlp.")
    cls = FEED_FORWARDS.get("routed_experts")
    assert {k: tuple(v.shape) for k, v in cls.tensor_specs(p, "l.").items()} == {k: tuple(v.shape) for k, v in t.items()}
    dt = TORCH[dtype]
    part = cls(p, "l.", env_of(dt, W), bank_of(t, dt))
    x = torch.tensor(rng.normal(size=(T, W)), dtype=torch.float32).to(dt)
    r = rounded(t, dt)
    r["l.mlp.router"], r["l.mlp.correction"] = t["l.mlp.router"].float().double(), t["l.mlp.correction"].float().double()
    if dt == torch.bfloat16:          # the part holds router and correction in 32-bit, of the stored (rounded) values
        r["l.mlp.router"] = t["l.mlp.router"].float().to(dt).double()
        r["l.mlp.correction"] = t["l.mlp.correction"].float().to(dt).double()
    plain_p = dict(router=dict(experts=E, identity=ident, top=top), shared=dict(ff=shared) if shared else None)
    ref = P.expert_mixture(x.double(), P.sub(r, "l.mlp."), plain_p)
    chosen, _ = P.route(x.double(), r["l.mlp.router"], r["l.mlp.correction"], top)
    if ident and T >= 9:
        assert int((chosen >= E).sum()) > 0
    got = part.forward(x.to(DEV), None)
    assert got.dtype == torch.float32 and rel(got, ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H", [48, 320, 1000])
def test_post_norm_addition_and_next_norm_in_one_pass(H, dtype):
    from railgun_b200 import ops
    rng = np.random.default_rng(H)
    dt = TORCH[dtype]
    resid = torch.tensor(rng.normal(size=(7, H)), dtype=torch.float32)
    y = torch.tensor(rng.normal(size=(7, H)) * 3, dtype=torch.float32).to(dt)
    wb = torch.tensor(1 + 0.3 * rng.normal(size=H), dtype=torch.float32)
    wn = torch.tensor(1 + 0.3 * rng.normal(size=H), dtype=torch.float32)
    new = resid.double() + P.rms_norm(y.double(), wb.double(), 1e-5)
    ref = P.rms_norm(new, wn.double(), 2e-6)
    r = resid.to(DEV)
    out = ops.add_postnorm_rmsnorm(r, ops.PendingNormed(y.to(DEV), wb.to(DEV), 1e-5), wn.to(DEV), 2e-6, dt)
    assert rel(r, new) < 1e-6 and out.dtype == dt and rel(out, ref) < (1e-6 if dtype == "float32" else 8e-3)
    # selected rows: the sum is not written back, the rows come out normed
    r2 = resid.to(DEV)
    rows = torch.tensor([5, 0], dtype=torch.int32, device=DEV)
    out2 = ops.add_postnorm_rmsnorm(r2, ops.PendingNormed(y.to(DEV), wb.to(DEV), 1e-5), wn.to(DEV), 2e-6, dt, rows)
    assert torch.equal(r2.cpu(), resid) and rel(out2, ref[[5, 0]]) < (1e-6 if dtype == "float32" else 8e-3)
    assert rel(ops.PendingNormed(y.to(DEV), wb.to(DEV), 1e-5).materialize(), P.rms_norm(y.double(), wb.double(), 1e-5)) < 1e-6


def test_soft_cap():
    from railgun_b200 import ops
    z = torch.linspace(-90, 90, 1001, dtype=torch.float32)
    got = ops.softcap_(z.clone().to(DEV), 7.5)
    assert rel(got, P.softcap(z.double(), 7.5)) < 1e-6 and float(got.abs().max()) <= 7.5


# ---- the model through the step function ----------------------------------------------------------------

LENGTHS = {"P": [5, 17, 33, 70, 100, 131, 64, 48], "Q": [300, 392, 129, 257, 64, 395], "S": [1, 2, 9, 40, 3],
           "N": [3, 90, 150, 64, 33], "M": [2, 66, 190, 31, 128], "A": [150, 7, 65, 99]}
PORTIONS = {"Q": (130, 2, 64, 7, 128, 3, 65, 2, 33, 129)}
MIXED = {"Q": (5, 1, 2, 70, 1, 1, 3, 140, 1, 2, 128, 17)}
_oracle: dict = {}
_margins: dict = {}


def oracle(name):
    if name not in _oracle:
        cfg = C.CASES[name][0]
        reqs = {f"r{i}": p for i, p in enumerate(C.prompts(cfg["vocab"], LENGTHS[name], seed=21))}
        plain = C.plain_model(name)
        both = {k: plain.forward(v, return_margins=True) for k, v in reqs.items()}
        _oracle[name] = (reqs, {k: v[0] for k, v in both.items()})
        _margins[name] = {k: v[1] for k, v in both.items()}
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


def compare(rows, reqs, logits, dtype, what, case=None):
    """Every position within TOL.  In bfloat16 (``case`` names the model) a position whose routing is close to a
    tie somewhere in the model is only held to 0.7, and so are up to 2 % of the others (they attend to such
    positions)."""
    worst, over, held, total = 0.0, 0, 0, 0
    for name, toks in reqs.items():
        ref = logits[name]
        scale = np.abs(ref).max()
        for p in range(len(toks)):
            err = np.abs(rows[(name, p)] - ref[p]).max() / scale
            clear = not (dtype == "bfloat16" and case is not None and _margins[case][name][p] < CLEAR_MARGIN)
            total += 1
            held += clear
            if dtype == "bfloat16" and case is not None and clear and TOL[dtype] < err <= 0.7:
                over += 1
                continue
            assert err <= (TOL[dtype] if clear else 0.7), (
                f"{what}: request {name} (length {len(toks)}) first differs at position {p}: relative error {err:.3e}")
            worst = max(worst, err)
    assert held >= 0.1 * total, f"{what}: only {held} of {total} positions are held to the tight bound"
    assert over <= 1 + 0.02 * held, f"{what}: {over} of {held} positions with clear routing are over the bound"
    return worst


@pytest.mark.parametrize("mode", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "S", "N", "M", "A"])
def test_replay_matches_plain(name, dtype, mode, tmp_path):
    """Whole prompts; the last 32 tokens one by one; portions down to two tokens, cut inside pages; up to four
    live requests in a pool so small that pages and slots are used again."""
    reqs, logits = oracle(name)
    rows = replay(name, dtype, make_trace(mode, reqs, name), tmp_path)
    print(f"{name} {dtype} {mode}: worst relative error {compare(rows, reqs, logits, dtype, f'{name} {dtype} {mode}', name):.3e}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "N"])
def test_every_token_decoded_alone_matches_whole_prompts(name, dtype, tmp_path):
    """Token-by-token decoding from the first token on (up to 150 single steps through the decode graphs)
    against the plain logits of the whole prompt, and with graphs off."""
    reqs, logits = oracle(name)
    few = dict(list(reqs.items())[3:5])
    steps = make_trace("every_token", few, name)
    compare(replay(name, dtype, steps, tmp_path / "g"), few, logits, dtype, "decoded", name)
    compare(replay(name, dtype, steps, tmp_path / "e", use_graphs=False), few, logits, dtype, "decoded, no graphs", name)


@pytest.mark.parametrize("page", [2, 64])
def test_other_page_sizes(page, tmp_path):
    reqs, logits = oracle("P")
    for mode in ("portions", "mixed"):
        steps = make_trace(mode, reqs, "P")
        compare(replay("P", "float32", steps, tmp_path / mode, page=page), reqs, logits, "float32", f"page {page}")


def test_batch_of_unequal_requests_equals_each_alone(tmp_path):
    """One step with four prompts of unequal length beside one another, then single tokens of all four in one
    step: the rows equal those of each request run alone, bit for bit in 32-bit."""
    reqs, logits = oracle("P")
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
        a = replay("P", dtype, together, tmp_path / f"t{dtype}")
        b = replay("P", dtype, alone, tmp_path / f"a{dtype}")
        sub = {n: reqs[n] for n in names}
        compare(a, sub, logits, dtype, "together", "P")
        for key in a:
            assert np.abs(a[key] - b[key]).max() <= (2e-5 if dtype == "float32" else 0.25), key


# ---- generation through the engine and the command line -------------------------------------------------

def greedy_consistent(plain, prompt, out, tol):
    """How many generated tokens are the plain model's choice given the tokens before them (teacher-forced), up
    to ``tol`` of the largest absolute logit."""
    logits = plain.forward(list(prompt) + list(out))
    return sum(int(logits[len(prompt) - 1 + i][t] >= logits[len(prompt) - 1 + i].max() - tol * np.abs(logits).max())
               for i, t in enumerate(out))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q"])
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
    exact = good = 0
    for p, o in zip(prompts, outs):
        assert o.finish_reason == "max_tokens" and len(o.token_ids) == 10
        good += greedy_consistent(plain, p, o.token_ids, 1e-4 if dtype == "float32" else 6e-2)
        exact += int(o.token_ids == plain.greedy(p, 10))
    # in bfloat16 a router near a tie may choose another expert than the plain model: a few tokens may differ
    assert good >= (60 if dtype == "float32" else 51)
    assert exact >= (len(prompts) if dtype == "float32" else 1)
    assert eng.stats()["num_free_blocks"] == 1024 // page and not eng.has_unfinished()


def test_long_decoding_through_the_engine():
    from railgun_b200.engine.engine import Engine
    from railgun_b200.engine.request import SamplingParams
    cfg, _, page = C.CASES["S"]
    plain = C.plain_model("S")
    prompt = C.prompts(cfg["vocab"], [3], seed=8)[0]
    eng = Engine(C.model_dir("S"), dtype="float32", block_size=page, num_gpu_blocks=100, max_num_seqs=2,
                 max_model_len=400)
    out = eng.generate([prompt], SamplingParams(max_new_tokens=300))[0]
    assert len(out.token_ids) == 300
    assert greedy_consistent(plain, prompt, out.token_ids, 1e-4) == 300


def test_command_line_and_trace_runner(tmp_path):
    import json
    d = C.model_dir("P")
    plain = C.plain_model("P")
    prompt = [7, 200, 3, 99]
    res = subprocess.run([sys.executable, "-m", "railgun_b200", "generate", "-m", str(d), "--prompt-ids",
                          ",".join(map(str, prompt)), "--max-tokens", "6", "--dtype", "f32", "--block-size", "8"],
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    line = [l for l in res.stdout.splitlines() if l and l[0].isdigit()][0]
    assert [int(t) for t in line.split(",")] == plain.greedy(prompt, 6)
    toks = C.prompts(211, [30], seed=6)[0]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:19], "want": [0, 18]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[19:21], "want": []}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": toks[21:], "want": [8]}], "end": ["a"]}]
    res = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", str(d), "--dtype", "float32", "--out",
                          str(tmp_path), "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                         cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [l for l in res.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    ref = plain.forward(toks)
    got0 = np.fromfile(tmp_path / "0.f32", dtype="<f4").reshape(2, 211)
    got2 = np.fromfile(tmp_path / "2.f32", dtype="<f4").reshape(1, 211)
    assert not (tmp_path / "1.f32").exists()
    assert np.abs(got0 - ref[[0, 18]]).max() < 1e-4 and np.abs(got2[0] - ref[29]).max() < 1e-4


# ---- the attention kernels and the re-injection alone ---------------------------------------------------

def plain_latent_rows(qa, rows, pos, R, scale, window=0):
    """One token's heads over its request's cache rows [0, pos]: scores over the whole row, values its first R."""
    lo = max(0, pos - window + 1) if window else 0
    keys = rows[lo:pos + 1]
    p = torch.softmax((qa @ keys.T) * scale, dim=-1)
    return p @ keys[:, :R]


@pytest.mark.parametrize("H,R,dr,page,window", [(5, 16, 16, 4, 0), (16, 512, 64, 16, 0), (70, 48, 16, 8, 0),
                                                (40, 96, 32, 32, 0), (3, 32, 0, 1, 0), (8, 64, 16, 16, 37)])
def test_latent_attention_kernels_alone(H, R, dr, page, window):
    """Both attention kernels over hand-made cache rows behind a shuffled block table: a portion of a prompt (a
    tile of 64 positions and one of 6) beside a single token of another request, and single tokens alone with
    their contexts cut into one, three and seven shares; more heads than a block takes, one head chunk, a latent
    of 512, a window."""
    from railgun_b200 import ops
    g = torch.Generator().manual_seed(H * 1000 + R)
    D, ctx = R + dr, (200, 77)
    n_pages = [-(-c // page) for c in ctx]
    perm = torch.randperm(sum(n_pages) + 3, generator=g)
    table = torch.zeros((2, max(n_pages)), dtype=torch.int32)
    table[0, :n_pages[0]] = perm[:n_pages[0]]
    table[1, :n_pages[1]] = perm[n_pages[0]:n_pages[0] + n_pages[1]]
    rows = [torch.randn(c, D, generator=g).to(torch.bfloat16) for c in ctx]
    cache = torch.zeros((sum(n_pages) + 3, page, D), dtype=torch.bfloat16)
    for r in range(2):
        for j in range(ctx[r]):
            cache[table[r, j // page], j % page] = rows[r][j]
    scale = 1.7 / D ** 0.5
    # rows 0..69: request 0 at positions 130..199; row 70: request 1 at position 76
    positions = torch.tensor(list(range(130, 200)) + [76], dtype=torch.int32)
    req = torch.tensor([0] * 70 + [1], dtype=torch.int32)
    qa = torch.randn(71, H, D, generator=g).to(torch.bfloat16)
    ref = torch.stack([plain_latent_rows(qa[t].double(), rows[int(req[t])].double(), int(positions[t]), R, scale, window)
                       for t in range(71)])
    dev = lambda t: t.to(DEV)
    got = ops.latent_attention_general(dev(qa), dev(cache), dev(table), dev(req), dev(positions), R, window, scale)
    assert rel(got, ref) < 8e-3
    assert ops.latent_attention_mma_ok(torch.bfloat16, H, R, D)
    out = torch.zeros((71, H, R), dtype=torch.bfloat16, device=DEV)
    tiles = torch.tensor([[0, 64, 0], [64, 6, 0]], dtype=torch.int32)
    ops.latent_attention_mma(dev(qa), out, dev(cache), dev(table), dev(tiles), None, 2, dev(req), dev(positions), R,
                             window, scale)
    ops.latent_attention_mma(dev(qa), out, dev(cache), dev(table), None, dev(torch.tensor([70], dtype=torch.int32)), 1,
                             dev(req), dev(positions), R, window, scale, 2)
    assert rel(out, ref) < 8e-3
    # single tokens only: three requests' last positions, rows 0..2
    pos1 = torch.tensor([199, 76, 150], dtype=torch.int32)
    req1 = torch.tensor([0, 1, 0], dtype=torch.int32)
    ref1 = torch.stack([plain_latent_rows(qa[t].double(), rows[int(req1[t])].double(), int(pos1[t]), R, scale, window)
                        for t in range(3)])
    for splits in (1, 3, 7):
        out1 = torch.zeros((3, H, R), dtype=torch.bfloat16, device=DEV)
        ops.latent_attention_mma(dev(qa[:3].contiguous()), out1, dev(cache), dev(table), None, None, 3, dev(req1),
                                 dev(pos1), R, window, scale, splits)
        assert rel(out1, ref1) < 8e-3, f"{splits} shares"
    assert not ops.latent_attention_mma_ok(torch.bfloat16, H, 40, 48) and not ops.latent_attention_mma_ok(torch.float32, H, R, D)


@pytest.mark.parametrize("dtype", DTYPES)
def test_reinjection_alone(dtype):
    """x <- W [x + pending; x0] with x0 the stream at the start of the step."""
    from railgun_b200 import ops
    from railgun_b200.parts.base import Stream
    from railgun_b200.parts.registry import STREAM_OPS
    rng = np.random.default_rng(5)
    Hd, T, dt = 40, 9, TORCH[dtype]
    t = {"loop.in": torch.tensor(rng.normal(size=(Hd, 2 * Hd)) * 0.2)}
    part = STREAM_OPS.get("reinject")(dict(hidden_size=Hd, name="loop.in"), "", env_of(dt, Hd), bank_of(t, dt))
    x0 = torch.tensor(rng.normal(size=(T, Hd)), dtype=torch.float32)
    moved = torch.tensor(rng.normal(size=(T, Hd)), dtype=torch.float32)
    y = torch.tensor(rng.normal(size=(T, Hd)), dtype=torch.float32).to(dt)
    wb = torch.tensor(1 + 0.2 * rng.normal(size=Hd), dtype=torch.float32)
    stream = Stream(x0.clone().to(DEV))
    part.begin(stream, None)
    stream.resid = moved.clone().to(DEV)                       # layers ran in between
    stream.pending = ops.PendingNormed(y.to(DEV), wb.to(DEV), 1e-5)
    part.apply(stream, None)
    w = rounded(t, dt)["loop.in"]
    x = moved.double() + P.rms_norm(y.double(), wb.double(), 1e-5)
    both = torch.cat([x, x0.double()], dim=-1)
    if dt == torch.bfloat16:
        both = both.to(torch.bfloat16).double()
    assert stream.pending is None and stream.resid.dtype == torch.float32
    assert rel(stream.resid, both @ w.T) < (1e-5 if dtype == "float32" else 2e-2)
