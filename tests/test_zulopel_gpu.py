"""Zulopel on the GPU against the plain implementation (tests/plain_zulopel.py): each mechanism alone, then whole
models through the engine's step function in true 32-bit and in bfloat16: whole prompts, prompts followed by
token-by-token decoding, portions down to two tokens, batches of unequal requests, pages and state slots that are given
back and used again, attention made sharp so that a key that is lost or let through a chunk's edge shows, decays so slow
that a lost state shows hundreds of tokens later, long decoding, greedy generation through the scheduler, and replay
through bin/trace_run."""
import json
import os

import numpy as np
import pytest
import torch

import llmengine
import plain_zulopel as P
from gpu_helpers import DEV, Harness
from llmengine.config.zulopel import ZulopelConfig
from llmengine.models.zulopel import describe_zulopel
from llmengine.ops import get_ops
from llmengine.parts import LayerCache, build_part
from tiny import MIXED_SIZES_LONG, Trace, random_ids, round64, run_trace, trace_mixed, trace_portions, trace_tail, trace_whole
from tiny_zulopel import ZULOPEL, ZULOPEL_A, ZULOPEL_B, ZULOPEL_C, make_tensors, write_model

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
NAMES = {torch.float32: "fp32", torch.bfloat16: "bf16"}


def close(got, want, dt, what=""):
    """float32: element by element; bfloat16: the root mean square of the difference against that of the values."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    if dt == torch.float32:
        err = np.abs(got - want).max() / max(1.0, np.abs(want).max())
        assert err < 1e-4, f"{what}: float32 differs by {err:.3e}"
    else:
        err = np.sqrt(((got - want) ** 2).mean()) / max(np.sqrt((want ** 2).mean()), 1e-6)
        assert err < 4e-2, f"{what}: bfloat16 differs by {err:.3e} of the values' size"


def rows_close(got, want, dt, what=""):
    """Logits of a request, a row a position. float32: as close(). bfloat16: a row's error is the root mean square of its
    difference against that of all values; rounding leaves most rows near one percent, except where it flips a router's
    choice between two experts that nearly tie, which changes that row and, through the recurrent state, may colour the
    rows after it. So: the median row within 3 percent, and at most one row in ten beyond 15 percent."""
    if dt == torch.float32:
        return close(got, want, dt, what)
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    e = np.sqrt(((got - want) ** 2).mean(1)) / max(np.sqrt((want ** 2).mean()), 1e-6)
    assert np.median(e) < 3e-2, f"{what}: bfloat16 rows differ by {np.median(e):.3e} of the values' size (median)"
    far = np.nonzero(e > 15e-2)[0]
    assert far.size <= max(1, len(e) // 10), f"{what}: {far.size} of {len(e)} bfloat16 rows differ by more than 15 percent, first {far[0]}"


def whole(delta):
    return delta if delta.dim() == 2 else delta.sum(0)


def layer_tensors(cfg, i, dt, sharp=False):
    """The tensors of layer i as the file would hold them -> (float64 for the plain side, on the device as the loader hands
    them over: matrices in the engine's precision, everything else float32)."""
    t = {k: v for k, v in make_tensors(cfg, 5, dt, sharp).items() if k.startswith(f"l{i}.")}
    spec = describe_zulopel(ZulopelConfig.from_dict(cfg)).layers[i]
    from llmengine.parts.registry import part_class
    needs = {n.name: n for n in part_class("block", spec.kind).tensor_needs(spec)}
    dev = {k: v.to(DEV, dt if needs[k].precision == "compute" else torch.float32) for k, v in t.items() if k in needs}
    return {k: v.double() for k, v in t.items()}, dev, spec


# ---------------------------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("E,top,groups,keep,n", [(6, 2, 3, 2, 40), (16, 4, 4, 3, 33), (4, 4, 2, 2, 5), (9, 3, 3, 1, 17), (5, 1, 1, 1, 9),
                                                 (64, 8, 8, 4, 12)])
def test_group_limited_router_alone(E, top, groups, keep, n):
    """Choice scores that the correction makes negative, groups that are dropped although they hold the largest score of all
    but one, weights from the scores without the correction."""
    g = torch.Generator().manual_seed(E * 7 + top)
    x, wr = torch.randn(n, 24, generator=g), torch.randn(E, 24, generator=g) * 0.6
    corr = torch.randn(E, generator=g) * 0.3 - 0.2
    idx = torch.empty(n, top, dtype=torch.int32, device=DEV)
    share = torch.empty(n, top, dtype=torch.float32, device=DEV)
    get_ops().route_grouped(x.to(DEV), wr.to(DEV), corr.to(DEV), top, groups, keep, 1e-20, idx, share)
    z = x.double() @ wr.double().T
    for t in range(n):
        chosen, wts = P.route(z[t], corr.double(), top, groups, keep)
        assert idx[t].tolist() == chosen, f"token {t}"
        np.testing.assert_allclose(share[t].cpu().numpy(), wts.numpy(), rtol=2e-5)


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg,i,n", [(ZULOPEL_A, 0, 19), (ZULOPEL_A, 1, 4), (ZULOPEL_A, 2, 70), (ZULOPEL_A, 4, 1), (ZULOPEL_B, 0, 150),
                                     (ZULOPEL_B, 2, 9), (ZULOPEL_C, 0, 33)], ids=["a0", "a1", "a2", "a4", "b0", "b2", "c0"])
def test_feed_forward_alone(dt, cfg, i, n):
    cpu, dev, spec = layer_tensors(cfg, i, dt)
    h = Harness(dt)
    part = build_part("feed_forward", spec.feed_forward, h.env)
    part.load(dev)
    x = torch.randn(n, cfg["width"], generator=torch.Generator().manual_seed(8)).to(dt)
    got = whole(part.forward(x.to(DEV), h.ctx([(1, n, [])]))).cpu()
    close(got, P.moe(x.double(), cpu, f"l{i}.mlp.", cfg["layers"][i]["mlp"]), dt)


def mixer_harness(dt, spec, page, part):
    h = Harness(dt, page=page, pages=120)
    c = LayerCache(group=0)
    for need in part.cache_needs():
        if hasattr(need, "head_dim"):
            c.k = torch.zeros(121, need.num_kv_heads, page, need.head_dim, dtype=dt, device=DEV)
            c.v = torch.zeros(121, need.num_kv_heads, page, need.value_dim, dtype=dt, device=DEV)
        else:
            c.states[need.name] = torch.zeros((5,) + tuple(need.shape), dtype=need.dtype, device=DEV)
    return h, c


def _one_attention_layer(heads, kv_heads, dim, vdim, chunk, dims):
    """A configuration of one attention layer, for the head sizes that the tensor-core kernel takes."""
    from tiny_zulopel import _att
    return {"architecture": "Zulopel", "vocab": 64, "width": 80, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "max_positions": 2048,
            "layers": [{"type": "attention", "mixer": _att(heads, kv_heads, dim, vdim, dim ** -0.5, dims, 1000.0, chunk), "mlp": None}]}


ATTENTION_CASES = [(ZULOPEL_A, 4), (ZULOPEL_B, 0), (ZULOPEL_C, 1), (_one_attention_layer(6, 2, 64, 32, 16, 24), 0),
                   (_one_attention_layer(8, 1, 128, 128, 0, 128), 0), (_one_attention_layer(2, 2, 32, 128, 7, 0), 0),
                   (_one_attention_layer(12, 3, 128, 64, 21, 64), 0)]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg,i", ATTENTION_CASES, ids=["a4", "b0", "c1", "64x32", "128x128", "32x128", "128x64"])
@pytest.mark.parametrize("sharp", [False, True])
def test_gated_attention_alone(dt, cfg, i, sharp):
    """The mixer over a prompt portion, then over single tokens and a second portion that read the first one's cache rows;
    no value mixing (a4, c1) or the role of the first mixer (b0), which only leaves its values."""
    cpu, dev, spec = layer_tensors(cfg, i, dt, sharp)
    h, cache = mixer_harness(dt, spec, 4, build_part("mixer", spec.mixer, Harness(dt).env))
    part = build_part("mixer", spec.mixer, h.env)
    part.load(dev)
    x = (2 * torch.randn(61, cfg["width"], generator=torch.Generator().manual_seed(6))).to(dt)
    state = {}
    for lo, hi in ((0, 17), (17, 18), (18, 19), (19, 50), (50, 51), (51, 61)):
        ctx = h.ctx([(1, hi - lo, [])])
        got = whole(part.forward(x[lo:hi].to(DEV), ctx, cache)).cpu()
        ref = P.attention_mixer(x[lo:hi].double(), cpu, f"l{i}.mix.", cfg["layers"][i]["mixer"], cfg["norm"]["eps"], lo, state, {})
        close(got, ref, dt, f"positions {lo}..{hi}")


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("chunk", [0, 700])
def test_gated_attention_single_tokens_after_a_long_context(dt, chunk):
    """1,500 tokens as one portion, then single tokens: in bfloat16 their key range runs in pieces side by side (counted from
    the chunk's start) and the sink and the gate are applied where the pieces are merged. The oracle forms every key and value
    at once and the last tokens' scores by one product each."""
    cfg = _one_attention_layer(8, 2, 64, 64, chunk, 32)
    m, eps = cfg["layers"][0]["mixer"], cfg["norm"]["eps"]
    cpu, dev, spec = layer_tensors(cfg, 0, dt, sharp=True)
    h, cache = mixer_harness(dt, spec, 16, build_part("mixer", spec.mixer, Harness(dt).env))
    part = build_part("mixer", spec.mixer, h.env)
    part.load(dev)
    if dt == torch.bfloat16:
        assert get_ops()._split_policy(2, min(1503, chunk) if chunk else 1503, 64)[0] > 1, "the case is meant to run in pieces"
    T = 1503
    x = (2 * torch.randn(T, cfg["width"], generator=torch.Generator().manual_seed(26))).to(dt)
    w = {k[len("l0.mix."):]: v for k, v in cpu.items() if k.startswith("l0.mix.")}
    xd = x.double()
    q = P.rms_norm((xd @ w["q"].T).view(T, 8, 64), w["q.norm"], eps)
    k = P.rms_norm((xd @ w["k"].T).view(T, 2, 64), w["k.norm"], eps)
    v = (xd @ w["v"].T).view(T, 2, 64)
    for t in range(T):
        q[t], k[t] = P.rotate(q[t], t, m["rot"]), P.rotate(k[t], t, m["rot"])
    gate = torch.sigmoid(xd @ w["g"].T)

    def oracle(t):
        lo = (t // chunk) * chunk if chunk else 0
        heads = []
        for a in range(8):
            s = (k[lo:t + 1, a // 4] @ q[t, a]) * m["scale"]
            p = torch.softmax(torch.cat([s, w["sink"][a:a + 1]]), dim=0)[:-1]
            heads.append(p @ v[lo:t + 1, a // 4])
        return (torch.cat(heads) * gate[t]) @ w["o"].T

    got = whole(part.forward(x[:1500].to(DEV), h.ctx([(1, 1500, [])]), cache)).cpu()
    for t in (0, 63, 699, 700, 1399, 1400, 1499):
        close(got[t], oracle(t), dt, f"position {t} of the portion")
    for t in (1500, 1501, 1502):
        got = whole(part.forward(x[t:t + 1].to(DEV), h.ctx([(1, 1, [])]), cache)).cpu()
        close(got[0], oracle(t), dt, f"single token at {t}")


def _one_scan_layer(inner, state, conv, dt_rank):
    from tiny_zulopel import _scan
    return {"architecture": "Zulopel", "vocab": 64, "width": 80, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "max_positions": 512,
            "layers": [{"type": "mamba1", "mixer": _scan(inner, state, conv, dt_rank), "mlp": None}]}


# (the last two: a rank and a channel count that the tensor-core step-size product takes, with states of 5 and 24 numbers, whose
# rows of B and C are not 16-byte aligned in the first)
SCAN_CASES = [(ZULOPEL_A, 0), (ZULOPEL_A, 3), (ZULOPEL_B, 1), (ZULOPEL_B, 2), (ZULOPEL_C, 0), (_one_scan_layer(64, 5, 3, 8), 0),
              (_one_scan_layer(48, 24, 4, 16), 0)]


@pytest.mark.parametrize("dt", DTYPES)
@pytest.mark.parametrize("cfg,i", SCAN_CASES, ids=["a0", "a3", "b1", "b2", "c0", "n5", "n24"])
def test_selective_scan_alone(dt, cfg, i):
    """Portions of 1, 2 and many tokens that hand the convolution's inputs and the state on through the slot."""
    cpu, dev, spec = layer_tensors(cfg, i, dt)
    h, cache = mixer_harness(dt, spec, 4, build_part("mixer", spec.mixer, Harness(dt).env))
    part = build_part("mixer", spec.mixer, h.env)
    part.load(dev)
    x = (2 * torch.randn(420, cfg["width"], generator=torch.Generator().manual_seed(16))).to(dt)
    state = {}
    # (the portion of 310 tokens runs in pieces side by side, with a carry between two passes)
    for lo, hi in ((0, 1), (1, 3), (3, 4), (4, 70), (70, 71), (71, 73), (73, 90), (90, 400), (400, 401), (401, 420)):
        ctx = h.ctx([(1, hi - lo, [])])
        got = whole(part.forward(x[lo:hi].to(DEV), ctx, cache)).cpu()
        ref = P.mamba_mixer(x[lo:hi].double(), cpu, f"l{i}.mix.", cfg["layers"][i]["mixer"], state)
        close(got, ref, dt, f"positions {lo}..{hi}")


@pytest.mark.parametrize("dim,rows", [(50, 7), (72, 5), (2048, 3), (4100, 2), (9000, 2)])
def test_norm_on_the_output_with_layer_scale_alone(dim, rows):
    """Rows of any length (the kernel has a form with 16-byte moves, one that keeps a row in registers and one that reads it twice)."""
    g = torch.Generator().manual_seed(3)
    hstream, a, b = torch.randn(rows, dim, generator=g), torch.randn(3, rows, dim, generator=g), torch.randn(rows, dim, generator=g)
    w, ls = 1 + 0.3 * torch.randn(dim, generator=g), 1 + 0.3 * torch.randn(dim, generator=g)
    want = hstream.double() + P.rms_norm(a.double().sum(0) + b.double(), w.double(), 1e-3) * ls.double()
    hd, copy = hstream.to(DEV), torch.empty(rows, dim, dtype=torch.bfloat16, device=DEV)
    get_ops().norm_add(hd, a.to(DEV), b.to(DEV), w.to(DEV), ls.to(DEV), 1e-3, copy=copy)
    np.testing.assert_allclose(hd.cpu().numpy(), want.numpy(), rtol=0, atol=2e-5)
    assert torch.equal(copy.cpu(), hd.cpu().to(torch.bfloat16))
    h2 = hstream.to(DEV)  # one set of sums, no layer scale, no copy
    get_ops().norm_add(h2, b.to(DEV), None, w.to(DEV), None, 1e-3)
    np.testing.assert_allclose(h2.cpu().numpy(), (hstream.double() + P.rms_norm(b.double(), w.double(), 1e-3)).numpy(), rtol=0, atol=2e-5)


# ---------------------------------------------------------------------------------------------- whole models
def replay(eng, trace):
    """The trace's steps through Engine.run_step, in this process -> {(request, position): logits row}."""
    ids, nxt, out = {}, 1, {}
    for k, s in enumerate(trace.steps):
        batch = []
        for e in s["entries"]:
            if e["id"] not in ids:
                ids[e["id"]], nxt = nxt, nxt + 1
            batch.append((ids[e["id"]], e["tokens"], e["want"]))
        lg = eng.run_step(batch, end=[ids[n] for n in s["end"]]).float().cpu().numpy()
        for n in s["end"]:
            ids.pop(n)
        for i, key in enumerate(trace.rows.get(k, [])):
            out[key] = lg[i].copy()
    return out


@pytest.fixture(scope="module", params=[(n, dt, sharp) for n in ("za", "zb", "zc") for dt in DTYPES for sharp in (False, True)
                                        if not (sharp and n == "zc")],
                ids=lambda p: f"{p[0]}-{NAMES[p[1]]}{'-sharp' if p[2] else ''}")
def model(request, tmp_path_factory):
    name, dt, sharp = request.param
    cfg, page = ZULOPEL[name]
    d = write_model(str(tmp_path_factory.mktemp("zulopel")), cfg, dt, sharp=sharp)
    pc, pw = P.read_model(d)
    lens = [5, 64, 33, 130, 97] if name != "zb" else [3, 47, 64, 200, 129]
    reqs = {f"r{i}": random_ids(n, cfg["vocab"], 50 + i) for i, n in enumerate(lens)}
    plain = {k: P.forward(pc, pw, v).numpy() for k, v in reqs.items()}
    eng = llmengine.Engine(d, NAMES[dt], block_size=page)
    longest = max(round64(len(v)) for v in reqs.values())
    tokens = longest + 3 * 64  # room for the longest request and three short ones: pages are used again
    eng.configure_cache(num_blocks=tokens // page, block_size=page, num_slots=4)
    return dt, eng, reqs, plain, tokens, (pc, pw), cfg


@pytest.mark.parametrize("cut", ["whole", "tail", "portions", "mixed"])
def test_cuts_match_plain_and_one_another(model, cut):
    """whole: each prompt in one step; tail: its last 32 tokens one by one (prefill against decoding through the cache and
    the state); portions: sizes 7, 2, 13, 2, 5, 3, ... ; mixed: up to four live requests, portions beside single tokens,
    with so few pages and slots that both are used again."""
    dt, eng, reqs, plain, tokens, _, _ = model
    named = {f"{cut}.{k}": v for k, v in reqs.items()}
    trace = {"whole": trace_whole, "tail": trace_tail, "portions": trace_portions}[cut](named) if cut != "mixed" else \
        trace_mixed(named, tokens, seed=5, sizes=MIXED_SIZES_LONG)
    rows = replay(eng, trace)
    assert eng.cm.num_requests == 0
    for k, ids in reqs.items():
        got = np.stack([rows[(f"{cut}.{k}", p)] for p in range(len(ids))])
        rows_close(got, plain[k], dt, f"{cut}, request {k}")
        if dt == torch.float32:  # where the first wrong position is, if any
            bad = np.nonzero(np.abs(got - plain[k]).max(1) > 1e-3 * max(1.0, np.abs(plain[k]).max()))[0]
            assert bad.size == 0, f"{cut}, request {k}: first wrong position {bad[0]} of {len(ids)}"


def test_scan_in_pieces_beside_single_tokens(model):
    """The mixed batches once more with the recurrent layers' scan cut into pieces already for portions of 65 tokens: pieces
    of unequal requests side by side, single tokens of other requests among them."""
    dt, eng, reqs, plain, tokens, _, cfg = model
    if dt == torch.bfloat16 and cfg is ZULOPEL_A:
        # one expert of five: where rounding flips that choice early in a request, the slow decays of these weights carry the
        # difference through the rest of it; this configuration's pieces are compared in float32
        pytest.skip("bfloat16 with a single chosen expert: compared in float32")
    ops = get_ops()
    ops.SCAN_PIECES_FROM = 65
    try:
        named = {f"pieces.{k}": v for k, v in reqs.items()}
        rows = replay(eng, trace_mixed(named, tokens, seed=9, sizes=(1, 2, 70, 130, 66)))
    finally:
        del ops.SCAN_PIECES_FROM
    for k, ids in reqs.items():
        rows_close(np.stack([rows[(f"pieces.{k}", p)] for p in range(len(ids))]), plain[k], dt, f"request {k}")


def test_keys_at_page_borders_chunk_edges_and_first_tokens(model):
    """A request that grows one token a step from its first token across page borders and chunk edges, beside a second one that
    starts later (so that its pages lie between the first one's, and its state in another slot)."""
    dt, eng, reqs, plain, _, _, _ = model
    a, b = reqs["r2"], reqs["r1"][:20]
    t = Trace()
    for p in range(len(a)):
        entries = [("a", a[p:p + 1], [0], p)]
        if 5 <= p < 5 + len(b):
            entries.append(("b", b[p - 5:p - 4], [0], p - 5))
        t.add(entries, end=[n for n, cond in (("a", p == len(a) - 1), ("b", p == 4 + len(b))) if cond])
    rows = replay(eng, t)
    rows_close(np.stack([rows[("a", p)] for p in range(len(a))]), plain["r2"], dt, "token by token")
    rows_close(np.stack([rows[("b", p)] for p in range(len(b))]), plain["r1"][:20], dt, "the request beside it")


def test_a_slot_that_is_used_again_starts_at_zero(model):
    """Two requests one after the other in an engine with a single live request at a time: the second gets the first one's
    slot and pages, and must not see its state."""
    dt, eng, reqs, plain, _, _, _ = model
    for k in ("r3", "r1", "r3"):
        n = len(reqs[k])
        got = eng.run_step([(77, reqs[k], list(range(n)))], end=[77]).float().cpu().numpy()
        rows_close(got, plain[k], dt, k)


def test_long_decoding_and_generation(model):
    """Greedy generation through the engine's entry point and scheduler (decode steps replay CUDA graphs in bfloat16); in
    float32 the tokens are the plain implementation's."""
    dt, eng, reqs, plain, _, (pc, pw), cfg = model
    prompt = reqs["r2"][:11]
    out, reason = eng.generate(prompt, 70)
    assert reason == "length" and len(out) == 81 and out[:11] == prompt
    logits = P.forward(pc, pw, out).numpy()
    if dt == torch.float32:
        for p in range(10, 80):  # the chosen token is the plain logits' best, or ties with it within rounding
            assert logits[p, out[p + 1]] >= logits[p].max() - 1e-4 * max(1.0, np.abs(logits[p]).max()), p
    else:  # bfloat16: close to the plain logits' best; a router's choice that rounding flips may move single positions further
        off = [p for p in range(10, 80) if logits[p, out[p + 1]] < logits[p].max() - 0.1 * max(1.0, np.abs(logits[p]).max())]
        assert len(off) <= 7, f"{len(off)} of 70 generated tokens are far from the plain logits' best, first at {off[0]}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_through_the_command(dtype, tmp_path):
    """bin/trace_run as a user runs it."""
    cfg, page = ZULOPEL["zb"]
    dt = torch.float32 if dtype == "float32" else torch.bfloat16
    d = write_model(str(tmp_path / "m"), cfg, dt)
    pc, pw = P.read_model(d)
    reqs = {f"q{i}": random_ids(n, cfg["vocab"], 80 + i) for i, n in enumerate([2, 70, 35, 150])}
    t = trace_mixed(reqs, 256 + 64, seed=3, sizes=MIXED_SIZES_LONG)
    rows = run_trace(d, dtype, t, str(tmp_path / "out"), 256 + 64, page, cfg["vocab"])
    for k, ids in reqs.items():
        rows_close(np.stack([rows[(k, p)] for p in range(len(ids))]), P.forward(pc, pw, ids).numpy(), dt, k)


def test_generation_from_the_command_line(tmp_path):
    from test_cli import run_cli
    d = write_model(str(tmp_path / "model"), ZULOPEL_C, torch.float32)
    r = run_cli("--model", d, "--prompt-ids", "5,17,3,90", "--max-new", "6", "--block-size", "8", "--num-blocks", "32")
    assert r.returncode == 0, r.stderr
    line = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")][0]
    pc, pw = P.read_model(d)
    assert line["token_ids"] == P.generate(pc, pw, [5, 17, 3, 90], 6) and line["finish_reason"] == "length"
