"""Zulopel without a GPU: configuration and its errors, the description in parts (tensor names, value-mixing roles, what a
file may carry unread), the rotation frequencies against the plain implementation's, the random-weights mode, and the plain
implementation against itself (whole prompts against portions and single tokens; the router's rules on cases made by hand)."""
import copy
import json

import numpy as np
import pytest
import torch

import llmengine
import plain_zulopel as P
from llmengine.config import ConfigError
from llmengine.config.registry import config_from_dir, get_architecture
from llmengine.config.zulopel import ZulopelConfig
from llmengine.models.zulopel import describe_zulopel
from llmengine.parts.position import ramp_frequencies
from llmengine.weights.random_init import model_tensor_needs
from cpu_ops import CpuOps
from tiny import random_ids
from tiny_zulopel import ZULOPEL, ZULOPEL_A, ZULOPEL_B, ZULOPEL_C, make_tensors, write_model


@pytest.mark.parametrize("name", sorted(ZULOPEL))
def test_configuration_round_trip_and_tensor_names(name):
    cfg = ZULOPEL[name][0]
    c = ZulopelConfig.from_dict(cfg)
    assert ZulopelConfig.from_dict(c.to_dict()) == c
    assert get_architecture("Zulopel").parse_config(cfg, None) == c
    spec = describe_zulopel(c)
    needs = model_tensor_needs(spec)
    made = make_tensors(cfg, 1, torch.float32)
    assert set(needs) <= set(made)
    for k in set(made) - set(needs):  # what the file carries and nobody reads is named in the description
        assert k in spec.ignore, k
    for k, n in needs.items():
        assert tuple(made[k].shape) == tuple(n.shape), k
    assert [b.kind for b in spec.layers] == ["post_norm"] * len(cfg["layers"])
    assert [r.layer for r in spec.order] == list(range(len(cfg["layers"])))


def test_description_reads_every_option():
    spec = describe_zulopel(ZulopelConfig.from_dict(ZULOPEL_A))
    kinds = [b.mixer.kind for b in spec.layers]
    assert kinds == ["selective_scan", "gated_attention", "gated_attention", "selective_scan", "gated_attention"]
    a1, a2, a4 = spec.layers[1].mixer, spec.layers[2].mixer, spec.layers[4].mixer
    assert (a1.value_mix, a2.value_mix, a4.value_mix) == ("first", "mix", None)
    assert a1.value_mix_weight is None and a2.value_mix_weight == "l2.mix.vmix"
    assert (a1.chunk, a2.chunk, a4.chunk) == (20, 12, 0)
    assert (a1.num_heads, a1.num_kv_heads, a1.head_dim, a1.value_dim) == (6, 2, 24, 10)
    assert a1.position.dims == 10 and a1.position.factor == 8.0 and a4.position.factor == 0.0
    s0 = spec.layers[0].mixer
    assert (s0.inner, s0.state, s0.taps, s0.dt_rank) == (40, 5, 3, 7)
    f0, f1, f4 = spec.layers[0].feed_forward, spec.layers[1].feed_forward, spec.layers[4].feed_forward
    assert (f0.experts, f0.top, f0.groups, f0.keep_groups, f0.shared.intermediate) == (6, 2, 3, 2, 20)
    assert (f1.groups, f1.keep_groups, f1.shared) == (1, 1, None)
    assert (f4.groups, f4.keep_groups) == (3, 1)
    assert spec.layers[3].feed_forward is None and spec.layers[3].norm2 is None
    assert spec.embedding.scale == 3.5 and spec.head.weight == "head" and spec.embedding.weight == "embed"


@pytest.mark.parametrize("change,word", [
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=4), "kv_heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=26), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][2]["mixer"].update(vdim=12), "mix values"),
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"].pop("state"), "state"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_configuration_errors(change, word):
    cfg = copy.deepcopy(ZULOPEL_A)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        ZulopelConfig.from_dict(cfg)
    assert word in str(e.value)


def test_rotation_frequencies_match_the_plain_ones():
    for cfg in (ZULOPEL_A, ZULOPEL_B, ZULOPEL_C):
        spec = describe_zulopel(ZulopelConfig.from_dict(cfg))
        for layer, block in zip(cfg["layers"], spec.layers):
            if layer["type"] != "attention":
                continue
            f, m = ramp_frequencies(block.mixer.position)
            pf, pm = P.rotary_frequencies(layer["mixer"]["rot"])
            np.testing.assert_allclose(f, pf, rtol=1e-14)
            assert abs(m - pm) < 1e-15


def test_random_weights_mode_writes_the_design(tmp_path):
    d = llmengine.write_random_model(str(tmp_path / "m"), ZULOPEL_C, seed=3, dtype=torch.bfloat16)
    arch, cfg = config_from_dir(d)
    assert arch.name == "Zulopel" and cfg == ZulopelConfig.from_dict(ZULOPEL_C)
    pc, pw = P.read_model(d)
    assert set(pw) == set(model_tensor_needs(describe_zulopel(cfg)))
    assert pw["l1.mix.sink"].shape == (5,) and pw["l0.mix.A_log"].shape == (24, 3)
    assert torch.isfinite(P.forward(pc, pw, [1, 2, 3, 4])).all()


@pytest.mark.parametrize("name", sorted(ZULOPEL))
def test_plain_portions_and_single_tokens_match_the_whole_prompt(name, tmp_path):
    cfg = ZULOPEL[name][0]
    d = write_model(str(tmp_path / "m"), cfg, torch.float32, sharp=True)
    pc, pw = P.read_model(d)
    ids = [(7 * i * i + 3 * i + 1) % cfg["vocab"] for i in range(75)]
    want = P.forward(pc, pw, ids)
    for cuts in ([1, 2, 30, 31, 33, 60, 75], list(range(1, 76))):
        m, state, got, lo = P.PlainZulopel(pc, pw), {}, [], 0
        for hi in cuts:
            got.append(m.forward(ids[lo:hi], state))
            lo = hi
        assert float((torch.cat(got) - want).abs().max()) < 1e-9


def test_plain_router_rules():
    z = torch.log(torch.tensor([0.05, 0.30, 0.10, 0.05, 0.28, 0.02, 0.12, 0.08], dtype=torch.float64))  # softmax(z) = these scores
    zero = torch.zeros(8, dtype=torch.float64)
    # no groups: the two largest scores, weights = their scores over their sum
    chosen, w = P.route(z, zero, 2, 1, 1)
    assert chosen == [1, 4] and np.allclose(w.numpy(), [0.30 / 0.58, 0.28 / 0.58])
    # four groups of two, two stay: groups 0 (0.30) and 2 (0.28); expert 6 (0.12, group 3) is out although it beats expert 0
    chosen, w = P.route(z, zero, 3, 4, 2)
    assert chosen == [1, 4, 0] and np.allclose(w.numpy(), np.array([0.30, 0.28, 0.05]) / 0.63)
    # a correction changes the choice, not the weights; choice scores may be negative and still win inside a kept group
    corr = torch.tensor([0.0, -0.5, 0.0, 0.0, -0.5, 0.0, 0.3, 0.0], dtype=torch.float64)
    chosen, w = P.route(z, corr, 2, 4, 1)
    assert chosen == [6, 7] and np.allclose(w.numpy(), np.array([0.12, 0.08]) / 0.20)
    chosen, w = P.route(z, corr - 1.0, 2, 4, 1)  # every choice score below zero
    assert chosen == [6, 7]


# ---------------------------------------------------------------------------------------------- the engine's host side
@pytest.fixture(scope="module", params=["za", "zc"])
def cpu_engine(request, tmp_path_factory):
    """The engine on the test double of the kernels: batch building, block tables, state slots, the wiring of the parts."""
    cfg, page = ZULOPEL[request.param]
    d = write_model(str(tmp_path_factory.mktemp("zulopel_" + request.param)), cfg, torch.float32, sharp=True)
    eng = llmengine.Engine(d, "fp32", device="cpu", ops=CpuOps(), block_size=page, num_blocks=40)
    eng.configure_cache(num_blocks=40, block_size=page, num_slots=3)
    return eng, P.read_model(d), cfg


def test_engine_on_the_test_double_matches_plain(cpu_engine):
    eng, (pc, pw), cfg = cpu_engine
    a, b = random_ids(37, cfg["vocab"], 1), random_ids(11, cfg["vocab"], 2)
    want = {k: P.forward(pc, pw, ids).numpy() for k, ids in (("a", a), ("b", b))}
    got = eng.run_step([(1, a, list(range(len(a))))], end=[1]).numpy()
    assert np.abs(got - want["a"]).max() < 2e-4
    # portions beside single tokens of another request; pages and state slots are given back and used again
    rows = {}
    steps = [([(2, a[:9], [8]), (3, b[:10], [9])], []), ([(2, a[9:11], [0, 1]), (3, b[10:], [0])], [3]),
             ([(2, a[11:36], [24]), (4, b[:3], [2])], []), ([(2, a[36:], [0]), (4, b[3:], [7])], [2, 4])]
    at = {2: 0, 3: 0, 4: 0}
    for batch, end in steps:
        lg = eng.run_step(batch, end=end).numpy().copy()  # the logits tensor is scratch of the engine
        i = 0
        for rid, toks, w in batch:
            for k in w:
                rows[(rid, at[rid] + k)] = lg[i]
                i += 1
            at[rid] += len(toks)
    for (rid, pos), row in rows.items():
        ref = want["a"] if rid == 2 else want["b"]
        assert np.abs(row - ref[pos]).max() < 2e-4, (rid, pos)
    assert eng.cm.num_requests == 0


def test_generation_through_the_scheduler_matches_plain(cpu_engine):
    eng, (pc, pw), cfg = cpu_engine
    prompt = random_ids(9, cfg["vocab"], 3)
    out, reason = eng.generate(prompt, 7)
    assert reason == "length" and out == P.generate(pc, pw, prompt, 7)


def test_command_line_random_weights_mode(tmp_path):
    from test_cli import run_cli
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(ZULOPEL_B))
    out = tmp_path / "model"
    r = run_cli("--random-weights", str(out), "--config", str(cfg), "--seed", "4", "--dtype", "bf16")
    assert r.returncode == 0, r.stderr
    arch, parsed = config_from_dir(str(out))
    assert arch.name == "Zulopel" and parsed == ZulopelConfig.from_dict(ZULOPEL_B)
    assert set(P.read_safetensors(str(out / "model.safetensors"))) >= {"embed", "head", "l0.mix.sink", "l1.mix.A_log", "l2.mlp.e15.down", "l0.mlp.shared.up"}
