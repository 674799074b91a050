"""Vapelix without a GPU: configuration, description, layer order, and the engine's host logic (batching,
pages, the order of parts) on the CPU test double of the kernels, against the plain implementation."""
import copy

import numpy as np
import pytest
import torch

import llmengine
import plain_vapelix as P
from cpu_ops import CpuOps
from llmengine.config.files import ConfigError
from llmengine.config.registry import config_from_dir, get_architecture
from llmengine.config.vapelix import VapelixConfig
from llmengine.models.vapelix import describe_vapelix, layer_order
from llmengine.parts.position import ramp_frequencies
from llmengine.parts.spec import ScaledRotarySpec
from tiny import make_model_dir, random_ids
from tiny_vapelix import VAPELIX, VAPELIX_A, VAPELIX_B


def test_configuration_round_trip_and_errors():
    cfg = VapelixConfig.from_dict(VAPELIX_A)
    assert cfg.width == 72 and cfg.vocab_size == 301 and cfg.side_dim == 6 and cfg.loop.times == 3
    assert cfg.layers[2].mlp is None and cfg.layers[1].mlp.top == 2 and cfg.layers[0].mlp.kind == "dense"
    assert VapelixConfig.from_dict(cfg.to_dict()) == cfg
    assert VapelixConfig.from_dict(VAPELIX_B).loop is None and VapelixConfig.from_dict(VAPELIX_B).side_dim == 0
    for path, value in ((("width",), None), (("layers", 0, "type"), "conv"), (("layers", 1, "mlp", "kind"), "sparse"),
                        (("loop", "stop"), 9), (("layers", 0, "mixer", "rot", "dims"), 7), (("layers", 3, "mlp", "router", "top"), 4)):
        bad = copy.deepcopy(VAPELIX_A)
        d = bad
        for k in path[:-1]:
            d = d[k]
        if value is None:
            del d[path[-1]]
        else:
            d[path[-1]] = value
        with pytest.raises(ConfigError):
            VapelixConfig.from_dict(bad)


def test_layer_order_and_tensor_names():
    cfg = VapelixConfig.from_dict(VAPELIX_A)
    order = layer_order(cfg)
    assert [(r.layer, r.add_embedding) for r in order] == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True),
                                                           (2, False), (3, False)]
    assert [(i, again) for i, again in P.run_order(VAPELIX_A)] == [(r.layer, r.add_embedding) for r in order]
    spec = describe_vapelix(cfg)
    from llmengine.weights.random_init import model_tensor_needs
    names = set(model_tensor_needs(spec))
    assert {"embed", "side.embed", "final.norm", "l0.mlp.gate", "l1.mlp.e4.down", "l1.mlp.router.b", "l2.mix.dkv.norm",
            "l3.side.proj", "l0.norm2"} <= names
    assert "l2.norm2" not in names and "l2.norm2" in spec.ignore and "l1.mlp.e5.up" not in names
    assert get_architecture("Vapelix").name == "Vapelix"


def test_rotation_frequencies_match_plain():
    for rot in (VAPELIX_A["layers"][0]["mixer"]["rot"], VAPELIX_B["layers"][1]["mixer"]["rot"]):
        sc = rot.get("scaling") or {}
        spec = ScaledRotarySpec("rope_ramp", rot["dims"], rot["base"], 16, sc.get("factor", 0.0), sc.get("original", 0.0),
                                sc.get("fast", 0.0), sc.get("slow", 0.0))
        f, m = ramp_frequencies(spec)
        pf, pm = P.rotary_frequencies(rot)
        np.testing.assert_allclose(f, np.asarray(pf), rtol=1e-12)
        assert abs(m - pm) < 1e-12
    ramp = VAPELIX_A["layers"][0]["mixer"]["rot"]
    plain, _ = P.rotary_frequencies({"dims": ramp["dims"], "base": ramp["base"]})
    scaled, _ = P.rotary_frequencies(ramp)
    assert scaled[0] == plain[0] and scaled[-1] < plain[-1], "the ramp leaves the fastest pair and slows the slowest"


@pytest.fixture(scope="module", params=["va", "vb"])
def cpu_engine(request, tmp_path_factory):
    cfg, page = VAPELIX[request.param]
    d = str(tmp_path_factory.mktemp("vapelix_" + request.param))
    make_model_dir(d, cfg, torch.float32)
    arch, parsed = config_from_dir(d)
    assert arch.name == "Vapelix" and parsed == VapelixConfig.from_dict(cfg)
    eng = llmengine.Engine(d, "fp32", device="cpu", ops=CpuOps(), block_size=page, num_blocks=40)
    eng.configure_cache(num_blocks=40, block_size=page, num_slots=3)
    return eng, P.read_model(d), cfg


def test_engine_on_the_test_double_matches_plain(cpu_engine):
    eng, (pc, pw), cfg = cpu_engine
    a, b = random_ids(37, cfg["vocab"], 1), random_ids(11, cfg["vocab"], 2)
    want = {k: P.forward(pc, pw, ids)[0].numpy() for k, ids in (("a", a), ("b", b))}
    got = eng.run_step([(1, a, list(range(len(a))))], end=[1]).numpy()
    assert np.abs(got - want["a"]).max() < 2e-4
    # portions beside single tokens of another request; pages are given back and used again
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
    import json
    from test_cli import run_cli
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(VAPELIX_B))
    out = tmp_path / "model"
    r = run_cli("--random-weights", str(out), "--config", str(cfg), "--seed", "4", "--dtype", "bf16")
    assert r.returncode == 0, r.stderr
    arch, parsed = config_from_dir(str(out))
    assert arch.name == "Vapelix" and parsed == VapelixConfig.from_dict(VAPELIX_B)
    assert set(P.read_safetensors(str(out / "model.safetensors"))) >= {"embed", "l0.mlp.e5.up", "l1.mlp.down", "final.norm"}
