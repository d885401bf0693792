"""Host-side tests of the Zazilix family (no GPU): the loader's plan, the registry, and properties of the plain statement that
the GPU tests lean on."""
import copy
import json
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import zazilix_plain as plain  # noqa: E402

from calm_b200 import container, registry, seqlib, zazilix  # noqa: E402

MOE = {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 3, "identity": 2, "top": 2, "scale": 1.4}, "shared": {"ff": 10}}
CFG = {"architecture": "Zazilix", "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5}, "vocab": 53, "width": 24, "streams": 3, "max_positions": 80, "layers": [
    {"type": "mlstm", "mixer": {"heads": 2, "dim": 8, "vdim": 12, "gate_cap": 7.0}, "mlp": MOE},
    {"type": "parallel", "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.4, "mask": {"size": 5}}, "right": {"heads": 2, "dim": 4, "vdim": 10},
                                   "left_scale": 0.7, "right_scale": 0.2}, "mlp": None},
    {"type": "mamba2", "mixer": {"heads": 2, "vdim": 6, "state": 8, "groups": 1, "conv": 3, "norm_groups": 2}, "mlp": MOE}]}


def as_f64(t):
    return {k: v.float().numpy().astype(np.float64) for k, v in t.items()}


def test_plan_binds_every_size_from_the_config():
    t = zazilix.random_tensors(CFG, 1)
    head, layers, up = zazilix.plan(CFG, t)
    assert head["streams"] == 3 and head["block"] == seqlib.BLOCK_HYPER and head["norm_scalar"] == 1 and head["max_positions"] == 80
    assert up[head["final_norm"]].shape == (1,) and up[head["pos_table"]].shape == (80, 24)
    a, b, c = layers
    assert a["type"] == seqlib.SEQ_MLSTM and up[a["w_in"]].shape == (2 * 8 * 2 + 2 * 12 * 2 + 2 * 2, 24) and a["gate_cap"] == 7.0
    assert torch.equal(up[a["w_in"]][-2:], t["l0.mix.f"]) and torch.equal(up[a["b_in"]][-4:-2], t["l0.mix.i.b"]) and not up[a["b_in"]][:-4].any()
    assert a["experts"] == 3 and a["ident"] == 2 and a["route_mode"] == 1 and a["route_scale"] == 1.4 and a["shared_ff"] == 10
    assert "w_router" not in a and up[a["w_sh_gate_up"]].shape == (2 * 10 + 5, 24) and torch.equal(up[a["w_sh_gate_up"]][20:], t["l0.mlp.router"])
    assert up[a["w_gate_up"]].shape == (3 * 24, 24) and torch.equal(up[a["w_gate_up"]][12:24], t["l0.mlp.e0.up"])
    assert b["type"] == seqlib.SEQ_PAIR and b["pair_scale"] == [0.7, 0.2] and "ff" not in b
    left, right = b["pair"]
    assert left["type"] == seqlib.SEQ_GQA and left["chunk"] == 5 and left["dist_bias"] == left["add_one"] == left["v_norm"] == left["no_gate"] == 1
    assert up[left["w_in"]].shape == (4 * 8 + 2 * 8 + 2 * 6, 24)
    assert right["type"] == seqlib.SEQ_HGRN2 and torch.equal(up[right["b_in"]][8:16], t["l1.mix.right.f.b"])
    assert c["type"] == seqlib.SEQ_MAMBA2 and c["dim"] == 8 and c["kv_heads"] == 1 and c["taps"] == 3 and c["norm_groups"] == 2
    assert len(a["hc1"]) == 3 and up[a["hc1"][2]].shape == (3, 3)


def test_plan_refuses_what_does_not_fit():
    t = zazilix.random_tensors(CFG, 1)
    wrong = copy.deepcopy(CFG)
    wrong["layers"][0]["mixer"]["heads"] = 3
    with pytest.raises(ValueError):
        zazilix.plan(wrong, t)
    short = dict(t)
    del short["l2.mix.conv.b"]
    with pytest.raises(KeyError):
        zazilix.plan(CFG, short)
    other = copy.deepcopy(CFG)
    other["layers"][1]["type"] = "attention"
    with pytest.raises(ValueError):
        zazilix.plan(other, t)


def test_registry_finds_the_family(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    container.write_tensors(str(tmp_path / "model.safetensors"), zazilix.random_tensors(CFG, 2))
    assert registry.architecture_of(str(tmp_path)) == "Zazilix"
    registry._defaults()
    assert registry.SEQ_LOADERS["Zazilix"] is zazilix.load
    back, _ = container.read_tensors(str(tmp_path / "model.safetensors"))
    assert back["l0.norm1"].shape == () and back["final.norm"].shape == ()


def test_plain_statement_is_causal_and_blocks_bound_the_attention():
    t = as_f64(zazilix.random_tensors(CFG, 3))
    rng = np.random.default_rng(0)
    a = [int(x) for x in rng.integers(0, 53, 30)]
    b = a[:20] + [int(x) for x in rng.integers(0, 53, 10)]
    la, lb = plain.forward(CFG, t, a), plain.forward(CFG, t, b)
    assert np.allclose(la[:20], lb[:20], atol=1e-12) and not np.allclose(la[20:], lb[20:])
    # the attention alone: a change at position 3 is invisible to position 5 (the next block of 5), visible to position 4
    mx = CFG["layers"][1]["mixer"]["left"]
    h = rng.normal(size=(12, 24))
    h2 = h.copy()
    h2[3] += 1.0
    o1, o2 = plain.chunk_attention(h, t, "l1.mix.left.", mx, 1e-5), plain.chunk_attention(h2, t, "l1.mix.left.", mx, 1e-5)
    assert not np.allclose(o1[4], o2[4]) and np.allclose(o1[5:], o2[5:], atol=1e-12) and np.allclose(o1[:3], o2[:3], atol=1e-12)


def test_penalty_per_head_and_the_one_in_the_denominator():
    assert np.allclose(plain.slopes(8), [2.0 ** -(k + 1) for k in range(8)])
    assert np.allclose(plain.slopes(3), [2.0 ** (-8 / 3), 2.0 ** (-16 / 3), 2.0 ** -8])
    # one key with score s: its weight is e^s / (1 + e^s); a single very negative score leaves almost nothing
    t = as_f64(zazilix.random_tensors(CFG, 4))
    mx = dict(CFG["layers"][1]["mixer"]["left"], scale=0.0)
    h = np.random.default_rng(1).normal(size=(1, 24))
    out = plain.chunk_attention(h, t, "l1.mix.left.", mx, 1e-5)
    v = plain.rms((h @ t["l1.mix.left.v"].T).reshape(1, 2, 6), 1e-5)
    want = np.concatenate([0.5 * v[0, a // 2] for a in range(4)]) @ t["l1.mix.left.o"].T
    assert np.allclose(out[0], want)


def test_router_ties_scale_and_identity():
    w = {"r.router": np.zeros((4, 6)), "r.correction": np.array([0.0, 0.2, 0.0, 0.1])}
    ml = {"router": {"experts": 2, "identity": 2, "top": 2, "scale": 3.0}}
    chosen, wt = plain.route(np.ones((1, 6)), w, "r.", ml)
    assert chosen.tolist() == [[1, 3]] and np.allclose(wt, 0.75)  # equal scores 1/4 each: the correction alone decides, weights are score * scale
    w["r.correction"] = np.zeros(4)
    assert plain.route(np.ones((1, 6)), w, "r.", ml)[0].tolist() == [[0, 1]]  # ties go to the lowest index
    # both choices identity: the output is the input times the sum of the weights
    w["r.correction"] = np.array([0.0, 0.0, 1.0, 1.0])
    h = np.arange(6.0)[None]
    assert np.allclose(plain.experts(h, w, "r.", ml), 1.5 * h)


def test_one_stream_with_unit_connections_is_the_plain_residual():
    cfg = copy.deepcopy(CFG)
    cfg["streams"] = 1
    t = zazilix.random_tensors(cfg, 5)
    for k in list(t):
        if ".hc" in k:
            t[k] = torch.ones_like(t[k])
    p = as_f64(t)
    toks = [3, 9, 27, 1, 4]
    x = p["embed"][toks] * 2.0 + p["pos"][:5]
    for i, lc in enumerate(cfg["layers"]):
        x = x + plain.MIXERS[lc["type"]](plain.rms(x, 1e-5) * p[f"l{i}.norm1"], p, f"l{i}.mix.", lc["mixer"], 1e-5)
        if lc["mlp"]:
            x = x + plain.experts(plain.rms(x, 1e-5) * p[f"l{i}.norm2"], p, f"l{i}.mlp.", lc["mlp"])
    assert np.allclose(plain.forward(cfg, p, toks), (plain.rms(x, 1e-5) * p["final.norm"]) @ p["head"].T)
