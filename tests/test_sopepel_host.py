"""Host-side tests of the Sopepel family (no GPU): the loader's plan, the registry, and properties of the plain statement that
the GPU tests lean on."""
import copy
import json
import math
import os
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import sopepel_plain as plain  # noqa: E402

from calm_b200 import container, registry, seqlib, sopepel  # noqa: E402

MOE = {"kind": "moe", "expert": {"ff": 12}, "router": {"experts": 3, "top": 2}, "shared": {"ff": 10}}
LEFT = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.4, "mask": {"size": 5}, "rot": {"dims": 4, "base": 100.0}}
RIGHT = {"heads": 2, "dim": 4, "vdim": 10, "tau": 3.0, "a_rank": 5}
MIX = {"left": LEFT, "right": RIGHT, "left_scale": 0.7, "right_scale": 0.2}
CFG = {"architecture": "Sopepel", "embedding": {"bigram": {"buckets": 11, "mul_prev": 7, "mul_cur": 3}}, "norm": {"eps": 1e-5}, "vocab": 53, "width": 24, "logit_scale": 1.25,
       "layers": [{"type": "parallel", "mixer": MIX, "mlp": MOE}, {"type": "parallel", "mixer": MIX, "mlp": None},
                  {"type": "parallel", "mixer": MIX, "mlp": {"kind": "dense", "ff": 14}}, {"type": "parallel", "mixer": MIX, "mlp": {"kind": "moe", "expert": {"ff": 6}, "router": {"experts": 2, "top": 1}}}]}


def as_f64(t):
    return {k: v.float().numpy().astype(np.float64) for k, v in t.items()}


def test_plan_binds_every_size_from_the_config():
    t = sopepel.random_tensors(CFG, 1)
    head, layers, up = sopepel.plan(CFG, t)
    assert head["block"] == seqlib.BLOCK_POST and head["norm_kind"] == seqlib.NORM_RMS and head["norm_offset"] == 0.0 and head["logit_scale"] == 1.25
    assert head["head"] == head["embed"] == "embed" and up[head["bigram"]].shape == (12, 24)
    assert (head["bigram_buckets"], head["bigram_mul_prev"], head["bigram_mul_cur"]) == (11, 7, 3)
    a, b, c, d = layers
    assert a["type"] == seqlib.SEQ_PAIR and a["pair_scale"] == [0.7, 0.2]
    left, right = a["pair"]
    assert left["type"] == seqlib.SEQ_GQA and left["chunk"] == 5 and left["window"] == 0 and left["rot_dims"] == 4 and left["rot_base"] == 100.0
    assert left["qk_per_head"] == left["gate_per_head"] == left["scores_f32"] == 1 and left["kv_heads"] == 2
    # one input matrix for the pair: the left's 64 rows [q | k | v | g] (a multiple of 8 already), then the right's [q | k | v | g | a1]
    assert "w_in" not in left and "w_in" not in right and up[a["w_in"]].shape == (64 + 2 * 2 * 4 + 2 * 2 * 10 + 5, 24)
    assert torch.equal(up[a["w_in"]][60:64], t["l0.mix.left.g"]) and torch.equal(up[a["w_in"]][64:72], t["l0.mix.right.q"]) and torch.equal(up[a["w_in"]][-5:], t["l0.mix.right.a1"])
    assert torch.equal(up[a["b_in"]][32:48], t["l0.mix.left.k.b"]) and not up[a["b_in"]][60:].any() and up[a["b_in"]].shape == (up[a["w_in"]].shape[0],)
    assert up[left["q_norm"]].shape == (8,) and up[left["b_o"]].shape == (24,)
    assert right["type"] == seqlib.SEQ_GLA and right["a_rank"] == 5 and right["tau"] == 3.0
    assert a["ff_kind"] == seqlib.FF_MOE and a["experts"] == 3 and a["top"] == 2 and a["route_mode"] == 2 and a["expert_act"] == a["weight_input"] == a["shared_gate"] == 1
    assert "w_router" not in a and up[a["w_sh_gate_up"]].shape == (1 + 3 + 10, 24)
    assert torch.equal(up[a["w_sh_gate_up"]][:1], t["l0.mlp.shared.sg"]) and torch.equal(up[a["w_sh_gate_up"]][1:4], t["l0.mlp.router"])
    assert up[a["w_gate_up"]].shape == (3 * 12, 24) and torch.equal(up[a["w_gate_up"]][12:24], t["l0.mlp.e1.up"]) and up[a["w_down"]].shape == (3 * 24, 12)
    assert "ff" not in b and "norm2" not in b
    assert c["ff_kind"] == seqlib.FF_GATED and c["ff_act"] == seqlib.ACT_GELU_TANH and torch.equal(up[c["w_gate_up"]][14:], t["l2.mlp.up"])
    assert d["w_router"] == "l3.mlp.router" and "shared_ff" not in d and d["top"] == 1


def test_plan_refuses_what_does_not_fit():
    t = sopepel.random_tensors(CFG, 1)
    wrong = copy.deepcopy(CFG)
    wrong["layers"][0]["mixer"]["left"]["heads"] = 3
    with pytest.raises(ValueError):
        sopepel.plan(wrong, t)
    short = dict(t)
    del short["l2.mix.left.o.b"]
    with pytest.raises(KeyError):
        sopepel.plan(CFG, short)
    other = copy.deepcopy(CFG)
    other["layers"][1]["type"] = "attention"
    with pytest.raises(ValueError):
        sopepel.plan(other, t)
    other = copy.deepcopy(CFG)
    other["layers"][2]["mlp"]["kind"] = "glu"
    with pytest.raises(ValueError):
        sopepel.plan(other, t)


def test_registry_finds_the_family(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    container.write_tensors(str(tmp_path / "model.safetensors"), sopepel.random_tensors(CFG, 2))
    assert registry.architecture_of(str(tmp_path)) == "Sopepel"
    registry._defaults()
    assert registry.SEQ_LOADERS["Sopepel"] is sopepel.load
    back, _ = container.read_tensors(str(tmp_path / "model.safetensors"))
    assert back["bigram"].shape == (12, 24) and "head" not in back


def test_records_match_the_header():
    """Every field the header adds for this family is in the ctypes mirror, in the header's order."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "include", "calm_b200_seq.h")).read()
    body = text[text.index("struct SeqLayer {"):text.index("struct SeqModel {")]
    names = [n for n, _ in seqlib.SeqLayer._fields_]
    tail = ["qk_per_head", "gate_per_head", "b_o", "scores_f32", "ff_act", "expert_act", "weight_input", "shared_gate"]
    assert names[-len(tail):] == tail
    at = [body.index(" " + n + ";") for n in tail]
    assert at == sorted(at)
    model = text[text.index("struct SeqModel {"):]
    mnames = [n for n, _ in seqlib.SeqModel._fields_]
    assert mnames[-5:] == ["bigram", "bigram_buckets", "bigram_mul_prev", "bigram_mul_cur", "logit_scale"]
    assert model.index("bigram;") < model.index("bigram_buckets, bigram_mul_prev, bigram_mul_cur;") < model.index("logit_scale;")


def test_plain_statement_is_causal_and_blocks_bound_the_attention():
    t = as_f64(sopepel.random_tensors(CFG, 3))
    rng = np.random.default_rng(0)
    a = [int(x) for x in rng.integers(0, 53, 30)]
    b = a[:20] + [int(x) for x in rng.integers(0, 53, 10)]
    la, lb = plain.forward(CFG, t, a), plain.forward(CFG, t, b)
    assert np.allclose(la[:20], lb[:20], atol=1e-12) and not np.allclose(la[20:], lb[20:])
    # the attention alone: a change at position 3 is invisible to position 5 (the next block of 5), visible to position 4
    h = rng.normal(size=(12, 24))
    h2 = h.copy()
    h2[3] += 1.0
    o1, o2 = plain.left_attention(t, "l1.mix.left.", LEFT, h, 1e-5), plain.left_attention(t, "l1.mix.left.", LEFT, h2, 1e-5)
    assert not np.allclose(o1[4], o2[4]) and np.allclose(o1[5:], o2[5:], atol=1e-12) and np.allclose(o1[:3], o2[:3], atol=1e-12)
    assert [j for j in range(12) if plain.sees(11, j, 5)] == [10, 11] and [j for j in range(12) if plain.sees(9, j, 5)] == [5, 6, 7, 8, 9]
    # the linear attention remembers across blocks
    r1, r2 = plain.right_linear(t, "l1.mix.right.", RIGHT, h, 1e-5), plain.right_linear(t, "l1.mix.right.", RIGHT, h2, 1e-5)
    assert np.allclose(r1[:3], r2[:3], atol=1e-12) and not np.allclose(r1[11], r2[11])


def test_bigram_rows_and_rotation_by_hand():
    t = {"embed": np.arange(53.0)[:, None] * np.ones((1, 2)), "bigram": 100.0 * np.arange(12.0)[:, None] * np.ones((1, 2))}
    bg = CFG["embedding"]["bigram"]
    x = plain.embed(t, bg, [4, 9, 9])
    assert x[0, 0] == 4 + 100 * 11                       # the first token: the last row
    assert x[1, 0] == 9 + 100 * ((4 * 7 + 9 * 3) % 11)   # (previous * 7 + token * 3) mod 11
    assert x[2, 0] == 9 + 100 * ((9 * 7 + 9 * 3) % 11)
    v = np.zeros((3, 1, 6))
    v[:, 0, 0] = 1.0   # channel 0 pairs with channel 2 (dims 4), channels 4 and 5 pass unchanged
    v[:, 0, 5] = 7.0
    r = plain.rotate(v, {"dims": 4, "base": 100.0})
    assert np.allclose(r[2, 0], [math.cos(2.0), 0.0, math.sin(2.0), 0.0, 0.0, 7.0])
    v[:] = 0.0
    v[:, 0, 1] = 1.0   # pair 1 turns by position * 100^(-2/4)
    assert np.allclose(plain.rotate(v, {"dims": 4, "base": 100.0})[2, 0], [0.0, math.cos(0.2), 0.0, math.sin(0.2), 0.0, 0.0])


def test_router_ties_weights_and_the_expert_form():
    sel, wt = plain.route(np.array([[0.0, 2.0, 2.0, -1.0]]), 2)
    assert sel.tolist() == [[1, 2]] and np.allclose(wt, 1.0 / (1.0 + math.exp(-2.0)))  # ties go to the lowest index; the weight is the score itself
    w = {"f.router": np.array([[10.0, 0.0], [0.0, 0.0]]), "f.e0.up": np.eye(2), "f.e0.down": np.eye(2), "f.e1.up": np.eye(2), "f.e1.down": np.eye(2)}
    ml = {"router": {"experts": 2, "top": 1}}
    h = np.array([[1.0, -3.0]])
    s = 1.0 / (1.0 + math.exp(-10.0))
    assert np.allclose(plain.experts(w, "f.", ml, h), [[(s * 1.0) ** 2, 0.0]])  # relu((s h))^2: the weight is squared with the input, the negative channel is cut
    assert np.allclose(plain.gelu_tanh(np.array([0.0, 1.0])), [0.0, 0.5 * (1.0 + math.tanh(math.sqrt(2.0 / math.pi) * 1.044715))])


def test_post_norm_block_by_hand():
    """One layer without feed-forward: x + norm1(mixer(x)), the mixer reading x itself, then the final norm against the embedding table."""
    cfg = copy.deepcopy(CFG)
    cfg["layers"] = cfg["layers"][1:2]
    t = as_f64(sopepel.random_tensors(cfg, 5))
    toks = [3, 9, 27, 1, 4, 4, 30]
    x = plain.embed(t, cfg["embedding"]["bigram"], toks)
    y = 0.7 * plain.left_attention(t, "l0.mix.left.", LEFT, x, 1e-5) + 0.2 * plain.right_linear(t, "l0.mix.right.", RIGHT, x, 1e-5)
    x = x + y / np.sqrt((y * y).mean(-1, keepdims=True) + 1e-5) * t["l0.norm1"]
    want = (x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-5) * t["final.norm"]) @ t["embed"].T * 1.25
    assert np.allclose(plain.forward(cfg, t, toks), want)
