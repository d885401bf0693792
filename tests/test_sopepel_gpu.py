"""The Sopepel family on the layer-list runtime against the plain float64 statement in sopepel_plain.py.

Every test makes its own small configuration and seeded weights.  float32 mode is compared tightly (it shows any wrong key, a
block edge that is one token off, a lost state or previous token, a wrong expert or weight); bfloat16 mode within bf16 rounding.
Where random weights would hide a fault the scores are sharpened (a large score scale, so that single keys dominate the softmax),
or one query and key are made to match."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import sopepel_plain as plain  # noqa: E402

pytestmark = pytest.mark.gpu

from calm_b200 import container, registry, serving, sopepel  # noqa: E402

DENSE = {"ff": 40, "kind": "dense"}


def moe(experts=6, top=2, ff=12, shared=20):
    ml = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        ml["shared"] = {"ff": shared}
    return ml


def pair(heads=6, kv_heads=2, dim=16, vdim=12, size=7, rot=8, base=300.0, scale=0.3, rheads=3, rdim=16, rvdim=24, tau=4.0, a_rank=6, ls=1.3, rs=0.6, mlp=DENSE):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        left["mask"] = {"size": size}
    if rot:
        left["rot"] = {"dims": rot, "base": base}
    right = {"heads": rheads, "dim": rdim, "vdim": rvdim, "tau": tau, "a_rank": a_rank}
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def config(layers, width=48, vocab=97, eps=1e-5, buckets=53, mul_prev=31, mul_cur=5, logit_scale=1.5):
    return {"architecture": "Sopepel", "embedding": {"bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}, "layers": layers,
            "norm": {"eps": eps}, "vocab": vocab, "width": width, "logit_scale": logit_scale}


def weights(cfg, seed=0):
    return sopepel.random_tensors(cfg, seed)


def as_f64(t):
    return {k: v.float().numpy().astype(np.float64) for k, v in t.items()}


def tokens(cfg, n, seed=1):
    return [int(x) for x in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]


def clear_rows(cfg, t, toks, dtype):
    """Rows that routing coin tosses cannot reach.  In bfloat16 the router's input carries the rounding of everything before it, so a
    score within a few hundredths of the next one may fall either way; that row then differs by an expert, not by rounding, and what
    later rows remember of it (the linear attention's state) differs too.  float32 needs no such care: every row counts."""
    keep = np.ones(len(toks), bool)
    if dtype == "float32":
        return keep
    plain.MARGINS.clear()
    plain.forward(cfg, as_f64(t), toks)
    for m in plain.MARGINS:
        keep &= m > 0.02
    if len(cfg["layers"]) > 1 and plain.MARGINS:
        keep = np.cumprod(keep).astype(bool)
    assert keep.sum() >= min(5, len(toks)), "too few rows with clear routing: choose another seed or a feed-forward without choices"
    return keep


def free_of_choices(dtype, **kw):
    """The feed-forward of tests that run in both modes with several layers: in bfloat16 every expert is taken (nothing to toss)."""
    ml = moe(**kw)
    if dtype != "float32":
        ml["router"]["top"] = ml["router"]["experts"]
    return ml


def rel_err_rows(got, ref, dtype="float32"):
    """Error of the worst row, relative to the spread of the reference logits.  In bfloat16 a few rows sit far above the others without
    any fault (a norm over a handful of values that happen to be small multiplies the rounding of what came before): there the measure
    is the larger of the ninth decile and a sixth of the worst row (a row computed from a wrong key or state is off by about one)."""
    d = got - ref
    d = d - d.mean(-1, keepdims=True)
    r = ref - ref.mean(-1, keepdims=True)
    rows = np.sqrt((d * d).mean(-1)) / np.sqrt((r * r).mean())
    if dtype == "float32":
        return float(rows.max())
    return float(max(np.quantile(rows, 0.9), rows.max() / 6))


rel_err = rel_err_rows
TOL = {"float32": 3e-5, "bfloat16": 4e-2}


def whole(model, toks):
    s = model.open()
    out = model.step([s], [toks], list(range(len(toks))))
    model.close_seq(s)
    return out


def check_all_ways(cfg, t, toks, dtype="float32", portions=(5, 2, 1), page=4):
    """whole prompt, prompt + token-by-token decoding, and portions: all against the plain statement."""
    ref = plain.forward(cfg, as_f64(t), toks)
    clear = clear_rows(cfg, t, toks, dtype)
    err = lambda got, want: rel_err_rows(got[clear], want[clear], dtype)  # noqa: E731
    with sopepel.from_tensors(cfg, t, dtype, max_tokens=4 * len(toks) + 64, max_seqs=4, page=page) as m:
        assert err(whole(m, toks), ref) < TOL[dtype]
        for first in {1, max(1, len(toks) // 2)}:
            s = m.open()
            rows = [m.step([s], [toks[:first]], list(range(first)))]
            for p in range(first, len(toks)):
                rows.append(m.step([s], [[toks[p]]], [0]))
            m.close_seq(s)
            assert err(np.concatenate(rows), ref) < TOL[dtype]
        for size in portions:
            s, rows, at = m.open(), [], 0
            while at < len(toks):
                part = toks[at:at + size]
                rows.append(m.step([s], [part], list(range(len(part)))))
                at += len(part)
                size = size + 1 if size > 2 else size  # growing portions: edges fall at ever different places
            m.close_seq(s)
            assert err(np.concatenate(rows), ref) < TOL[dtype]
    return ref


LAYERS = {
    "pair-dense": pair(),
    "pair-noff": pair(mlp=None),
    "mha-unbounded-full-rotation": pair(heads=3, kv_heads=3, dim=8, vdim=8, size=0, rot=8),
    "block-of-one-no-rotation": pair(heads=2, kv_heads=1, size=1, rot=0, rheads=1),
    "block-longer-than-prompt-unit-factors": pair(size=64, ls=1.0, rs=1.0),
    "one-head-each": pair(heads=1, kv_heads=1, dim=32, vdim=8, rot=2, rheads=1, rdim=8, rvdim=32, tau=1.0, a_rank=1),
    "wide-state": pair(rheads=2, rdim=64, rvdim=8, tau=16.0),
    "moe-top1-shared": pair(mlp=moe(experts=5, top=1)),
    "moe-top2-no-shared": pair(mlp=moe(experts=4, top=2, shared=0)),
    "moe-all-experts": pair(mlp=moe(experts=3, top=3, ff=20, shared=12)),
    "moe-one-expert": pair(mlp=moe(experts=1, top=1, ff=8, shared=8)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(LAYERS))
def test_each_mechanism_alone(name, dtype):
    cfg = config([LAYERS[name]])
    check_all_ways(cfg, weights(cfg, 3), tokens(cfg, 37), dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_align_with_nothing(dtype):
    """Width, head sizes, state sizes, expert widths, decay ranks, bucket counts and vocabulary that are multiples of neither 8 nor 4."""
    cfg = config([pair(heads=3, kv_heads=3, dim=10, vdim=7, size=5, rot=6, rheads=1, rdim=7, rvdim=5, a_rank=3, mlp=free_of_choices(dtype, experts=3, top=2, ff=9, shared=11)),
                  pair(heads=6, kv_heads=2, dim=6, vdim=10, size=9, rot=2, rheads=2, rdim=10, rvdim=6, a_rank=5, mlp={"ff": 13, "kind": "dense"}),
                  pair(heads=2, kv_heads=1, dim=14, vdim=3, size=0, rot=14, rheads=3, rdim=5, rvdim=9, mlp=free_of_choices(dtype, experts=2, top=1, ff=3, shared=0))],
                 width=50, vocab=61, buckets=17, mul_prev=1, mul_cur=1, logit_scale=1.0)
    check_all_ways(cfg, weights(cfg, 31), tokens(cfg, 45), dtype, portions=(17, 2))


def test_other_layer_orders():
    for k, order in enumerate(([pair(mlp=moe()), pair(mlp=None), pair(), pair(mlp=moe(top=1, shared=0))], [pair(mlp=None), pair(mlp=None), pair(size=4, mlp=moe(experts=2)), pair(), pair()])):
        cfg = config(order, width=40)
        check_all_ways(cfg, weights(cfg, 5 + k), tokens(cfg, 41), portions=(6,))


def test_residual_stream_after_every_layer():
    cfg = config([pair(), pair(mlp=moe()), pair(mlp=None), pair(mlp=moe(top=1))])
    t, toks = weights(cfg, 8), tokens(cfg, 19)
    trace = []
    plain.forward(cfg, as_f64(t), toks, trace)
    with sopepel.from_tensors(cfg, t, "float32", max_tokens=64, max_seqs=2) as m:
        m.set_trace(True)
        whole(m, toks)
        got = m.read_trace(len(toks))
    assert got.shape[0] == len(trace) == 4
    for g, r in zip(got, trace):
        assert np.abs(g - r).max() < 1e-4 * max(1.0, np.abs(r).max())


def test_block_edges_and_the_attention_details_show(monkeypatch):
    """Sharp scores: a block size that is one position off moves the logits far more than the tolerance, in prompts, portions and
    decoding alike (the same check passes for the right value); so do the norm per head and the gate per head when the plain
    statement reads them otherwise, and the rotation's constants."""
    cfg = config([pair(size=6, scale=1.5, ls=1.0, rs=0.2, mlp=None)])
    t, toks = weights(cfg, 11), tokens(cfg, 60)
    ref = check_all_ways(cfg, t, toks, portions=(7, 2))
    for off in (-1, 1):
        wrong = copy.deepcopy(cfg)
        wrong["layers"][0]["mixer"]["left"]["mask"]["size"] += off
        assert rel_err(plain.forward(wrong, as_f64(t), toks), ref) > 100 * TOL["float32"]
    for key, val in (("dims", 6), ("base", 200.0)):
        wrong = copy.deepcopy(cfg)
        wrong["layers"][0]["mixer"]["left"]["rot"][key] = val
        assert rel_err(plain.forward(wrong, as_f64(t), toks), ref) > 100 * TOL["float32"]
    for knob in ("norm_per_head", "gate_per_head"):
        monkeypatch.setitem(plain.KNOBS, knob, False)
        assert rel_err(plain.forward(cfg, as_f64(t), toks), ref) > 100 * TOL["float32"]
        monkeypatch.setitem(plain.KNOBS, knob, True)


def test_the_first_tokens_and_the_previous_token(monkeypatch):
    """The bigram row of a token depends on the token before it: the first token of a sequence takes the table's last row, the first
    token of a later portion the row of (last token of the portion before, token).  Portions of two and decoding pass only if the slot
    remembers that token; leaving the table out of the plain statement shows far above the tolerance."""
    cfg = config([pair(mlp=None)], buckets=7, mul_prev=3, mul_cur=2)
    t, toks = weights(cfg, 12), tokens(cfg, 24)
    ref = check_all_ways(cfg, t, toks, portions=(3, 2))
    monkeypatch.setitem(plain.KNOBS, "bigram", False)
    assert rel_err(plain.forward(cfg, as_f64(t), toks), ref) > 100 * TOL["float32"]
    monkeypatch.setitem(plain.KNOBS, "bigram", True)
    shifted = copy.deepcopy(cfg)
    shifted["embedding"]["bigram"]["mul_prev"] = 4
    assert rel_err(plain.forward(shifted, as_f64(t), toks), ref) > 100 * TOL["float32"]
    p = as_f64(t)
    with sopepel.from_tensors(cfg, t, "float32", max_tokens=64, max_seqs=2) as m:
        s = m.open()  # one token alone is a whole sequence: the last row of the table
        assert rel_err(m.step([s], [[toks[0]]], [0]), plain.forward(cfg, p, toks[:1])) < TOL["float32"]


def test_router_details_show(monkeypatch):
    """The weight is the sigmoid score itself (not renormalised), it goes in at the expert's input (relu^2 squares it), the shared
    unit is gated per token, and the logits are scaled."""
    cfg = config([pair(mlp=moe(experts=5, top=2, ff=16, shared=12))])
    t, toks = weights(cfg, 13), tokens(cfg, 40)
    ref = check_all_ways(cfg, t, toks, portions=(9,))
    p = as_f64(t)
    sel, wt = plain.route(np.random.default_rng(0).normal(size=(200, 5)), 2)
    assert not np.allclose(wt.sum(-1), 1.0) and (wt[:, 0] >= wt[:, 1]).all() and len(np.unique(sel)) == 5
    for knob in ("weight_on_input", "shared_gate"):
        monkeypatch.setitem(plain.KNOBS, knob, False)
        assert rel_err(plain.forward(cfg, p, toks), ref) > 100 * TOL["float32"]
        monkeypatch.setitem(plain.KNOBS, knob, True)
    other = copy.deepcopy(cfg)
    other["logit_scale"] = 1.0
    assert rel_err(plain.forward(other, p, toks), ref) > 100 * TOL["float32"]
    other = copy.deepcopy(cfg)
    other["layers"][0]["mlp"]["router"]["top"] = 1
    assert rel_err(plain.forward(other, p, toks), ref) > 100 * TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_context_with_shared_out_keys(dtype):
    """Decoding few tokens over a context of several hundred with no block bound (and with a block of 200): the attention kernel shares
    one query's keys out over several CTAs and folds the shares; positions in the hundreds turn the rotated channels by hundreds of
    radians; pages are crossed all along.  The recurrent states carry 128 key channels."""
    cfg = config([pair(heads=4, kv_heads=2, size=0, scale=1.0 if dtype == "float32" else 0.3, rot=16, base=50.0, rheads=1, rdim=128, rvdim=16, mlp=None),
                  pair(size=200, scale=0.3, mlp=None)])
    t, toks = weights(cfg, 15), tokens(cfg, 330)
    ref = plain.forward(cfg, as_f64(t), toks)
    with sopepel.from_tensors(cfg, t, dtype, max_tokens=700, max_seqs=2, page=16) as m:
        s = m.open()
        rows = [m.step([s], [toks[:300]], list(range(300)))]
        for p in range(300, 330):
            rows.append(m.step([s], [[toks[p]]], [0]))
        assert rel_err(np.concatenate(rows), ref, dtype) < TOL[dtype]
        s2 = m.open()  # the same prompt in two-token portions beside the finished sequence
        rows = [m.step([s2], [toks[a:a + 2]], [0, 1]) for a in range(0, 330, 2)]
        assert rel_err(np.concatenate(rows), ref, dtype) < TOL[dtype]


def test_a_far_key_stands_out_inside_its_block_and_not_outside():
    """One position holds a key that later queries match.  Queries and keys come from the same projection, which reads only the first
    half of the input columns; token 5 and token 3 share that half of their embedding rows (the bigram rows leave it alone), so the
    queries of token 3 score the key of token 5 as high as their own, far above every other key, while its value differs.  With a
    block of 128 a query near the end of the block still finds that key 120 positions back, the queries of the next blocks do not;
    without a block bound they find it hundreds of positions back.  Prompt and decoding alike."""
    for size in (128, 0):
        cfg = config([pair(heads=2, kv_heads=1, dim=32, vdim=8, size=size, rot=0, scale=1.0, ls=1.0, rs=0.1, mlp=None)])
        t, toks = weights(cfg, 16), tokens(cfg, 300)
        half = cfg["width"] // 2
        t["l0.mix.left.k"][:, half:] = 0
        t["l0.mix.left.q"] = torch.cat([t["l0.mix.left.k"], t["l0.mix.left.k"]], 0)
        t["l0.mix.left.q.b"] = torch.cat([t["l0.mix.left.k.b"], t["l0.mix.left.k.b"]], 0)
        t["l0.mix.left.q.norm"] = t["l0.mix.left.k.norm"] = torch.ones(32, dtype=torch.bfloat16)
        t["bigram"][:, :half] = 0
        t["embed"][5, :half] = t["embed"][3, :half]
        for x in range(len(toks)):  # the key at 5; queries near the end of its block, at the start of the next, and far away
            toks[x] = 5 if x == 5 else 3 if x in (126, 128, 299) else 4 if toks[x] in (3, 5) else toks[x]
        ref = plain.forward(cfg, as_f64(t), toks)
        other = copy.deepcopy(cfg)
        if size:
            del other["layers"][0]["mixer"]["left"]["mask"]
        else:
            other["layers"][0]["mixer"]["left"]["mask"] = {"size": 128}
        diff = plain.forward(other, as_f64(t), toks)
        assert rel_err(diff[128:129], ref[128:129]) > 100 * TOL["float32"] and rel_err(diff[299:], ref[299:]) > 100 * TOL["float32"]
        assert rel_err(diff[126:127], ref[126:127]) < 1e-9  # the same block either way
        with sopepel.from_tensors(cfg, t, "float32", max_tokens=1024, max_seqs=2, page=16) as m:
            assert rel_err(whole(m, toks), ref) < TOL["float32"]
            s = m.open()
            rows = [m.step([s], [toks[:120]], list(range(120)))] + [m.step([s], [[x]], [0]) for x in toks[120:135]] + [m.step([s], [toks[135:290]], list(range(155)))]
            rows += [m.step([s], [[x]], [0]) for x in toks[290:]]
            assert rel_err(np.concatenate(rows), ref) < TOL["float32"]


def test_the_state_remembers_what_the_block_bound_hides():
    """A decay close to one keeps the first tokens in the linear attention's state: changing token 2 moves the logits hundreds of
    positions later although every attention block there starts long after it; with a fast decay it does not.  The runtime follows the
    plain statement in both cases, through a prompt in portions and decoding."""
    for bias, moved in ((9.0, True), (-6.0, False)):
        cfg = config([pair(size=16, rs=1.0, tau=8.0 if moved else 0.5, mlp=None)])
        t, toks = weights(cfg, 19), tokens(cfg, 260)
        t["l0.mix.right.a2.b"] = torch.full_like(t["l0.mix.right.a2.b"], bias)
        t["l0.mix.right.a2"] = torch.zeros_like(t["l0.mix.right.a2"])
        p = as_f64(t)
        ref = plain.forward(cfg, p, toks)
        changed = list(toks)
        changed[2] = (toks[2] + 1) % cfg["vocab"]
        far = rel_err(plain.forward(cfg, p, changed)[250:], ref[250:])
        assert far > 100 * TOL["float32"] if moved else far < TOL["float32"]
        with sopepel.from_tensors(cfg, t, "float32", max_tokens=600, max_seqs=2, page=8) as m:
            s = m.open()
            rows = [m.step([s], [toks[:100]], list(range(100))), m.step([s], [toks[100:240]], list(range(140)))] + [m.step([s], [[x]], [0]) for x in toks[240:]]
            assert rel_err(np.concatenate(rows), ref) < TOL["float32"]


def test_prompt_attention_as_products_keeps_the_scores_exact(monkeypatch):
    """bfloat16 mode computes a long portion's attention as tensor-core products over gathered keys, short portions with the fused fp32
    kernel.  Scores and softmax weights keep fp32 accuracy on both (queries, keys and probabilities travel as bf16 value + remainder
    pairs), so with sharp scores -- where a key rounded to bf16 alone would move the weights by percents -- the two agree as closely
    as the rest of the bf16 path allows, also for a portion that continues a cached prefix in the middle of a block of positions; a
    block size that is one off shows far above that."""
    for size in (23, 4, 0):
        cfg = config([pair(size=size, scale=2.0, ls=1.0, rs=0.3, mlp=None), pair(size=0, heads=4, kv_heads=4, dim=8, vdim=8, scale=1.0, mlp=DENSE)])
        t, toks = weights(cfg, 17), tokens(cfg, 120)
        ref = plain.forward(cfg, as_f64(t), toks)
        errs, outs = {}, {}
        for products in ("1", "0"):
            monkeypatch.setenv("CALM_B200_SEQ_ATTN_PRODUCTS", products)
            with sopepel.from_tensors(cfg, t, "bfloat16", max_tokens=300, max_seqs=3, page=8) as m:
                s1, s2 = m.open(), m.open()
                a = m.step([s1], [toks[:50]], list(range(50)))
                b = m.step([s1, s2], [toks[50:], toks[:3]], list(range(73)))  # 70 more tokens on the products path beside a 3-token portion
                outs[products] = np.concatenate([a, b[:70]])
                errs[products] = rel_err(outs[products], ref, "bfloat16")
                assert rel_err(b[70:], ref[:3], "bfloat16") < TOL["bfloat16"]
        assert errs["1"] < TOL["bfloat16"] and errs["0"] < TOL["bfloat16"] and errs["1"] < 1.5 * errs["0"] + 1e-3
        if size:
            for off in (-1, 1):
                wrong = copy.deepcopy(cfg)
                wrong["layers"][0]["mixer"]["left"]["mask"]["size"] += off
                assert rel_err(plain.forward(wrong, as_f64(t), toks), ref) > 4 * errs["1"]


def test_tensor_core_products_match_the_warp_level_ones(monkeypatch):
    """bfloat16 mode runs products over many tokens on tcgen05 (the grouped ones of the experts included, with the weight per row and
    the split epilogue of the shared unit's first product) and everything else on mma.sync; same bf16 inputs, fp32 sums in another order."""
    cfg = config([pair(heads=2, kv_heads=1, dim=32, vdim=24, size=50, rdim=32, rvdim=40, a_rank=8, mlp=moe(experts=5, top=5, ff=40, shared=56)),
                  pair(heads=4, kv_heads=2, dim=32, vdim=24, size=0, rdim=32, rvdim=40, a_rank=8, mlp={"ff": 72, "kind": "dense"}),
                  pair(heads=4, kv_heads=4, dim=16, vdim=24, rheads=2, rdim=32, rvdim=24, a_rank=8, mlp=moe(experts=3, top=3, ff=72, shared=0))], width=88, vocab=131)
    t, toks = weights(cfg, 18), tokens(cfg, 300)
    outs = {}
    for tc in ("1", "0"):
        monkeypatch.setenv("CALM_B200_SEQ_TC", tc)
        with sopepel.from_tensors(cfg, t, "bfloat16", max_tokens=640, max_seqs=2, page=16) as m:
            s1 = m.open()
            outs[tc] = np.concatenate([m.step([s1], [toks[:237]], list(range(237))), m.step([s1], [toks[237:]], list(range(63)))])
            if tc == "1":
                m.perf(True)
                whole(m, toks)
                stats = m.perf_stats()
                m.perf(False)
                assert stats["gemm_tcgen05"][3] > 0
    assert rel_err(outs["1"], outs["0"]) < 5e-3  # identical inputs; intermediate bf16 roundings may flip on last-bit differences
    assert rel_err(outs["1"], plain.forward(cfg, as_f64(t), toks), "bfloat16") < TOL["bfloat16"]


def test_long_decoding_keeps_state():
    """130 tokens one by one: the recurrent state, the previous token and the cache grow by single steps, over many blocks and pages."""
    cfg = config([pair(), pair(size=12, mlp=moe()), pair(mlp=None)])
    t, toks = weights(cfg, 14), tokens(cfg, 130)
    ref = plain.forward(cfg, as_f64(t), toks)
    with sopepel.from_tensors(cfg, t, "float32", max_tokens=200, max_seqs=2, page=8) as m:
        s = m.open()
        rows = [m.step([s], [[x]], [0]) for x in toks]
        assert rel_err(np.concatenate(rows), ref) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_equals_each_alone(dtype):
    ml = free_of_choices(dtype)
    cfg = config([pair(mlp=ml), pair(), pair(size=4, mlp=ml), pair(mlp=None)])
    t = weights(cfg, 21)
    prompts = [tokens(cfg, n, seed=n) for n in (1, 9, 40, 2)]
    tails = [tokens(cfg, n, seed=50 + n) for n in (6, 3, 0, 6)]
    p = as_f64(t)
    refs = [plain.forward(cfg, p, a + b) for a, b in zip(prompts, tails)]
    with sopepel.from_tensors(cfg, t, dtype, max_tokens=192, max_seqs=5, page=4) as m:
        slots = [m.open() for _ in prompts]
        out = m.step(slots, prompts, list(range(sum(len(a) for a in prompts))))
        got, at = [], 0
        for a in prompts:
            got.append([out[at:at + len(a)]])
            at += len(a)
        for k in range(6):  # decoded together; the shorter ones leave earlier
            live = [i for i, b in enumerate(tails) if k < len(b)]
            o = m.step([slots[i] for i in live], [[tails[i][k]] for i in live], list(range(len(live))))
            for j, i in enumerate(live):
                got[i].append(o[j:j + 1])
        for i, r in enumerate(refs):
            assert rel_err(np.concatenate(got[i]), r, dtype) < TOL[dtype]
        if dtype == "float32":  # a row does not depend on what else is in the batch, beyond rounding
            alone = whole(m, prompts[2])
            assert np.abs(alone - np.concatenate(got[2])[:40]).max() < 1e-5 * np.abs(alone).max()


def test_slots_and_pages_are_used_again():
    """A slot that is opened again starts from zero state, no previous token and fresh pages."""
    cfg = config([pair(), pair(mlp=moe()), pair(mlp=None)])
    t = weights(cfg, 22)
    p = as_f64(t)
    with sopepel.from_tensors(cfg, t, "float32", max_tokens=48, max_seqs=2, page=4) as m:
        free0 = m.free_pages()
        for rnd in range(4):  # every pass fills the pool almost completely, with other lengths than the pass before
            a, b = tokens(cfg, 20 + rnd, seed=rnd), tokens(cfg, 23 - rnd, seed=9 + rnd)
            sa, sb = m.open(), m.open()
            out = m.step([sa, sb], [a, b], list(range(len(a) + len(b))))
            assert rel_err(out[:len(a)], plain.forward(cfg, p, a)) < TOL["float32"]
            assert rel_err(out[len(a):], plain.forward(cfg, p, b)) < TOL["float32"]
            m.close_seq(sb if rnd % 2 else sa)
            m.close_seq(sa if rnd % 2 else sb)
            assert m.free_pages() == free0
        s = m.open()
        with pytest.raises(Exception):
            m.step([s], [tokens(cfg, 4 * free0 + 1)], [0])  # more than the pool holds: refused, nothing has run
        assert m.length(s) == 0
        one = tokens(cfg, 3, seed=77)  # the refused step left no previous token behind
        assert rel_err(m.step([s], [one], [0, 1, 2]), plain.forward(cfg, p, one)) < TOL["float32"]


def test_greedy_generation_through_the_scheduler():
    cfg = config([pair(), pair(mlp=moe()), pair(mlp=None)])
    t = weights(cfg, 23)
    p = as_f64(t)
    prompts = [tokens(cfg, n, seed=70 + n) for n in (5, 17, 1)]
    with sopepel.from_tensors(cfg, t, "float32", max_tokens=256, max_seqs=2, page=8) as m:
        outs = serving.generate(m, prompts, 12, max_batch=2)  # three requests, two slots: a second batch follows the first
        assert m.free_pages() == 256 // 8 + 2
    for pr, out in zip(prompts, outs):
        assert len(out) == 12
        lg = plain.forward(cfg, p, pr + out)
        for k, tok in enumerate(out):  # each generated token is the plain statement's argmax given the same history
            row = lg[len(pr) + k - 1]
            assert tok == int(row.argmax()) or row.max() - row[tok] < 1e-4 * np.abs(row).max()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_from_a_model_folder(tmp_path, dtype):
    """bin/trace_run end to end: a model folder written with the container writer and found through the registry, steps on
    standard input (a batch of unequal prompts, decoding together while requests leave, a second batch afterwards), logits
    files compared with the plain statement."""
    ml = free_of_choices(dtype)
    cfg = config([pair(heads=4, kv_heads=1, dim=16, vdim=8, size=11, scale=0.5, mlp=ml), pair(heads=2, kv_heads=2, dim=8, vdim=8, size=3, rheads=1, rdim=8, rvdim=40, mlp=None),
                  pair(mlp={"ff": 24, "kind": "dense"})], width=72, vocab=211, eps=1e-6, logit_scale=0.7)
    t = weights(cfg, 41)
    folder, out = tmp_path / "model", tmp_path / "out"
    folder.mkdir(), out.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    container.write_tensors(str(folder / "model.safetensors"), t)
    assert registry.architecture_of(str(folder)) == "Sopepel"
    # (request c takes other tokens than seed 3 would give.  At a sequence's first token the linear attention reads out (q.k) v, and the norm
    # behind it leaves sign(q.k) v / rms(v): for that seed's first token one head has q.k = -0.001 against |q||k| = 3.7, so bf16 rounding
    # decides the sign of that head's whole output -- float32 shows the same row at ten times the others' error)
    reqs = {"a": tokens(cfg, 46, 1), "b": tokens(cfg, 9, 2), "c": tokens(cfg, 4, 7), "d": tokens(cfg, 30, 4), "e": tokens(cfg, 2, 5)}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": reqs["a"][:40], "want": [0, 17, 39]}, {"id": "b", "tokens": reqs["b"][:6], "want": [5]},
                                     {"id": "c", "tokens": reqs["c"][:1], "want": [0]}], "end": []}]
    for k in range(3):
        ent = [{"id": "a", "tokens": [reqs["a"][40 + k]], "want": [0]}, {"id": "b", "tokens": [reqs["b"][6 + k]], "want": [0] if k != 1 else []},
               {"id": "c", "tokens": [reqs["c"][1 + k]], "want": [0]}]
        steps.append({"step": 1 + k, "entries": ent, "end": ["b", "c"] if k == 2 else []})
    for k in range(3):
        steps.append({"step": 4 + k, "entries": [{"id": "a", "tokens": [reqs["a"][43 + k]], "want": [0]}], "end": ["a"] if k == 2 else []})
    steps.append({"step": 7, "entries": [{"id": "d", "tokens": reqs["d"][:29], "want": [28]}, {"id": "e", "tokens": reqs["e"][:1], "want": []}], "end": []})
    steps.append({"step": 8, "entries": [{"id": "d", "tokens": reqs["d"][29:], "want": [0]}, {"id": "e", "tokens": reqs["e"][1:], "want": [0]}], "end": ["d", "e"]})
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.run([os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype", dtype, "--out", str(out), "--max-tokens", "96"],
                       input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [ln for ln in p.stdout.splitlines() if ln.startswith("done")] == ["done %d" % s["step"] for s in steps]
    ref = {k: plain.forward(cfg, as_f64(t), v) for k, v in reqs.items()}
    at = {k: 0 for k in reqs}
    for s in steps:
        rows = []
        for e in s["entries"]:
            rows += [ref[e["id"]][at[e["id"]] + w] for w in e["want"]]
            at[e["id"]] += len(e["tokens"])
        path = out / ("%d.f32" % s["step"])
        if rows:
            got = np.fromfile(path, "<f4").reshape(len(rows), cfg["vocab"])
            assert rel_err(got, np.stack(rows), dtype) < TOL[dtype]
        else:
            assert not path.exists()
