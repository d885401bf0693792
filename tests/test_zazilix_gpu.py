"""The Zazilix family on the layer-list runtime against the plain float64 statement in zazilix_plain.py.

Every test makes its own small configuration and seeded weights.  float32 mode is compared tightly (it shows a block edge that
is one position off, a lost or wrongly started state, a missing sink, a wrong expert); bfloat16 mode within bf16 rounding.
Where random weights would hide a fault the scores are sharpened (a large score scale, so that single keys dominate the
softmax) or the plain statement is run with one mechanism switched off, to show that the mechanism reaches the logits."""
import copy
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import zazilix_plain as plain  # noqa: E402

pytestmark = pytest.mark.gpu

from calm_b200 import container, registry, serving, zazilix  # noqa: E402


def moe(experts=5, identity=2, top=2, ff=12, scale=1.3, shared=20):
    ml = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": scale}}
    if shared:
        ml["shared"] = {"ff": shared}
    return ml


MOE = moe()


def mlstm(heads=3, dim=16, vdim=20, cap=9.0, mlp=MOE):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def pair(heads=6, kv_heads=2, dim=16, vdim=12, size=7, scale=0.3, rheads=3, rdim=8, rvdim=20, ls=0.7, rs=0.4, mlp=MOE):
    left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size:
        left["mask"] = {"size": size}
    return {"type": "parallel", "mixer": {"left": left, "right": {"heads": rheads, "dim": rdim, "vdim": rvdim}, "left_scale": ls, "right_scale": rs}, "mlp": mlp}


def mamba(heads=4, vdim=12, state=16, groups=2, conv=4, norm_groups=3, mlp=MOE):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}, "mlp": mlp}


def config(layers, width=48, vocab=97, eps=1e-5, scale=2.0, streams=3, max_positions=256):
    return {"architecture": "Zazilix", "embedding": {"scale": scale}, "layers": layers, "norm": {"eps": eps}, "vocab": vocab, "width": width, "streams": streams,
            "max_positions": max_positions}


def weights(cfg, seed=0):
    return zazilix.random_tensors(cfg, seed)


def as_f64(t):
    return {k: v.float().numpy().astype(np.float64) for k, v in t.items()}


def tokens(cfg, n, seed=1):
    return [int(x) for x in np.random.default_rng(seed).integers(0, cfg["vocab"], n)]


def clear_rows(cfg, t, toks, dtype):
    """Rows that routing coin tosses cannot reach.  In bfloat16 the router's input carries the rounding of everything before it, so a
    choice score within a few hundredths of the next one may fall either way; that row then differs by an expert, not by rounding,
    and with more layers above, so does what later rows remember of it.  float32 needs no such care: every row counts."""
    keep = np.ones(len(toks), bool)
    if dtype == "float32":
        return keep
    plain.MARGINS.clear()
    plain.forward(cfg, as_f64(t), toks)
    for m in plain.MARGINS:
        keep &= m > 0.03
    if len(cfg["layers"]) > 1 and plain.MARGINS:
        keep = np.cumprod(keep).astype(bool)
    assert keep.sum() >= min(5, len(toks)), "too few rows with clear routing: choose another seed or a feed-forward without choices"
    return keep


def free_of_choices(dtype, **kw):
    """The feed-forward of tests that run in both modes with several layers: in bfloat16 every expert is taken (nothing to toss)."""
    ml = moe(**kw)
    if dtype != "float32":
        ml["router"]["top"] = ml["router"]["experts"] + ml["router"]["identity"]
    return ml


def rel_err_rows(got, ref, dtype="float32"):
    """Error of the worst row, relative to the spread of the reference logits.  In bfloat16 a few rows sit far above the others without
    any fault: a norm over a handful of values that happen to be small multiplies the rounding of what came before.  There the measure
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
    rel_err = lambda got, want: rel_err_rows(got[clear], want[clear], dtype)  # noqa: E731
    with zazilix.from_tensors(cfg, t, dtype, max_tokens=4 * len(toks) + 64, max_seqs=4, page=page) as m:
        assert rel_err(whole(m, toks), ref) < TOL[dtype]
        for first in {1, max(1, len(toks) // 2)}:
            s = m.open()
            rows = [m.step([s], [toks[:first]], list(range(first)))]
            for p in range(first, len(toks)):
                rows.append(m.step([s], [[toks[p]]], [0]))
            m.close_seq(s)
            assert rel_err(np.concatenate(rows), ref) < TOL[dtype]
        for size in portions:
            s, rows, at = m.open(), [], 0
            while at < len(toks):
                part = toks[at:at + size]
                rows.append(m.step([s], [part], list(range(len(part)))))
                at += len(part)
                size = size + 1 if size > 2 else size  # growing portions: edges fall at ever different places
            m.close_seq(s)
            assert rel_err(np.concatenate(rows), ref) < TOL[dtype]
    return ref


LAYERS = {
    "mlstm": mlstm(),
    "mlstm-noff": mlstm(mlp=None),
    "mlstm-one-head-tight-cap": mlstm(heads=1, dim=32, vdim=8, cap=1.5),
    "pair": pair(),
    "pair-noff": pair(mlp=None),
    "pair-mha-unbounded": pair(heads=3, kv_heads=3, dim=8, vdim=8, size=0),
    "pair-block-of-one": pair(heads=2, kv_heads=1, size=1, rheads=1),
    "pair-block-longer-than-prompt": pair(size=64, ls=1.0, rs=1.0),
    "mamba2": mamba(),
    "mamba2-noff": mamba(mlp=None),
    "mamba2-one-group-one-tap": mamba(heads=3, groups=1, conv=1, norm_groups=1),
    "mamba2-group-per-head": mamba(heads=2, vdim=16, state=8, groups=2, conv=2, norm_groups=2),
    "moe-no-identity-top1": mlstm(mlp=moe(experts=4, identity=0, top=1)),
    "moe-top-all-no-shared": mamba(mlp=moe(experts=3, identity=1, top=4, shared=0)),
    "moe-mostly-identity": pair(mlp=moe(experts=1, identity=4, top=2, scale=1.0)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(LAYERS))
def test_each_mechanism_alone(name, dtype):
    cfg = config([LAYERS[name]])
    check_all_ways(cfg, weights(cfg, 3), tokens(cfg, 37), dtype)


@pytest.mark.parametrize("streams", [1, 2, 5])
def test_stream_counts(streams):
    cfg = config([mlstm(), pair(mlp=None), mamba()], streams=streams)
    check_all_ways(cfg, weights(cfg, 4), tokens(cfg, 21), portions=(4,))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_sizes_that_align_with_nothing(dtype):
    """Width, head sizes, state sizes, expert widths and vocabulary that are multiples of neither 8 nor 4."""
    cfg = config([mlstm(heads=3, dim=10, vdim=7, mlp=free_of_choices(dtype, experts=3, identity=1, top=2, ff=9, shared=11)),
                  pair(heads=3, kv_heads=3, dim=10, vdim=6, size=5, rheads=1, rdim=7, rvdim=5, mlp=None),
                  mamba(heads=3, vdim=5, state=6, groups=1, conv=3, norm_groups=5, mlp=free_of_choices(dtype, experts=2, identity=0, top=1, ff=3, shared=0)),
                  pair(heads=6, kv_heads=2, dim=6, vdim=10, size=9, rheads=2, rdim=10, rvdim=6, mlp=free_of_choices(dtype))], width=50, vocab=61, scale=1.0, streams=2)
    check_all_ways(cfg, weights(cfg, 31), tokens(cfg, 45), dtype, portions=(17, 2))


def test_other_layer_orders():
    for k, order in enumerate(([mamba(), mamba(mlp=None), pair(), mlstm()], [pair(mlp=None), mlstm(), mlstm(mlp=None), pair(size=4), mamba()])):
        cfg = config(order, width=40, streams=2 + k)
        check_all_ways(cfg, weights(cfg, 5 + k), tokens(cfg, 41), portions=(6,))


def test_residual_stream_after_every_layer():
    cfg = config([mlstm(), pair(), mamba(), mlstm(mlp=None)])
    t, toks = weights(cfg, 8), tokens(cfg, 19)
    trace = []
    plain.forward(cfg, as_f64(t), toks, trace)
    with zazilix.from_tensors(cfg, t, "float32", max_tokens=64, max_seqs=2) as m:
        m.set_trace(True)
        whole(m, toks)
        got = m.read_trace(len(toks))
    assert got.shape[0] == len(trace) == 4
    for g, r in zip(got, trace):
        assert np.abs(g - r).max() < 1e-4 * max(1.0, np.abs(r).max())


def test_block_edges_sink_penalty_and_value_norm_show(monkeypatch):
    """Sharp scores: a block size that is one position off moves the logits far more than the tolerance, in prompts, portions and
    decoding alike (the same check passes for the right value); so do the one in the denominator, the distance penalty and the norm
    of the values when the plain statement leaves them out."""
    cfg = config([pair(size=6, scale=1.5, ls=1.0, rs=0.2, mlp=None)])
    t, toks = weights(cfg, 11), tokens(cfg, 60)
    ref = check_all_ways(cfg, t, toks, portions=(7, 2))
    for off in (-1, 1):
        wrong = copy.deepcopy(cfg)
        wrong["layers"][0]["mixer"]["left"]["mask"]["size"] += off
        assert rel_err(plain.forward(wrong, as_f64(t), toks), ref) > 100 * TOL["float32"]
    for knob in ("sink", "penalty", "value_norm"):
        monkeypatch.setitem(plain.KNOBS, knob, False)
        assert rel_err(plain.forward(cfg, as_f64(t), toks), ref) > 100 * TOL["float32"]
        monkeypatch.setitem(plain.KNOBS, knob, True)


def test_the_first_tokens_of_the_matrix_memory():
    """The running maximum of the log gates starts at zero: with input gates far below zero the first tokens' maximum comes from
    that start, and their outputs are divided by exp(-m) > 1 rather than by their own small normaliser."""
    cfg = config([mlstm(heads=2, dim=8, vdim=8, cap=10.0, mlp=None)], streams=1)
    t = weights(cfg, 12)
    t["l0.mix.i.b"] = torch.full_like(t["l0.mix.i.b"], -6.0)
    check_all_ways(cfg, t, tokens(cfg, 24), portions=(3,))
    t["l0.mix.i.b"] = torch.full_like(t["l0.mix.i.b"], 9.0)  # and far above zero: the maximum follows the input gates at once
    check_all_ways(cfg, t, tokens(cfg, 24), portions=(3,))


def test_router_details_show():
    """The correction moves choices but not weights, the scale is applied, identity experts return their input, weights are not renormalised."""
    cfg = config([mlstm(mlp=moe(experts=3, identity=3, top=2, scale=1.7))])
    t, toks = weights(cfg, 13), tokens(cfg, 40)
    t["l0.mlp.correction"] = (0.3 * torch.randn(6, generator=torch.Generator().manual_seed(5))).to(torch.bfloat16)
    ref = check_all_ways(cfg, t, toks, portions=(9,))
    p = as_f64(t)
    h = np.random.default_rng(0).normal(size=(200, cfg["width"]))
    chosen, wt = plain.route(h, p, "l0.mlp.", cfg["layers"][0]["mlp"])
    assert (chosen >= 3).any() and (chosen < 3).any() and not np.allclose(wt.sum(-1), 1.7)
    no_corr = dict(p, **{"l0.mlp.correction": np.zeros(6)})
    assert (plain.route(h, no_corr, "l0.mlp.", cfg["layers"][0]["mlp"])[0] != chosen).any()
    assert rel_err(plain.forward(cfg, no_corr, toks), ref) > 100 * TOL["float32"]
    for key, val in (("scale", 1.0), ("identity", 2)):
        wrong = copy.deepcopy(cfg)
        wrong["layers"][0]["mlp"]["router"][key] = val
        pw = dict(p)
        if key == "identity":  # one identity expert fewer: the router loses its last row
            pw["l0.mlp.router"], pw["l0.mlp.correction"] = p["l0.mlp.router"][:5], p["l0.mlp.correction"][:5]
        assert rel_err(plain.forward(wrong, pw, toks), ref) > 100 * TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_context_with_shared_out_keys(dtype):
    """Decoding few tokens over a context of several hundred with no block bound: the attention kernel shares one query's keys out over
    several CTAs and folds the shares (the one in the denominator counted once, the distance penalty per key); keys hundreds of
    positions back, over many page borders, still reach the last heads, whose penalty is small.  The recurrent states carry 128 key channels."""
    cfg = config([pair(heads=4, kv_heads=2, size=0, scale=1.0 if dtype == "float32" else 0.3, rheads=1, rdim=128, rvdim=16, mlp=None),
                  pair(size=200, scale=0.3, mlp=None), mlstm(heads=1, dim=128, vdim=16, mlp=None)], max_positions=400)
    t, toks = weights(cfg, 15), tokens(cfg, 330)
    ref = plain.forward(cfg, as_f64(t), toks)
    with zazilix.from_tensors(cfg, t, dtype, max_tokens=700, max_seqs=2, page=16) as m:
        s = m.open()
        rows = [m.step([s], [toks[:300]], list(range(300)))]
        for p in range(300, 330):
            rows.append(m.step([s], [[toks[p]]], [0]))
        assert rel_err(np.concatenate(rows), ref, dtype) < TOL[dtype]
        s2 = m.open()  # the same prompt in two-token portions beside the finished sequence
        rows = [m.step([s2], [toks[a:a + 2]], [0, 1]) for a in range(0, 330, 2)]
        assert rel_err(np.concatenate(rows), ref, dtype) < TOL[dtype]


def test_a_far_key_stands_out():
    """One early position gets a key that the last queries match: scaled so that its score beats every penalty, it must dominate the
    softmax hundreds of positions later, through prompts and decoding; a block bound puts it out of sight."""
    cfg = config([pair(heads=2, kv_heads=1, dim=32, vdim=8, size=0, scale=1.0, ls=1.0, rs=0.1, mlp=None)], streams=1, max_positions=512)
    t, toks = weights(cfg, 16), tokens(cfg, 420)
    # queries and keys from the same projection, no norm weights: a query finds the positions that hold its own token
    t["l0.mix.left.q"] = torch.cat([t["l0.mix.left.k"], t["l0.mix.left.k"]], 0)
    t["l0.mix.left.q.norm"], t["l0.mix.left.k.norm"] = torch.ones(64, dtype=torch.bfloat16), torch.ones(32, dtype=torch.bfloat16)
    toks[5] = toks[-1] = toks[-7] = 3  # the same token: the same key direction as the queries that look for it
    for x in range(len(toks)):
        if x not in (5, len(toks) - 1, len(toks) - 7) and toks[x] == 3:
            toks[x] = 4
    ref = plain.forward(cfg, as_f64(t), toks)
    bounded = copy.deepcopy(cfg)
    bounded["layers"][0]["mixer"]["left"]["mask"] = {"size": 128}
    assert rel_err(plain.forward(bounded, as_f64(t), toks)[-8:], ref[-8:]) > 100 * TOL["float32"]
    with zazilix.from_tensors(cfg, t, "float32", max_tokens=1024, max_seqs=2, page=16) as m:
        assert rel_err(whole(m, toks), ref) < TOL["float32"]
        s = m.open()
        rows = [m.step([s], [toks[:400]], list(range(400)))] + [m.step([s], [[x]], [0]) for x in toks[400:]]
        assert rel_err(np.concatenate(rows), ref) < TOL["float32"]


def test_prompt_attention_as_products_matches_the_fused_kernel(monkeypatch):
    """bfloat16 mode computes a long portion's attention as tensor-core products over gathered keys, short portions with the fused
    kernel.  Both sit within bf16 rounding of the plain statement, also for a portion that continues a cached prefix in the middle
    of a block of positions; a block size that is one off shows far above that."""
    for size in (23, 4, 0):
        ml = free_of_choices("bfloat16")
        cfg = config([pair(size=size, scale=0.8, ls=1.0, rs=0.3, mlp=ml), pair(size=0, heads=4, kv_heads=4, dim=8, vdim=8, mlp=ml)])
        t, toks = weights(cfg, 17), tokens(cfg, 120)
        ref = plain.forward(cfg, as_f64(t), toks)
        errs = {}
        for products in ("1", "0"):
            monkeypatch.setenv("CALM_B200_SEQ_ATTN_PRODUCTS", products)
            with zazilix.from_tensors(cfg, t, "bfloat16", max_tokens=300, max_seqs=3, page=8) as m:
                s1, s2 = m.open(), m.open()
                a = m.step([s1], [toks[:50]], list(range(50)))
                b = m.step([s1, s2], [toks[50:], toks[:3]], list(range(73)))  # 70 more tokens on the products path beside a 3-token portion
                errs[products] = rel_err(np.concatenate([a, b[:70]]), ref, "bfloat16")
                assert rel_err(b[70:], ref[:3], "bfloat16") < TOL["bfloat16"]
        assert errs["1"] < TOL["bfloat16"] and errs["0"] < TOL["bfloat16"] and errs["1"] < 3 * errs["0"] + 1e-3
        if size:
            for off in (-1, 1):
                wrong = copy.deepcopy(cfg)
                wrong["layers"][0]["mixer"]["left"]["mask"]["size"] += off
                assert rel_err(plain.forward(wrong, as_f64(t), toks), ref) > 4 * errs["1"]


def test_tensor_core_products_match_the_warp_level_ones(monkeypatch):
    """bfloat16 mode runs products over many tokens on tcgen05 (grouped ones for the experts included) and everything else on
    mma.sync; same bf16 inputs, fp32 sums in another order."""
    cfg = config([mlstm(heads=2, dim=32, vdim=24, mlp=moe(experts=5, identity=1, top=6, ff=40, shared=56)), pair(heads=4, kv_heads=2, dim=32, vdim=24, size=50, rdim=32, rvdim=40, mlp=None),
                  mamba(heads=4, vdim=24, state=32, mlp=moe(experts=3, identity=0, top=3, ff=72, shared=0))], width=88, vocab=131, max_positions=320)
    t, toks = weights(cfg, 18), tokens(cfg, 300)
    outs = {}
    for tc in ("1", "0"):
        monkeypatch.setenv("CALM_B200_SEQ_TC", tc)
        with zazilix.from_tensors(cfg, t, "bfloat16", max_tokens=640, max_seqs=2, page=16) as m:
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
    """130 tokens one by one: every recurrent state, the convolution's last inputs, the running maximum and the cache grow by single steps
    (and a forget gate near one keeps the first tokens in the state to the end)."""
    cfg = config([mlstm(), pair(size=12), mamba(), mlstm(mlp=None)])
    t, toks = weights(cfg, 14), tokens(cfg, 130)
    for name in t:
        if name.endswith("mix.f.b"):
            t[name] = torch.full_like(t[name], 5.0)
    ref = plain.forward(cfg, as_f64(t), toks)
    with zazilix.from_tensors(cfg, t, "float32", max_tokens=200, max_seqs=2, page=8) as m:
        s = m.open()
        rows = [m.step([s], [[x]], [0]) for x in toks]
        assert rel_err(np.concatenate(rows), ref) < TOL["float32"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_unequal_batch_equals_each_alone(dtype):
    ml = free_of_choices(dtype)
    cfg = config([mlstm(mlp=ml), pair(mlp=ml), mamba(mlp=ml), pair(size=4, mlp=None)])
    t = weights(cfg, 21)
    prompts = [tokens(cfg, n, seed=n) for n in (1, 9, 40, 2)]
    tails = [tokens(cfg, n, seed=50 + n) for n in (6, 3, 0, 6)]
    p = as_f64(t)
    refs = [plain.forward(cfg, p, a + b) for a, b in zip(prompts, tails)]
    with zazilix.from_tensors(cfg, t, dtype, max_tokens=192, max_seqs=5, page=4) as m:
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
    """A slot that is opened again starts from zero state (matrix memory, normaliser, running maximum, convolution inputs) and fresh pages."""
    cfg = config([mlstm(), pair(), mamba()])
    t = weights(cfg, 22)
    p = as_f64(t)
    with zazilix.from_tensors(cfg, t, "float32", max_tokens=48, max_seqs=2, page=4) as m:
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


def test_no_sequence_outgrows_the_position_table():
    cfg = config([mlstm(mlp=None)], max_positions=12)
    t = weights(cfg, 24)
    with zazilix.from_tensors(cfg, t, "float32", max_tokens=64, max_seqs=2) as m:
        s = m.open()
        m.step([s], [tokens(cfg, 11)], [10])
        m.step([s], [[1]], [0])
        with pytest.raises(Exception):
            m.step([s], [[1]], [0])
        assert m.length(s) == 12
        sched = serving.Scheduler(m)
        sched.add(serving.Request("fits", tokens(cfg, 4), 9))  # positions 0 .. 11: the ninth new token is not fed back
        with pytest.raises(ValueError):
            sched.add(serving.Request("long", tokens(cfg, 4), 10))


def test_greedy_generation_through_the_scheduler():
    cfg = config([mlstm(), pair(), mamba(mlp=None)])
    t = weights(cfg, 23)
    p = as_f64(t)
    prompts = [tokens(cfg, n, seed=70 + n) for n in (5, 17, 1)]
    with zazilix.from_tensors(cfg, t, "float32", max_tokens=256, max_seqs=2, page=8) as m:
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
    cfg = config([mamba(heads=2, vdim=16, state=32, groups=1, norm_groups=4, mlp=ml), pair(heads=4, kv_heads=1, dim=16, vdim=8, size=11, scale=0.5, mlp=ml), mlstm(heads=2, dim=8, vdim=8, mlp=None),
                  pair(heads=2, kv_heads=2, dim=8, vdim=8, size=3, rheads=1, rdim=8, rvdim=40, mlp=ml)], width=72, vocab=211, eps=1e-6, scale=3.0, streams=2, max_positions=64)
    t = weights(cfg, 41)
    folder, out = tmp_path / "model", tmp_path / "out"
    folder.mkdir(), out.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    container.write_tensors(str(folder / "model.safetensors"), t)
    assert registry.architecture_of(str(folder)) == "Zazilix"
    reqs = {"a": tokens(cfg, 46, 1), "b": tokens(cfg, 9, 2), "c": tokens(cfg, 4, 3), "d": tokens(cfg, 30, 4), "e": tokens(cfg, 2, 5)}
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
