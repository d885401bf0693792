"""Sopepel: a decoder whose config.json lists its layers.  A sublayer reads the residual stream itself and its output comes back
through an RMS norm, x <- x + norm1(mixer(x)), x <- x + norm2(feed-forward(x)).  The embedding adds a row of a second table
picked by a hash of the previous and the current token.  Every mixer is a pair on the same input: grouped-query attention
(biased projections, RMS norm per head on queries and keys with one weight vector for all heads, partial rotation, softmax
inside blocks of positions counted from the sequence's start, one sigmoid gate per head, biased output projection) beside gated
linear attention (a decaying [dim x vdim] state per head), each with its factor.  Feed-forward: down(gelu(gate) * up), or routed
experts of the form down(relu(up)^2) whose sigmoid scores weight the expert's INPUT, with a shared unit of the same form behind a
sigmoid gate per token.  The logits come from the embedding table and are scaled.

This module is the host side, like vimulorn.py, bovinex.py and zazilix.py: it reads config.json, checks every tensor's shape,
stacks what reads the same input into one matrix and binds everything in the records of seqlib.  Kernels, cache and state live
in libcalm_b200_seq.so; every size and constant comes from the config or a tensor's shape."""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Tuple

import torch

from . import container, seqlib

ARCHITECTURE = "Sopepel"


def plan(cfg: dict, tensors: Dict[str, torch.Tensor]) -> Tuple[dict, List[dict], Dict[str, torch.Tensor]]:
    """config + checkpoint tensors -> (model head, layer records, tensors to upload)."""
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config")
    width, vocab = int(cfg["width"]), int(cfg["vocab"])
    up: Dict[str, torch.Tensor] = {}

    def need(name: str, shape) -> str:
        if name not in tensors:
            raise KeyError(f"checkpoint lacks tensor {name}")
        t = tensors[name]
        if list(t.shape) != list(shape):
            raise ValueError(f"tensor {name} has shape {list(t.shape)}, the config asks for {list(shape)}")
        up[name] = t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)
        return name

    def stack(name: str, parts: List[str]) -> str:
        up[name] = torch.cat([up.pop(p) for p in parts], 0).contiguous()
        return name

    def attention(m: str, mx: dict) -> dict:
        H, D, Dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
        G = int(mx.get("kv_heads", H))
        rot, mask = mx.get("rot") or {}, mx.get("mask") or {}
        rec = {"type": seqlib.SEQ_GQA, "heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "taps": 1, "scale": float(mx["scale"]), "window": 0,
               "chunk": int(mask.get("size", 0)), "rot_dims": int(rot.get("dims", 0)), "rot_base": float(rot.get("base", 10000.0)),
               "qk_per_head": 1, "gate_per_head": 1, "scores_f32": 1}
        rows = [("q", H * D), ("k", G * D), ("v", G * Dv)]
        rec["w_in"] = stack(m + "in", [need(m + n, [r, width]) for n, r in rows] + [need(m + "g", [H, width])])
        up[m + "in.b"] = torch.cat([up.pop(need(m + n + ".b", [r])) for n, r in rows] + [torch.zeros(H, dtype=torch.bfloat16)], 0)  # the gate has no bias
        rec["b_in"] = m + "in.b"
        rec["q_norm"], rec["k_norm"] = need(m + "q.norm", [D]), need(m + "k.norm", [D])
        rec["w_o"], rec["b_o"] = need(m + "o", [width, H * Dv]), need(m + "o.b", [width])
        return rec

    def linear(m: str, mx: dict) -> dict:
        H, D, Dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
        if (m + "a1") not in tensors:
            raise KeyError(f"checkpoint lacks tensor {m}a1")
        ra = int(tensors[m + "a1"].shape[0])  # the decay's inner width is the tensor's
        rec = {"type": seqlib.SEQ_GLA, "heads": H, "kv_heads": H, "dim": D, "vdim": Dv, "taps": 1, "a_rank": ra, "tau": float(mx["tau"])}
        rec["w_in"] = stack(m + "in", [need(m + "q", [H * D, width]), need(m + "k", [H * D, width]), need(m + "v", [H * Dv, width]), need(m + "g", [H * Dv, width]),
                                       need(m + "a1", [ra, width])])
        rec["w_a2"], rec["b_a2"], rec["out_norm"] = need(m + "a2", [H * D, ra]), need(m + "a2.b", [H * D]), need(m + "norm", [Dv])
        rec["w_o"] = need(m + "o", [width, H * Dv])
        return rec

    layers = []
    for i, lc in enumerate(cfg["layers"]):
        p, mx, kind = f"l{i}.", lc["mixer"], lc["type"]
        if kind != "parallel":
            raise ValueError(f"layer {i}: unknown mixer {kind}")
        m = p + "mix."
        left, right = attention(m + "left.", mx["left"]), linear(m + "right.", mx["right"])
        # both mixers read the same input: their input rows are one matrix (the left's, zero rows up to a multiple of 8, the right's) and one product
        lw, lb, rw = up.pop(left.pop("w_in")), up.pop(left.pop("b_in")), up.pop(right.pop("w_in"))
        pad = -lw.shape[0] % 8
        up[m + "in"] = torch.cat([lw, torch.zeros(pad, width, dtype=torch.bfloat16), rw], 0).contiguous()
        up[m + "in.b"] = torch.cat([lb, torch.zeros(pad + rw.shape[0], dtype=torch.bfloat16)], 0)
        rec = {"type": seqlib.SEQ_PAIR, "pair": [left, right], "pair_scale": [float(mx.get("left_scale", 1.0)), float(mx.get("right_scale", 1.0))], "w_in": m + "in", "b_in": m + "in.b",
               "norm1": need(p + "norm1", [width])}
        ml = lc.get("mlp")
        if ml:
            f = p + "mlp."
            rec["norm2"] = need(p + "norm2", [width])
            if ml["kind"] == "dense":
                ff = int(ml["ff"])
                rec.update(ff=ff, ff_kind=seqlib.FF_GATED, ff_act=seqlib.ACT_GELU_TANH, w_down=need(f + "down", [width, ff]))
                rec["w_gate_up"] = stack(f + "gate_up", [need(f + "gate", [ff, width]), need(f + "up", [ff, width])])
            elif ml["kind"] == "moe":
                ff, E, top = int(ml["expert"]["ff"]), int(ml["router"]["experts"]), int(ml["router"]["top"])
                rec.update(ff=ff, ff_kind=seqlib.FF_MOE, experts=E, top=top, route_mode=2, route_scale=1.0, expert_act=1, weight_input=1)
                # experts side by side: [experts][up] and [experts][down], so that one grouped product serves all of them
                rec["w_gate_up"] = stack(f + "ups", [need(f + f"e{e}.up", [ff, width]) for e in range(E)])
                rec["w_down"] = stack(f + "downs", [need(f + f"e{e}.down", [width, ff]) for e in range(E)])
                sh = ml.get("shared")
                if sh:
                    # everything that reads the feed-forward's input first is one product: the shared unit's gate row, the router's rows, then
                    # the shared unit's up rows (which leave the product's epilogue as relu(.)^2)
                    sf = int(sh["ff"])
                    rec.update(shared_ff=sf, shared_gate=1)
                    rec["w_sh_gate_up"] = stack(f + "shared.in", [need(f + "shared.sg", [1, width]), need(f + "router", [E, width]), need(f + "shared.up", [sf, width])])
                    rec["w_sh_down"] = need(f + "shared.down", [width, sf])
                else:
                    rec["w_router"] = need(f + "router", [E, width])
            else:
                raise ValueError(f"layer {i}: feed-forward kind {ml['kind']} is not part of this design")
        layers.append(rec)
    bg = (cfg.get("embedding") or {}).get("bigram")
    head = {"vocab": vocab, "width": width, "eps": float(cfg["norm"]["eps"]), "embed": need("embed", [vocab, width]), "head": "embed",
            "final_norm": need("final.norm", [width]), "norm_kind": seqlib.NORM_RMS, "norm_offset": 0.0, "block": seqlib.BLOCK_POST,
            "logit_scale": float(cfg.get("logit_scale", 1.0))}
    if bg:
        B = int(bg["buckets"])
        head.update(bigram=need("bigram", [B + 1, width]), bigram_buckets=B, bigram_mul_prev=int(bg["mul_prev"]), bigram_mul_cur=int(bg["mul_cur"]))
    return head, layers, up


def load(folder: str, dtype: str = "bfloat16", max_tokens: int = 4096, max_seqs: int = 64, page: int = 16) -> seqlib.SeqDeviceModel:
    """config.json + model.safetensors of `folder` onto the GPU."""
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    tensors, _ = container.read_tensors(os.path.join(folder, "model.safetensors"))
    return from_tensors(cfg, tensors, dtype, max_tokens, max_seqs, page)


def from_tensors(cfg: dict, tensors: Dict[str, torch.Tensor], dtype: str = "bfloat16", max_tokens: int = 4096, max_seqs: int = 64, page: int = 16):
    if dtype not in ("bfloat16", "float32"):
        raise ValueError("dtype must be bfloat16 or float32")
    head, layers, up = plan(cfg, tensors)
    return seqlib.SeqDeviceModel(head, layers, up, exact=dtype == "float32", max_tokens=max_tokens, max_seqs=max_seqs, page=page)


# ---------------------------------------------------------------- synthetic checkpoints (tests, bench)

def tensor_shapes(cfg: dict, a_rank: int = 16) -> Dict[str, list]:
    W, out = int(cfg["width"]), {}
    out["embed"] = [cfg["vocab"], W]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        out["bigram"] = [bg["buckets"] + 1, W]
    for i, lc in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", lc["mixer"]
        out[p + "norm1"] = [W]
        lm, rm = mx["left"], mx["right"]
        m = p + "mix.left."
        H, G, D, Dv = lm["heads"], lm.get("kv_heads", lm["heads"]), lm["dim"], lm["vdim"]
        out.update({m + "q": [H * D, W], m + "q.b": [H * D], m + "k": [G * D, W], m + "k.b": [G * D], m + "v": [G * Dv, W], m + "v.b": [G * Dv],
                    m + "q.norm": [D], m + "k.norm": [D], m + "g": [H, W], m + "o": [W, H * Dv], m + "o.b": [W]})
        m = p + "mix.right."
        H, D, Dv, ra = rm["heads"], rm["dim"], rm["vdim"], rm.get("a_rank", a_rank)
        out.update({m + "q": [H * D, W], m + "k": [H * D, W], m + "v": [H * Dv, W], m + "g": [H * Dv, W], m + "o": [W, H * Dv], m + "norm": [Dv],
                    m + "a1": [ra, W], m + "a2": [H * D, ra], m + "a2.b": [H * D]})
        ml = lc.get("mlp")
        if ml:
            f = p + "mlp."
            out[p + "norm2"] = [W]
            if ml["kind"] == "dense":
                out.update({f + "gate": [ml["ff"], W], f + "up": [ml["ff"], W], f + "down": [W, ml["ff"]]})
            else:
                ff = ml["expert"]["ff"]
                for e in range(ml["router"]["experts"]):
                    out.update({f + f"e{e}.up": [ff, W], f + f"e{e}.down": [W, ff]})
                out[f + "router"] = [ml["router"]["experts"], W]
                if ml.get("shared"):
                    sf = ml["shared"]["ff"]
                    out.update({f + "shared.up": [sf, W], f + "shared.down": [W, sf], f + "shared.sg": [1, W]})
    out["final.norm"] = [W]
    return out


def random_tensors(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Seeded bf16 weights with magnitudes that keep every mechanism active (decays away from 0 and 1, gates open, router choices
    spread over the experts, sublayer outputs of a size that the norms do not hide)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm", "norm1", "norm2"):
            t = (0.5 if leaf in ("norm1", "norm2") else 1.0) * (1.0 + 0.2 * torch.randn(shape, generator=g))
        elif name.endswith("a2.b"):
            t = 1.5 + 1.5 * torch.randn(shape, generator=g)
        elif leaf == "b":
            t = 0.3 * torch.randn(shape, generator=g)
        elif leaf in ("embed", "bigram"):
            t = torch.randn(shape, generator=g) * (0.7 if leaf == "embed" else 0.5)
        elif leaf in ("router", "sg"):
            t = torch.randn(shape, generator=g) * (2.0 / math.sqrt(shape[-1]))
        else:
            t = torch.randn(shape, generator=g) * (1.2 / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16)
    return out
