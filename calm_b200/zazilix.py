"""Zazilix: a decoder whose config.json lists its layers.  The residual is `streams` copies (hyper-connections: every sublayer reads a
weighted sum of the copies and writes all of them from the old ones and its output), norms are RMS norms whose weight is one number,
positions are learned rows added to the scaled embedding.  Mixers: mLSTM (matrix memory with exponential gating), a pair of mixers
side by side (grouped-query attention inside blocks of positions with a distance penalty per head, normed values and one added to the
softmax denominator; next to HGRN2, linear attention whose bounded forget gate also writes), and Mamba-2.  Feed-forward: routed
SiLU-gated experts chosen on softmax score + correction, identity experts, and a shared unit.

This module is the host side, like vimulorn.py and bovinex.py: it reads config.json, checks every tensor's shape, stacks what reads
the same input into one matrix and binds everything in the records of seqlib.  Kernels, cache and state live in
libcalm_b200_seq.so; every size and constant comes from the config or a tensor's shape."""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Tuple

import torch

from . import container, seqlib

ARCHITECTURE = "Zazilix"


def plan(cfg: dict, tensors: Dict[str, torch.Tensor]) -> Tuple[dict, List[dict], Dict[str, torch.Tensor]]:
    """config + checkpoint tensors -> (model head, layer records, tensors to upload)."""
    if cfg.get("architecture") != ARCHITECTURE:
        raise ValueError(f"not a {ARCHITECTURE} config")
    width, vocab, streams = int(cfg["width"]), int(cfg["vocab"]), int(cfg.get("streams", 1))
    up: Dict[str, torch.Tensor] = {}

    def need(name: str, shape) -> str:
        if name not in tensors:
            raise KeyError(f"checkpoint lacks tensor {name}")
        t = tensors[name]
        if list(t.shape) != list(shape):
            raise ValueError(f"tensor {name} has shape {list(t.shape)}, the config asks for {list(shape)}")
        t = t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)
        up[name] = t if shape else t.reshape(1)  # a single number travels as a vector of one
        return name

    def stack(name: str, parts: List[str]) -> str:
        up[name] = torch.cat([up.pop(p) for p in parts], 0).contiguous()
        return name

    def bias(name: str, rows: List[Tuple[str, int]]) -> str:
        """bias of a stacked projection: the named vectors where the checkpoint has them, zeros elsewhere"""
        up[name] = torch.cat([up.pop(need(n, [r])) if n else torch.zeros(r, dtype=torch.bfloat16) for n, r in rows], 0)
        return name

    def mlstm(m: str, mx: dict) -> dict:
        H, D, Dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
        rec = {"type": seqlib.SEQ_MLSTM, "heads": H, "kv_heads": H, "dim": D, "vdim": Dv, "taps": 1, "gate_cap": float(mx["gate_cap"])}
        rec["w_in"] = stack(m + "in", [need(m + "q", [H * D, width]), need(m + "k", [H * D, width]), need(m + "v", [H * Dv, width]), need(m + "g", [H * Dv, width]),
                                       need(m + "i", [H, width]), need(m + "f", [H, width])])
        rec["b_in"] = bias(m + "in.b", [("", 2 * H * D + 2 * H * Dv), (m + "i.b", H), (m + "f.b", H)])
        rec["out_norm"], rec["w_o"] = need(m + "norm", [H * Dv]), need(m + "o", [width, H * Dv])
        return rec

    def attention(m: str, mx: dict) -> dict:
        H, D, Dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
        G = int(mx.get("kv_heads", H))
        rec = {"type": seqlib.SEQ_GQA, "heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "taps": 1, "scale": float(mx["scale"]), "window": 0,
               "chunk": int((mx.get("mask") or {}).get("size", 0)), "dist_bias": 1, "add_one": 1, "v_norm": 1, "no_gate": 1}
        rec["w_in"] = stack(m + "in", [need(m + "q", [H * D, width]), need(m + "k", [G * D, width]), need(m + "v", [G * Dv, width])])
        rec["q_norm"], rec["k_norm"], rec["w_o"] = need(m + "q.norm", [H * D]), need(m + "k.norm", [G * D]), need(m + "o", [width, H * Dv])
        return rec

    def hgrn2(m: str, mx: dict) -> dict:
        H, D, Dv = int(mx["heads"]), int(mx["dim"]), int(mx["vdim"])
        rec = {"type": seqlib.SEQ_HGRN2, "heads": H, "kv_heads": H, "dim": D, "vdim": Dv, "taps": 1}
        rec["w_in"] = stack(m + "in", [need(m + "q", [H * D, width]), need(m + "f", [H * D, width]), need(m + "v", [H * Dv, width])])
        rec["b_in"] = bias(m + "in.b", [("", H * D), (m + "f.b", H * D), ("", H * Dv)])
        rec["lower"], rec["out_norm"], rec["w_o"] = need(m + "lower", [H * D]), need(m + "norm", [Dv]), need(m + "o", [width, H * Dv])
        return rec

    def mamba2(m: str, mx: dict) -> dict:
        H, Dv, Ns, G, taps = int(mx["heads"]), int(mx["vdim"]), int(mx["state"]), int(mx["groups"]), int(mx["conv"])
        inner, ch = H * Dv, H * Dv + 2 * G * Ns
        rec = {"type": seqlib.SEQ_MAMBA2, "heads": H, "kv_heads": G, "dim": Ns, "vdim": Dv, "taps": taps, "norm_groups": int(mx.get("norm_groups", 1))}
        rec["w_in"] = need(m + "in", [2 * inner + 2 * G * Ns + H, width])
        rec["conv"], rec["conv_b"] = need(m + "conv", [ch, taps]), need(m + "conv.b", [ch])
        rec["dt_bias"], rec["a_log"], rec["skip_d"] = need(m + "dt_bias", [H]), need(m + "A_log", [H]), need(m + "D", [H])
        rec["out_norm"], rec["w_o"] = need(m + "norm", [inner]), need(m + "o", [width, inner])
        return rec

    layers = []
    for i, lc in enumerate(cfg["layers"]):
        p, mx, kind = f"l{i}.", lc["mixer"], lc["type"]
        m = p + "mix."
        if kind == "mlstm":
            rec = mlstm(m, mx)
        elif kind == "mamba2":
            rec = mamba2(m, mx)
        elif kind == "parallel":
            rec = {"type": seqlib.SEQ_PAIR, "pair": [attention(m + "left.", mx["left"]), hgrn2(m + "right.", mx["right"])],
                   "pair_scale": [float(mx.get("left_scale", 1.0)), float(mx.get("right_scale", 1.0))]}
        else:
            raise ValueError(f"layer {i}: unknown mixer {kind}")
        rec["norm1"] = need(p + "norm1", [])
        rec["hc1"] = [need(p + "hc1.in", [streams]), need(p + "hc1.out", [streams]), need(p + "hc1.mix", [streams, streams])]
        ml = lc.get("mlp")
        if ml:
            if ml.get("kind", "moe") != "moe":
                raise ValueError(f"layer {i}: feed-forward kind {ml['kind']} is not part of this design")
            f, r = p + "mlp.", ml["router"]
            ff, E, I, top = int(ml["expert"]["ff"]), int(r["experts"]), int(r.get("identity", 0)), int(r["top"])
            rec.update(ff=ff, ff_kind=seqlib.FF_MOE, experts=E, ident=I, top=top, route_mode=1, route_scale=float(r.get("scale", 1.0)))
            rec["norm2"] = need(p + "norm2", [])
            rec["hc2"] = [need(p + "hc2.in", [streams]), need(p + "hc2.out", [streams]), need(p + "hc2.mix", [streams, streams])]
            rec["w_router"] = need(f + "router", [E + I, width])
            if (f + "correction") in tensors:
                rec["correction"] = need(f + "correction", [E + I])
            # experts side by side: [experts][gate | up] and [experts][down], so that one grouped product serves all of them
            rec["w_gate_up"] = stack(f + "gate_up", [x for e in range(E) for x in (need(f + f"e{e}.gate", [ff, width]), need(f + f"e{e}.up", [ff, width]))])
            rec["w_down"] = stack(f + "downs", [need(f + f"e{e}.down", [width, ff]) for e in range(E)])
            sh = ml.get("shared")
            if sh:
                sf = int(sh["ff"])
                rec["shared_ff"] = sf
                # the shared unit's first rows and the router's read the same normed input: one product, the router's rows last
                rec["w_sh_gate_up"] = stack(f + "shared.in", [need(f + "shared.gate", [sf, width]), need(f + "shared.up", [sf, width]), rec.pop("w_router")])
                rec["w_sh_down"] = need(f + "shared.down", [width, sf])
        layers.append(rec)
    maxpos = int(cfg["max_positions"])
    head = {"vocab": vocab, "width": width, "eps": float(cfg["norm"]["eps"]), "embed": need("embed", [vocab, width]), "head": need("head", [vocab, width]),
            "final_norm": need("final.norm", []), "norm_kind": seqlib.NORM_RMS, "norm_offset": 0.0, "norm_scalar": 1, "block": seqlib.BLOCK_HYPER,
            "streams": streams, "embed_scale": float((cfg.get("embedding") or {}).get("scale", 1.0)), "pos_table": need("pos", [maxpos, width]), "max_positions": maxpos}
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

def tensor_shapes(cfg: dict) -> Dict[str, list]:
    W, S, out = int(cfg["width"]), int(cfg.get("streams", 1)), {}
    out["embed"], out["pos"] = [cfg["vocab"], W], [cfg["max_positions"], W]

    def lin(m, names, H, D, Dv):
        for n, rows in names:
            out[m + n] = [rows, W]
        out[m + "o"] = [W, H * Dv]

    for i, lc in enumerate(cfg["layers"]):
        p, mx = f"l{i}.", lc["mixer"]
        m = p + "mix."
        out[p + "norm1"] = []
        if lc["type"] == "mlstm":
            H, D, Dv = mx["heads"], mx["dim"], mx["vdim"]
            lin(m, [("q", H * D), ("k", H * D), ("v", H * Dv), ("g", H * Dv), ("i", H), ("f", H)], H, D, Dv)
            out.update({m + "i.b": [H], m + "f.b": [H], m + "norm": [H * Dv]})
        elif lc["type"] == "mamba2":
            H, Dv, Ns, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
            ch = H * Dv + 2 * G * Ns
            out.update({m + "in": [2 * H * Dv + 2 * G * Ns + H, W], m + "conv": [ch, mx["conv"]], m + "conv.b": [ch], m + "dt_bias": [H], m + "A_log": [H], m + "D": [H],
                        m + "norm": [H * Dv], m + "o": [W, H * Dv]})
        else:
            lm, rm = mx["left"], mx["right"]
            H, G, D, Dv = lm["heads"], lm.get("kv_heads", lm["heads"]), lm["dim"], lm["vdim"]
            lin(m + "left.", [("q", H * D), ("k", G * D), ("v", G * Dv)], H, D, Dv)
            out.update({m + "left.q.norm": [H * D], m + "left.k.norm": [G * D]})
            H, D, Dv = rm["heads"], rm["dim"], rm["vdim"]
            lin(m + "right.", [("q", H * D), ("f", H * D), ("v", H * Dv)], H, D, Dv)
            out.update({m + "right.f.b": [H * D], m + "right.lower": [H * D], m + "right.norm": [Dv]})
        out.update({p + "hc1.in": [S], p + "hc1.out": [S], p + "hc1.mix": [S, S]})
        ml = lc.get("mlp")
        if ml:
            f, r, ff = p + "mlp.", ml["router"], ml["expert"]["ff"]
            out[p + "norm2"] = []
            for e in range(r["experts"]):
                out.update({f + f"e{e}.gate": [ff, W], f + f"e{e}.up": [ff, W], f + f"e{e}.down": [W, ff]})
            Et = r["experts"] + r.get("identity", 0)
            out.update({f + "router": [Et, W], f + "correction": [Et]})
            if ml.get("shared"):
                sf = ml["shared"]["ff"]
                out.update({f + "shared.gate": [sf, W], f + "shared.up": [sf, W], f + "shared.down": [W, sf]})
            out.update({p + "hc2.in": [S], p + "hc2.out": [S], p + "hc2.mix": [S, S]})
    out["final.norm"] = []
    out["head"] = [cfg["vocab"], W]
    return out


def random_tensors(cfg: dict, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Seeded bf16 weights with magnitudes that keep every mechanism active (gates away from their ends, decays between 0 and 1, the
    router's choices spread over real and identity experts, streams that neither die nor blow up)."""
    g = torch.Generator().manual_seed(seed)
    scale = float((cfg.get("embedding") or {}).get("scale", 1.0))
    S = int(cfg.get("streams", 1))
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        rnd = lambda *a: torch.randn(shape, generator=g)
        if name.endswith(("q.norm", "k.norm", "mix.norm", "right.norm")) or leaf in ("norm1", "norm2") or name == "final.norm":
            t = 1.0 + 0.2 * rnd()
        elif name.endswith("hc1.mix") or name.endswith("hc2.mix"):
            t = 0.8 * torch.eye(S) + 0.2 / S + 0.1 * rnd()
        elif leaf == "in" and name.split(".")[-2] in ("hc1", "hc2"):
            t = 1.0 / S + 0.2 * rnd()
        elif leaf == "out":
            t = 1.0 + 0.3 * rnd()
        elif leaf == "lower":
            t = 0.1 + 0.8 * torch.rand(shape, generator=g)
        elif leaf == "A_log":
            t = -0.5 + 0.5 * rnd()
        elif leaf == "dt_bias":
            t = -1.0 + 0.5 * rnd()
        elif leaf == "D":
            t = 1.0 + 0.3 * rnd()
        elif name.endswith("f.b"):
            t = 2.0 + 1.0 * rnd()
        elif leaf == "correction":
            t = 0.05 * rnd()
        elif leaf == "b":
            t = 0.3 * rnd()
        elif leaf == "embed":
            t = rnd() / scale
        elif leaf == "pos":
            t = 0.5 * rnd()
        elif leaf == "router":
            t = rnd() * (2.0 / math.sqrt(shape[-1]))
        elif leaf == "conv":
            t = rnd() * 0.6
        else:
            t = rnd() * (1.2 / math.sqrt(shape[-1]))
        out[name] = t.to(torch.bfloat16)
    return out
