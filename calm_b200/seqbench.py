"""Throughput of the layer-list families at layer sizes of real models (random weights), each beside its closest existing
model on the same GPU: Vimulorn beside a Llama-shaped stack of the same width, depth, head geometry and feed-forward width in
fp16 on the calm engine; Bovinex beside Vimulorn at the same width, depth, head geometry, window and feed-forward width on
the same runtime (both have windowed grouped-query attention and a recurrent mixer with a [dim x vdim] state per head); Zazilix
beside Bovinex likewise (both have grouped-query attention with a bounded view, linear recurrences on the same scan kernel and routed experts);
Sopepel beside Bovinex too (the same two mixers, grouped-query attention and gated linear attention, side by side in every layer with half the heads each).

Per size: prompt throughput (one prompt of `prompt` tokens as one step), decode throughput for one sequence and for a
batch, each after warm-up, timed with CUDA events on the library's stream; then one profiled pass that brackets every
launch with events and reports, per kind of kernel, its time and its distance from the roofline (bytes / measured copy
bandwidth, flops / measured bf16 GEMM throughput, whichever is larger).  Inputs exceed L2 at every size (weights alone
are hundreds of MB), so no flush between iterations."""
from __future__ import annotations

import json
import math
import os
import time
from dataclasses import replace

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SIZES = {
    # name: (width, ff, blocks of [latent, delta, window], heads, head dim, kv heads, kv_rank, q_rank, window, vocab)
    "w1024": dict(width=1024, ff=2816, blocks=2, heads=8, dim=128, kv_heads=2, kv_rank=256, q_rank=384, window=512, vocab=32000),
    "w2048": dict(width=2048, ff=5632, blocks=2, heads=16, dim=128, kv_heads=4, kv_rank=512, q_rank=768, window=1024, vocab=32000),
    "w4096": dict(width=4096, ff=11264, blocks=1, heads=32, dim=128, kv_heads=8, kv_rank=512, q_rank=1536, window=1024, vocab=32000),
}


def vimulorn_config(z: dict) -> dict:
    mlp = {"ff": z["ff"], "kind": "dense", "limit": 7.0}
    H, D = z["heads"], z["dim"]
    block = [
        {"type": "latent_attention", "mixer": {"heads": H, "dim": D, "vdim": D, "kv_rank": z["kv_rank"], "q_rank": z["q_rank"], "scale": D ** -0.5}, "mlp": mlp},
        {"type": "channel_delta", "mixer": {"heads": H, "kv_heads": H, "dim": D, "vdim": D, "conv": 4, "a_rank": 64, "g_rank": 64}, "mlp": mlp},
        {"type": "attention", "mixer": {"heads": H, "kv_heads": z["kv_heads"], "dim": D, "vdim": D, "conv": 4, "mask": {"size": z["window"]}, "scale": D ** -0.5}, "mlp": mlp},
    ]
    return {"architecture": "Vimulorn", "layers": block * z["blocks"], "norm": {"eps": 1e-5}, "vocab": z["vocab"], "width": z["width"]}


def bovinex_config(z: dict) -> dict:
    """Blocks of [attention + dense, linear attention + routed experts, linear attention + dense]; two of eight experts of half the
    dense width are active per token, which is the dense feed-forward's work in three matrices instead of two."""
    H, D = z["heads"], z["dim"]
    dense = {"ff": z["ff"], "kind": "dense"}
    moe = {"kind": "moe", "expert": {"ff": z["ff"] // 2}, "router": {"experts": 8, "top": 2}}
    rot = {"dims": D // 2, "base": 1e6, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    block = [
        {"type": "attention", "mixer": {"heads": H, "kv_heads": z["kv_heads"], "dim": D, "vdim": D, "scale": D ** -0.5, "rot": rot,
                                        "mask": {"size": z["window"], "keep_first": 64}}, "mlp": dense},
        {"type": "gla", "mixer": {"heads": H, "dim": D, "vdim": D, "tau": 16.0, "a_rank": 64}, "mlp": moe},
        {"type": "gla", "mixer": {"heads": H, "dim": D, "vdim": D, "tau": 16.0, "a_rank": 64}, "mlp": dense},
    ]
    return {"architecture": "Bovinex", "embedding": {"scale": math.sqrt(z["width"])}, "layers": block * z["blocks"], "norm": {"eps": 1e-5}, "vocab": z["vocab"],
            "width": z["width"]}


def zazilix_config(z: dict, max_positions: int = 4096) -> dict:
    """Blocks of [mLSTM, attention in blocks of positions beside HGRN2, Mamba-2], every layer with eight routed experts of half the dense
    width (two active per token), two identity experts and a shared unit of a quarter of the dense width; four residual streams."""
    H, D = z["heads"], z["dim"]
    moe = {"kind": "moe", "expert": {"ff": z["ff"] // 2}, "router": {"experts": 8, "identity": 2, "top": 2, "scale": 1.5}, "shared": {"ff": z["ff"] // 4}}
    block = [
        {"type": "mlstm", "mixer": {"heads": H, "dim": D, "vdim": D, "gate_cap": 15.0}, "mlp": moe},
        {"type": "parallel", "mixer": {"left": {"heads": H, "kv_heads": z["kv_heads"], "dim": D, "vdim": D, "scale": D ** -0.5, "mask": {"size": z["window"]}},
                                       "right": {"heads": H, "dim": D, "vdim": D}, "left_scale": 0.7, "right_scale": 0.7}, "mlp": moe},
        {"type": "mamba2", "mixer": {"heads": H, "vdim": D, "state": 128, "groups": z["kv_heads"], "conv": 4, "norm_groups": z["kv_heads"]}, "mlp": moe},
    ]
    return {"architecture": "Zazilix", "embedding": {"scale": math.sqrt(z["width"])}, "layers": block * z["blocks"], "norm": {"eps": 1e-5}, "vocab": z["vocab"],
            "width": z["width"], "streams": 4, "max_positions": max_positions}


def sopepel_config(z: dict) -> dict:
    """Blocks of [pair + dense, pair + routed experts, pair + dense]; a pair is grouped-query attention inside blocks of `window` positions beside
    gated linear attention, half of the size's heads each, so a layer's mixer has the width of one of Bovinex's; eight relu^2 experts of half the
    dense width (two active per token) and a gated shared unit of a quarter of it."""
    H, D = z["heads"], z["dim"]
    dense = {"ff": z["ff"], "kind": "dense"}
    moe = {"kind": "moe", "expert": {"ff": z["ff"] // 2}, "router": {"experts": 8, "top": 2}, "shared": {"ff": z["ff"] // 4}}
    mixer = {"left": {"heads": H // 2, "kv_heads": max(z["kv_heads"] // 2, 1), "dim": D, "vdim": D, "scale": D ** -0.5, "rot": {"dims": D // 2, "base": 1e6}, "mask": {"size": z["window"]}},
             "right": {"heads": H // 2, "dim": D, "vdim": D, "tau": 16.0, "a_rank": 64}, "left_scale": 1.0, "right_scale": 0.5}
    block = [{"type": "parallel", "mixer": mixer, "mlp": dense}, {"type": "parallel", "mixer": mixer, "mlp": moe}, {"type": "parallel", "mixer": mixer, "mlp": dense}]
    return {"architecture": "Sopepel", "embedding": {"bigram": {"buckets": 16381, "mul_prev": 36313, "mul_cur": 27191}}, "layers": block * z["blocks"], "norm": {"eps": 1e-5},
            "vocab": z["vocab"], "width": z["width"], "logit_scale": 1.0}


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), float(d["bf16_tflops"]), "measured"
    return 6650.0, 1590.0, "fallback"


def roofline_table(stats: dict, hbm_gbs: float, tflops: float) -> dict:
    out = {}
    for k, (ms, by, fl, n) in stats.items():
        if not n or ms <= 0:
            continue
        floor_ms = max(by / (hbm_gbs * 1e9), fl / (tflops * 1e12)) * 1e3
        out[k] = {"ms": round(ms, 4), "launches": n, "gbs": round(by / 1e9 / (ms / 1e3), 1), "tflops": round(fl / 1e12 / (ms / 1e3), 2),
                  "bound": "hbm" if by / (hbm_gbs * 1e9) >= fl / (tflops * 1e12) else "tensor", "frac_of_roofline": round(floor_ms / ms, 4)}
    return out


def bench_family(family: str, name: str, prompt: int, batch: int, steps: int, warmup: int, seed: int = 0) -> list:
    from . import bovinex, sopepel, vimulorn, zazilix

    z = SIZES[name]
    mod, cfg = {"bovinex": (bovinex, bovinex_config(z)), "zazilix": (zazilix, zazilix_config(z, prompt + steps + 2 * warmup + 64)),
                "sopepel": (sopepel, sopepel_config(z))}.get(family, (vimulorn, vimulorn_config(z)))
    hbm, tf, src = peaks()
    t0 = time.time()
    tensors = mod.random_tensors(cfg, seed)
    params = sum(t.numel() for t in tensors.values())
    rng = np.random.default_rng(seed)
    lines = []
    with mod.from_tensors(cfg, tensors, "bfloat16", max_tokens=(batch + 1) * (prompt + steps + warmup + 8), max_seqs=batch + 1, page=16) as m:
        del tensors
        toks = [int(x) for x in rng.integers(0, z["vocab"], prompt)]

        def prefill_once(profile=False):
            s = m.open()
            m.timer_start()
            m.step([s], [toks], [prompt - 1], fetch=False)
            ms = m.timer_stop()
            m.close_seq(s)
            return ms

        for _ in range(max(warmup // 4, 3)):
            prefill_once()
        ms = min(prefill_once() for _ in range(5))
        m.perf(True)
        prefill_once()
        table = roofline_table(m.perf_stats(), hbm, tf)
        m.perf(False)
        lines.append({"family": family, "size": name, "phase": "prefill", "tokens": prompt, "ms": round(ms, 3), "tokens_per_s": round(prompt / ms * 1e3, 1),
                      "params": params, "kernels": table, "peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "source": src}})
        for b in sorted({1, batch}):
            slots = [m.open() for _ in range(b)]
            m.step(slots, [toks] * b, [], fetch=False)
            nxt = [[int(rng.integers(0, z["vocab"]))] for _ in range(b)]
            for _ in range(warmup):
                m.step(slots, nxt, list(range(b)), fetch=False)
            m.timer_start()
            for _ in range(steps):
                m.step(slots, nxt, list(range(b)), fetch=False)
            ms = m.timer_stop() / steps
            m.perf(True)
            m.step(slots, nxt, list(range(b)), fetch=False)
            table = roofline_table(m.perf_stats(), hbm, tf)
            m.perf(False)
            for s in slots:
                m.close_seq(s)
            lines.append({"family": family, "size": name, "phase": "decode", "batch": b, "context": prompt, "ms_per_step": round(ms, 4),
                          "tokens_per_s": round(b / ms * 1e3, 1), "kernels": table})
    for ln in lines:
        ln["setup_s"] = round(time.time() - t0, 1)
    return lines


def bench_llama_twin(name: str, prompt: int, steps: int, warmup: int, seed: int = 0) -> list:
    """The calm engine on a Llama-shaped model of the same width / depth / heads / feed-forward, fp16 weights."""
    from . import lib
    from . import modelgen as mg

    z = SIZES[name]
    spec = mg.ModelSpec("twin-" + name, z["width"], z["ff"], 3 * z["blocks"], z["heads"], z["kv_heads"], z["dim"], z["vocab"], "fp16", max_seq_len=prompt + steps + warmup + 64)
    host = mg.HostModel(spec, seed=seed)
    toks = mg.teacher_tokens(spec.vocab_size, prompt)
    L = lib.load()
    lines = []
    with lib.DeviceModel(spec, host.tensors, seq_len=spec.max_seq_len) as dm:
        best, served = 1e30, 0
        for i in range(5):
            L.calm_b200_timer_start()
            served = dm.prefill(toks, 0)
            best = min(best, L.calm_b200_timer_stop()) if i >= 2 else best
        lines.append({"family": "llama-twin", "size": name, "phase": "prefill", "tokens": prompt, "ms": round(best, 3), "tokens_per_s": round(prompt / best * 1e3, 1),
                      "tensor_core_pass": bool(served)})
        dm.decode_greedy(1, prompt, warmup)
        L.calm_b200_timer_start()
        dm.decode_greedy(1, prompt + warmup, steps)
        ms = L.calm_b200_timer_stop() / steps
        stats, span = dm.profile(23, prompt + warmup + steps, 8)
        hbm = peaks()[0]
        table = {k: {"us_per_launch": round(v[0] / max(v[2], 1) * 1e3, 2), "frac_of_roofline": round(v[1] / 1e9 / (v[0] / 1e3) / hbm, 4)} for k, v in stats.items() if v[2] and v[0] > 0}
        lines.append({"family": "llama-twin", "size": name, "phase": "decode", "batch": 1, "context": prompt, "ms_per_step": round(ms, 4), "tokens_per_s": round(1e3 / ms, 1),
                      "kernels": table})
    return lines


def main(sizes, prompt=2048, batch=16, steps=32, warmup=8, twin=True, family="vimulorn"):
    from . import build as cbuild

    cbuild.build(target="seq")
    llama = twin and family == "vimulorn"
    if llama:
        cbuild.build(target="engine")
    os.environ.setdefault("CALM_B200_QUIET", "1")
    out = []
    for name in sizes:
        lines = bench_family(family, name, prompt, batch, steps, warmup)
        if twin and family == "bovinex":
            lines += bench_family("vimulorn", name, prompt, batch, steps, warmup)
        if twin and family in ("zazilix", "sopepel"):
            lines += bench_family("bovinex", name, prompt, batch, steps, warmup)
        if llama:
            lines += bench_llama_twin(name, prompt, steps, warmup)
        for ln in lines:
            print(json.dumps(ln), flush=True)
            out.append(ln)
    return out
