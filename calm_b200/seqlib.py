"""ctypes binding of libcalm_b200_seq.so (include/calm_b200_seq.h): layer-list models served to batches of sequences.

Same protocol as the calm boundary in lib.py: upload every tensor, bind the device pointers in the records, prepare, then
step.  No CPU path: loading builds the library when it is missing and fails loudly when that cannot be done."""
from __future__ import annotations

import ctypes as C
import os
from typing import Dict, List, Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SEQ_LATENT, SEQ_DELTA, SEQ_WINDOW, SEQ_GQA, SEQ_GLA, SEQ_MLSTM, SEQ_HGRN2, SEQ_MAMBA2, SEQ_PAIR = 0, 1, 2, 3, 4, 5, 6, 7, 8
NORM_DYT, NORM_RMS = 0, 1
BLOCK_SERIAL, BLOCK_PARALLEL, BLOCK_HYPER, BLOCK_POST = 0, 1, 2, 3
FF_CLAMPED, FF_RELU2, FF_MOE, FF_GATED = 0, 1, 2, 3
ACT_SILU, ACT_GELU_TANH = 0, 1
_fptr = C.POINTER(C.c_float)
_iptr = C.POINTER(C.c_int)


class SeqNorm(C.Structure):
    _fields_ = [("w", C.c_void_p), ("b", C.c_void_p), ("alpha", C.c_void_p)]


class SeqHyper(C.Structure):
    _fields_ = [("in_", C.c_void_p), ("out", C.c_void_p), ("mix", C.c_void_p)]


class SeqLayer(C.Structure):
    pass


SeqLayer._fields_ = [(n, C.c_int) for n in ("type", "heads", "kv_heads", "dim", "vdim", "q_rank", "kv_rank", "taps", "window", "a_rank", "g_rank", "ff")] + \
               [("scale", C.c_float), ("limit", C.c_float)] + [(n, SeqNorm) for n in ("norm1", "norm1b", "norm2", "norm2b")] + \
               [(n, C.c_void_p) for n in ("w_in", "w_o", "dq_norm", "dkv_norm", "w_uq", "w_ukT", "w_uv", "conv", "w_a2", "w_g2", "a_log", "dt_bias",
                                          "out_norm", "sink", "w_gate_up", "w_down", "b_in", "q_norm", "k_norm", "b_a2")] + \
               [(n, C.c_int) for n in ("keep_first", "rot_dims")] + \
               [(n, C.c_float) for n in ("rot_base", "rot_factor", "rot_original", "rot_fast", "rot_slow", "tau")] + \
               [(n, C.c_int) for n in ("ff_kind", "experts", "top")] + [(n, C.c_void_p) for n in ("w_router", "b_router")] + [("in_tail", C.c_int)] + \
               [(n, C.c_int) for n in ("chunk", "dist_bias", "add_one", "v_norm", "no_gate")] + [("gate_cap", C.c_float)] + \
               [(n, C.c_void_p) for n in ("lower", "conv_b", "skip_d")] + [("norm_groups", C.c_int), ("pair", C.POINTER(SeqLayer)), ("pair_scale", C.c_float * 2),
                                                                         ("hc1", SeqHyper), ("hc2", SeqHyper), ("route_mode", C.c_int), ("ident", C.c_int),
                                                                         ("route_scale", C.c_float), ("correction", C.c_void_p), ("shared_ff", C.c_int),
                                                                         ("w_sh_gate_up", C.c_void_p), ("w_sh_down", C.c_void_p),
                                                                         ("qk_per_head", C.c_int), ("gate_per_head", C.c_int), ("b_o", C.c_void_p), ("scores_f32", C.c_int), ("ff_act", C.c_int),
                                                                         ("expert_act", C.c_int), ("weight_input", C.c_int), ("shared_gate", C.c_int)]


class SeqModel(C.Structure):
    _fields_ = [(n, C.c_int) for n in ("vocab", "width", "n_layers", "loop_start", "loop_stop", "loop_times")] + [("eps", C.c_float)] + \
               [(n, C.c_int) for n in ("exact", "max_tokens", "max_seqs", "page")] + \
               [("embed", C.c_void_p), ("head", C.c_void_p), ("final_norm", SeqNorm), ("layers", C.POINTER(SeqLayer)),
                ("norm_kind", C.c_int), ("norm_offset", C.c_float), ("block", C.c_int), ("embed_scale", C.c_float),
                ("streams", C.c_int), ("norm_scalar", C.c_int), ("pos_table", C.c_void_p), ("max_positions", C.c_int),
                ("bigram", C.c_void_p), ("bigram_buckets", C.c_int), ("bigram_mul_prev", C.c_int), ("bigram_mul_cur", C.c_int), ("logit_scale", C.c_float)]


_lib = None


def load() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    from . import build as cbuild

    path = cbuild.build(target="seq")  # compiles on first use (a fresh checkout), a no-op afterwards
    L = C.CDLL(path)
    L.calm_b200_seq_upload.argtypes, L.calm_b200_seq_upload.restype = [C.c_void_p, C.c_size_t], C.c_void_p
    L.calm_b200_seq_free.argtypes, L.calm_b200_seq_free.restype = [C.c_void_p], None
    L.calm_b200_seq_prepare.argtypes, L.calm_b200_seq_prepare.restype = [C.POINTER(SeqModel)], C.c_void_p
    L.calm_b200_seq_release.argtypes, L.calm_b200_seq_release.restype = [C.c_void_p], None
    L.calm_b200_seq_open.argtypes, L.calm_b200_seq_open.restype = [C.c_void_p], C.c_int
    L.calm_b200_seq_close.argtypes, L.calm_b200_seq_close.restype = [C.c_void_p, C.c_int], C.c_int
    L.calm_b200_seq_length.argtypes, L.calm_b200_seq_length.restype = [C.c_void_p, C.c_int], C.c_int
    L.calm_b200_seq_free_pages.argtypes, L.calm_b200_seq_free_pages.restype = [C.c_void_p], C.c_int
    L.calm_b200_seq_step.argtypes = [C.c_void_p, C.c_int, _iptr, _iptr, _iptr, C.c_int, _iptr, _fptr]
    L.calm_b200_seq_step.restype = C.c_int
    L.calm_b200_seq_argmax.argtypes, L.calm_b200_seq_argmax.restype = [C.c_void_p, _iptr], None
    L.calm_b200_seq_device_logits.argtypes, L.calm_b200_seq_device_logits.restype = [C.c_void_p], C.c_void_p
    L.calm_b200_seq_set_trace.argtypes, L.calm_b200_seq_set_trace.restype = [C.c_void_p, C.c_int], None
    L.calm_b200_seq_layer_runs.argtypes, L.calm_b200_seq_layer_runs.restype = [C.c_void_p], C.c_int
    L.calm_b200_seq_read_trace.argtypes, L.calm_b200_seq_read_trace.restype = [C.c_void_p, C.c_int, _fptr], None
    L.calm_b200_seq_launch_count.argtypes, L.calm_b200_seq_launch_count.restype = [], C.c_uint64
    L.calm_b200_seq_timer_start.argtypes, L.calm_b200_seq_timer_start.restype = [C.c_void_p], None
    L.calm_b200_seq_timer_stop.argtypes, L.calm_b200_seq_timer_stop.restype = [C.c_void_p], C.c_float
    L.calm_b200_seq_set_perf.argtypes, L.calm_b200_seq_set_perf.restype = [C.c_void_p, C.c_int], None
    L.calm_b200_seq_perf_stats.argtypes = [C.c_void_p, C.c_int, C.c_char_p, C.c_int, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(C.c_double),
                                           C.POINTER(C.c_long)]
    L.calm_b200_seq_perf_stats.restype = C.c_int
    _lib = L
    return L


class SeqError(RuntimeError):
    pass


class SeqDeviceModel:
    """A layer-list model on the GPU.  `layers` are dicts of SeqLayer fields whose tensor-valued entries name tensors in
    `tensors` (host torch tensors, uploaded here); vimulorn.py, bovinex.py, zazilix.py and sopepel.py are the hosts that fill them from a checkpoint."""

    def __init__(self, head: Dict[str, object], layers: List[Dict[str, object]], tensors: Dict[str, "object"], exact: bool = False,
                 max_tokens: int = 4096, max_seqs: int = 64, page: int = 16):
        self.lib = load()
        self._uploaded: Dict[str, int] = {}
        self._keep = tensors

        def ptr(name: Optional[str]) -> Optional[int]:
            if name is None:
                return None
            if name not in self._uploaded:
                t = tensors[name].contiguous()
                self._uploaded[name] = self.lib.calm_b200_seq_upload(t.data_ptr(), t.numel() * t.element_size())
            return self._uploaded[name]

        def norm(prefix: str) -> SeqNorm:  # an RMS norm has only its weight
            return SeqNorm(ptr(prefix), ptr(prefix + ".b") if prefix + ".b" in tensors else None, ptr(prefix + ".alpha") if prefix + ".alpha" in tensors else None)

        self._subs = []  # the records that pairs point at

        def fill(rec: SeqLayer, d: Dict[str, object]) -> None:
            for k, v in d.items():
                if k in ("norm1", "norm1b", "norm2", "norm2b"):
                    setattr(rec, k, norm(v) if v else SeqNorm())
                elif k in ("hc1", "hc2"):  # names of the three tensors of a hyper-connection: in, out, mix
                    setattr(rec, k, SeqHyper(*[ptr(x) for x in v]) if v else SeqHyper())
                elif k == "pair":
                    two = (SeqLayer * 2)()
                    fill(two[0], v[0]), fill(two[1], v[1])
                    self._subs.append(two)
                    rec.pair = C.cast(two, C.POINTER(SeqLayer))
                elif k == "pair_scale":
                    rec.pair_scale[0], rec.pair_scale[1] = float(v[0]), float(v[1])
                elif isinstance(v, str) or v is None:
                    setattr(rec, k, ptr(v))
                else:
                    setattr(rec, k, v)

        self._layers = (SeqLayer * len(layers))()
        for rec, d in zip(self._layers, layers):
            fill(rec, d)
        m = SeqModel()
        m.vocab, m.width, m.n_layers = head["vocab"], head["width"], len(layers)
        m.loop_start, m.loop_stop, m.loop_times = head.get("loop_start", 0), head.get("loop_stop", 0), head.get("loop_times", 1)
        m.eps, m.exact, m.max_tokens, m.max_seqs, m.page = head["eps"], int(exact), int(max_tokens), int(max_seqs), int(page)
        m.embed, m.head, m.final_norm = ptr(head["embed"]), ptr(head["head"]), norm(head["final_norm"])
        m.norm_kind, m.norm_offset = int(head.get("norm_kind", NORM_DYT)), float(head.get("norm_offset", 0.0))
        m.block, m.embed_scale = int(head.get("block", BLOCK_SERIAL)), float(head.get("embed_scale", 1.0))
        m.streams, m.norm_scalar = int(head.get("streams", 1)), int(head.get("norm_scalar", 0))
        m.pos_table, m.max_positions = ptr(head.get("pos_table")), int(head.get("max_positions", 0))
        m.bigram, m.bigram_buckets = ptr(head.get("bigram")), int(head.get("bigram_buckets", 0))
        m.bigram_mul_prev, m.bigram_mul_cur = int(head.get("bigram_mul_prev", 0)), int(head.get("bigram_mul_cur", 0))
        m.logit_scale = float(head.get("logit_scale", 1.0))
        m.layers = C.cast(self._layers, C.POINTER(SeqLayer))
        self.desc = m
        self.vocab, self.width = m.vocab, m.width
        self.handle = self.lib.calm_b200_seq_prepare(C.byref(m))

    # ---- state manager
    def open(self) -> int:
        slot = self.lib.calm_b200_seq_open(self.handle)
        if slot < 0:
            raise SeqError("no free sequence slot")
        return slot

    def close_seq(self, slot: int) -> None:
        if self.lib.calm_b200_seq_close(self.handle, slot) != 0:
            raise SeqError(f"slot {slot} is not open")

    def length(self, slot: int) -> int:
        return self.lib.calm_b200_seq_length(self.handle, slot)

    def free_pages(self) -> int:
        return self.lib.calm_b200_seq_free_pages(self.handle)

    # ---- the step function
    def step(self, slots: Sequence[int], token_lists: Sequence[Sequence[int]], want: Sequence[int], fetch: bool = True) -> Optional[np.ndarray]:
        """Feed token_lists[i] to the sequence in slots[i]; `want` = packed indices whose logits are computed.  Returns
        float32 [len(want), vocab] (None when want is empty or fetch is False: the logits then stay on the device)."""
        sl = np.ascontiguousarray(slots, np.int32)
        cn = np.ascontiguousarray([len(t) for t in token_lists], np.int32)
        tk = np.ascontiguousarray([x for t in token_lists for x in t], np.int32)
        wn = np.ascontiguousarray(want, np.int32)
        out = np.empty((len(wn), self.vocab), np.float32) if (fetch and len(wn)) else None
        rc = self.lib.calm_b200_seq_step(self.handle, len(sl), sl.ctypes.data_as(_iptr), cn.ctypes.data_as(_iptr), tk.ctypes.data_as(_iptr), len(wn),
                                         wn.ctypes.data_as(_iptr), out.ctypes.data_as(_fptr) if out is not None else None)
        if rc == -2:
            raise SeqError("the page pool is exhausted: more live tokens than max_tokens")
        if rc != 0:
            raise SeqError("bad step: a slot that is not open, an empty entry, a token outside the vocabulary, a wanted index outside the batch "
                           "or a sequence longer than the model's position table")
        return out

    def argmax(self, n_want: int) -> np.ndarray:
        out = np.zeros(n_want, np.int32)
        self.lib.calm_b200_seq_argmax(self.handle, out.ctypes.data_as(_iptr))
        return out

    def set_trace(self, on: bool) -> None:
        self.lib.calm_b200_seq_set_trace(self.handle, int(on))

    def read_trace(self, n_tokens: int) -> np.ndarray:
        runs = self.lib.calm_b200_seq_layer_runs(self.handle)
        out = np.zeros((runs, n_tokens, self.width), np.float32)
        for r in range(runs):
            self.lib.calm_b200_seq_read_trace(self.handle, r, out[r].ctypes.data_as(_fptr))
        return out

    def perf(self, on: bool) -> None:
        self.lib.calm_b200_seq_set_perf(self.handle, int(on))

    def perf_stats(self) -> Dict[str, tuple]:
        out, k = {}, 0
        name = C.create_string_buffer(64)
        ms, by, fl, nl = C.c_double(), C.c_double(), C.c_double(), C.c_long()
        while self.lib.calm_b200_seq_perf_stats(self.handle, k, name, 64, C.byref(ms), C.byref(by), C.byref(fl), C.byref(nl)):
            out[name.value.decode()] = (ms.value, by.value, fl.value, nl.value)
            k += 1
        return out

    def timer_start(self) -> None:
        self.lib.calm_b200_seq_timer_start(self.handle)

    def timer_stop(self) -> float:
        return self.lib.calm_b200_seq_timer_stop(self.handle)

    def close(self) -> None:
        if self.handle:
            self.lib.calm_b200_seq_release(self.handle)
            for p in self._uploaded.values():
                self.lib.calm_b200_seq_free(p)
            self.handle, self._uploaded = None, {}

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()
