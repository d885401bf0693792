"""Serving loop of the layer-list runtime: a scheduler that forms batches, steps them through the model's step function,
samples, and gives finished sequences' pages and slots back.

Batching policy (static batches): waiting requests are admitted together, as many as slots and pages allow; the batch's
prompts run as one packed step, then the batch decodes one token per live request per step; requests leave as they
finish and the next batch is admitted when the batch is empty.  Sampling: greedy on the device; temperature / min-p
through the library's device sampler (the calm sampler kernels, lib.sample_logits) with its xorshift* generator.

Command line:  python -m calm_b200.serving MODEL_DIR --tokens 5,17,3 [--tokens ...] -n 32 [-t 0.8 --minp 0.05 --seed 1]"""
from __future__ import annotations

import argparse
import sys
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import numpy as np


@dataclass
class Request:
    rid: str
    prompt: List[int]
    max_new: int
    temperature: float = 0.0
    minp: float = 0.05
    eos: Optional[int] = None
    out: List[int] = field(default_factory=list)
    slot: int = -1
    done: bool = False


class Scheduler:
    def __init__(self, model, max_batch: int = 32, seed: int = 1):
        self.model, self.max_batch = model, max_batch
        self.waiting: List[Request] = []
        self.batch: List[Request] = []
        self.rng_state = seed or 1
        self.page = model.desc.page

    def add(self, req: Request) -> None:
        if not req.prompt:
            raise ValueError("empty prompt")
        limit = int(getattr(getattr(self.model, "desc", None), "max_positions", 0) or 0)
        if limit and len(req.prompt) + req.max_new - 1 > limit:  # the last generated token is never fed back
            raise ValueError(f"request {req.rid}: {len(req.prompt)} prompt tokens + {req.max_new} new ones pass the model's {limit} positions")
        self.waiting.append(req)

    def _pages_for(self, r: Request) -> int:
        return -(-(len(r.prompt) + r.max_new) // self.page)

    def _admit(self) -> None:
        budget = self.model.free_pages()
        while self.waiting and len(self.batch) < self.max_batch:
            need = self._pages_for(self.waiting[0])
            if need > budget:
                if not self.batch:
                    raise RuntimeError(f"request {self.waiting[0].rid} needs {need} pages, the pool has {budget}")
                break
            r = self.waiting.pop(0)
            r.slot = self.model.open()
            budget -= need
            self.batch.append(r)

    def _sample(self, reqs: List[Request], n: int, logits: Optional[np.ndarray]) -> List[int]:
        if logits is None:
            return [int(t) for t in self.model.argmax(n)]
        from . import build as cbuild
        from . import lib

        cbuild.build(target="engine")  # the device sampler lives in the calm engine's library: built on first use
        out = []
        for r, row in zip(reqs, logits):
            tok, self.rng_state = lib.sample_logits(row, r.temperature, r.minp, self.rng_state)
            out.append(int(tok))
        return out

    def _advance(self, live: List[Request], token_lists: List[List[int]]) -> None:
        ends, at = [], 0
        for t in token_lists:
            at += len(t)
            ends.append(at - 1)
        greedy = all(r.temperature == 0.0 for r in live)
        logits = self.model.step([r.slot for r in live], token_lists, ends, fetch=not greedy)
        for r, tok in zip(live, self._sample(live, len(live), logits)):
            r.out.append(tok)
            if len(r.out) >= r.max_new or (r.eos is not None and tok == r.eos):
                r.done = True
                self.model.close_seq(r.slot)

    def run(self) -> Dict[str, List[int]]:
        """Serve everything that was added; returns rid -> generated tokens."""
        finished: Dict[str, List[int]] = {}
        while self.waiting or self.batch:
            if not self.batch:
                self._admit()
                self._advance(self.batch, [r.prompt for r in self.batch])
            else:
                self._advance(self.batch, [[r.out[-1]] for r in self.batch])
            for r in self.batch:
                if r.done:
                    finished[r.rid] = r.out
            self.batch = [r for r in self.batch if not r.done]
        return finished


def generate(model, prompts: List[List[int]], max_new: int, temperature: float = 0.0, minp: float = 0.05, seed: int = 1, max_batch: int = 32):
    s = Scheduler(model, max_batch=max_batch, seed=seed)
    for i, p in enumerate(prompts):
        s.add(Request(str(i), list(p), max_new, temperature, minp))
    done = s.run()
    return [done[str(i)] for i in range(len(prompts))]


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="generate token ids with a layer-list model")
    ap.add_argument("model")
    ap.add_argument("--tokens", action="append", required=True, help="a prompt as comma-separated token ids (repeatable)")
    ap.add_argument("-n", type=int, default=32, help="tokens to generate per prompt")
    ap.add_argument("-t", "--temperature", type=float, default=0.0)
    ap.add_argument("--minp", type=float, default=0.05)
    ap.add_argument("--seed", type=int, default=1)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    a = ap.parse_args(argv)
    from . import registry

    prompts = [[int(x) for x in p.split(",")] for p in a.tokens]
    total = sum(len(p) + a.n for p in prompts)
    with registry.load_model(a.model, dtype=a.dtype, max_tokens=total, max_seqs=len(prompts)) as model:
        for p, out in zip(prompts, generate(model, prompts, a.n, a.temperature, a.minp, a.seed, max_batch=len(prompts))):
            print(",".join(map(str, out)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
