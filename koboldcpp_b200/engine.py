"""Scheduler, batching and sampling over a SequenceModel.

`Engine.step` is the one place a batch reaches the model: it takes (request, next tokens, wanted places) entries, lays the
tokens of each request next to each other, and returns the logits of the wanted places.  `Engine.generate` is the serving
loop on top of it: requests wait in a queue, are admitted while sequences and cache cells are free, their prompts are fed
in portions beside the single tokens of the requests that already decode, and a finished request gives its sequence back.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .lib import B200Error


@dataclass
class Sampler:
    """temperature 0 = greedy (lowest index among equal logits); else softmax(logits / temperature) over the top_k largest,
    cut to the smallest set whose mass reaches top_p."""
    temperature: float = 0.0
    top_k: int = 0
    top_p: float = 1.0
    seed: int = 0
    _rng: np.random.Generator = field(default=None, repr=False)

    def pick(self, logits: np.ndarray) -> int:
        if self.temperature <= 0.0:
            return int(np.argmax(logits))
        if self._rng is None:
            self._rng = np.random.default_rng(self.seed)
        z = logits.astype(np.float64) / self.temperature
        order = np.argsort(-z, kind="stable")
        if self.top_k > 0:
            order = order[: self.top_k]
        p = np.exp(z[order] - z[order[0]])
        p /= p.sum()
        if self.top_p < 1.0:
            keep = int(np.searchsorted(np.cumsum(p), self.top_p) + 1)
            order, p = order[:keep], p[:keep] / p[:keep].sum()
        return int(order[self._rng.choice(len(order), p=p)])


@dataclass
class Request:
    prompt: list[int]
    max_new_tokens: int
    sampler: Sampler = field(default_factory=Sampler)
    stop: tuple[int, ...] = ()
    # state
    seq: int = -1
    fed: int = 0                 # prompt tokens already in the cache
    output: list[int] = field(default_factory=list)
    done: bool = False


class Engine:
    def __init__(self, model, max_step_tokens: int | None = None):
        self.model = model
        self.max_step_tokens = min(max_step_tokens or model.max_batch, model.max_batch)
        self.seqs: dict[object, int] = {}   # request handle -> sequence id

    # ---------------------------------------------------------------- one step
    def step(self, entries) -> np.ndarray:
        """entries: iterable of (handle, tokens, want) -- the next tokens of the request `handle` (any hashable; a new one opens a
        sequence) and the places among them whose logits are wanted.  Returns [wanted places in entry order, vocab]."""
        toks, sids, want = [], [], []
        for handle, tokens, places in entries:
            if handle not in self.seqs:
                self.seqs[handle] = self.model.seq_open()
            w = np.zeros(len(tokens), dtype=np.int8)
            w[list(places)] = 1
            toks.extend(tokens); sids.extend([self.seqs[handle]] * len(tokens)); want.extend(w)
        if not toks:
            return np.empty((0, self.model.vocab), dtype=np.float32)
        return self.model.decode_batch(toks, sids, want)

    def finish(self, handle) -> None:
        """The request is over: its cache cells and state slot are free again."""
        seq = self.seqs.pop(handle, None)
        if seq is not None:
            self.model.seq_close(seq)

    # ---------------------------------------------------------------- serving loop
    def generate(self, requests: list[Request]) -> list[list[int]]:
        """Run all requests to completion with continuous batching; returns the generated tokens per request."""
        m = self.model
        for r in requests:
            if not r.prompt:
                raise B200Error("a request needs at least one prompt token")
            if len(r.prompt) + r.max_new_tokens > m.n_ctx:
                raise B200Error(f"a request of {len(r.prompt)} + {r.max_new_tokens} tokens does not fit {m.n_ctx} cache cells")
        waiting = list(requests)
        running: list[Request] = []
        reserved = 0  # cells promised to the running requests
        while waiting or running:
            while waiting and len(running) < m.n_seq_max and reserved + len(waiting[0].prompt) + waiting[0].max_new_tokens <= m.n_ctx:
                r = waiting.pop(0)
                reserved += len(r.prompt) + r.max_new_tokens
                running.append(r)
            budget = self.max_step_tokens
            entries, owners = [], []
            for r in running:  # decoding requests first: one token each
                if r.fed == len(r.prompt) and budget > 0:
                    entries.append((id(r), [r.output[-1]], [0])); owners.append(r); budget -= 1
            for r in running:  # then portions of prompts
                if r.fed < len(r.prompt) and budget > 0:
                    n = min(budget, len(r.prompt) - r.fed)
                    last = r.fed + n == len(r.prompt)
                    entries.append((id(r), r.prompt[r.fed:r.fed + n], [n - 1] if last else [])); owners.append(r if last else None)
                    r.fed += n; budget -= n
            logits = self.step(entries)
            row = 0
            for r in owners:
                if r is None:
                    continue
                tok = r.sampler.pick(logits[row]); row += 1
                r.output.append(tok)
                if len(r.output) >= r.max_new_tokens or tok in r.stop:
                    r.done = True
            for r in [r for r in running if r.done]:
                running.remove(r)
                reserved -= len(r.prompt) + r.max_new_tokens
                self.finish(id(r))
        return [r.output for r in requests]
