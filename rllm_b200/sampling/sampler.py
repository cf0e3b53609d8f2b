"""Chooses tokens from a step's logits on the device: argmax rows and sampled rows in one
pass each, parameters per row. Pipeline of the reference's `sample_from_logits`
(src/model/sampler.rs:328-547): penalties -> logit bias -> temperature -> top-k -> softmax
[-> log-probabilities] -> min-p -> top-p -> inverse CDF."""
from __future__ import annotations

import torch

from .params import SamplingParams
from .rng import uniform


class Sampler:
    def __init__(self, backend):
        self.backend = backend
        self.device = backend.device
        self._ring, self._turn = [], 0
        self._held = []          # pinned lists a kernel may still read, each with its event

    def __call__(self, logits: torch.Tensor, params: list[SamplingParams], seeds: list[int],
                 indices: list[int], histories: list[list[int]] | None = None) -> list[int]:
        """The drawn tokens as a host list (waits for the device)."""
        return self.draw(logits, params, seeds, indices, histories).tolist()

    def draw(self, logits: torch.Tensor, params: list[SamplingParams], seeds: list[int],
             indices: list[int], histories: list[list[int]] | None = None, logprobs: bool = False):
        """logits float32 [R, V]; row r is drawn with params[r] and the uniform number of
        (seeds[r], indices[r]). `histories[r]`: the tokens generated so far (for penalties).
        Returns int32 [R] on the device; nothing here waits for it. With `logprobs` it returns
        (tokens, None) or (tokens, (rows, lp, ids)) for the rows whose parameters ask for
        log-probabilities: lp float32 [n, 1 + N], ids int32 [n, N] on the device, N the largest
        `top_logprobs` among them (`ops.logprobs`)."""
        drawn, logits = self._draw(logits, params, seeds, indices, histories)
        if not logprobs:
            return drawn
        rows = [r for r, p in enumerate(params) if p.logprobs]
        if not rows:
            return drawn, None
        R = len(params)
        n_top = max(params[r].top_logprobs for r in rows)
        buf, ints, done = self._staging(R)
        done.synchronize()
        buf.numpy()[0, :R] = [p.temperature for p in params]
        ia = ints.numpy()
        ia[1, :R] = [p.top_k for p in params]
        ia[2, :len(rows)] = rows
        lp, ids = self.backend.logprobs(logits, buf[0, :R], ints[1, :R] if any(p.top_k > 0 for p in params) else None,
                                        drawn, ints[2, :len(rows)], n_top)
        done.record()
        return drawn, (rows, lp, ids)

    def _draw(self, logits, params, seeds, indices, histories):
        """The drawn tokens and the logits they were drawn from (after penalties and bias)."""
        R = logits.shape[0]
        assert R == len(params) == len(seeds) == len(indices)
        if any(p.has_penalties or p.logit_bias for p in params):
            logits = self._adjust(logits, params, histories)
        be = self.backend
        if all(p.greedy for p in params):
            return be.argmax(logits), logits
        # The rows' parameters go into pinned host memory that the kernel reads itself: nothing is
        # copied, so nothing waits for the stream (steps are launched ahead of the host). Four
        # buffers take turns; one is written again only after the kernel that read it has run.
        buf, ints, done = self._staging(R)
        done.synchronize()
        a = buf.numpy()
        a[0, :R] = [p.temperature if not p.greedy else 0.0 for p in params]
        a[1, :R] = [uniform(s, i) for s, i in zip(seeds, indices)]
        top_k = top_p = min_p = None
        if any(p.top_k > 0 for p in params):
            ints.numpy()[2, :R] = [p.top_k for p in params]
            top_k = ints[2, :R]
        if any(p.top_p < 1.0 for p in params):
            a[3, :R] = [p.top_p for p in params]
            top_p = buf[3, :R]
        if any(p.min_p > 0.0 for p in params):
            a[4, :R] = [p.min_p for p in params]
            min_p = buf[4, :R]
        # greedy rows beside drawn ones: argmax of every row first; the draw skips rows of temperature 0
        out = be.argmax(logits) if any(p.greedy for p in params) else None
        drawn = be.sample(logits, buf[0, :R], buf[1, :R], top_k, top_p, min_p, out=out)
        done.record()
        return drawn, logits

    def _staging(self, R: int):
        """The next of four pinned parameter buffers [5, rows] (float32, and the same memory seen as
        int32 for top-k), with the event that tells when its last reader has run."""
        if not self._ring or self._ring[0][0].shape[1] < R:
            cap = max(64, 1 << (R - 1).bit_length())
            for _, _, done in self._ring:        # a kernel may still be reading the buffers that go
                done.synchronize()
            self._ring = []
            for _ in range(4):
                buf = torch.zeros((5, cap), dtype=torch.float32).pin_memory()
                self._ring.append((buf, buf.view(torch.int32), torch.cuda.Event()))
        self._turn = (self._turn + 1) % len(self._ring)
        return self._ring[self._turn]

    def _adjust(self, logits, params, histories):
        """logit[token] -= frequency_penalty * count + presence_penalty for tokens already
        generated, then logit[token] += logit_bias[token] (src/model/sampler.rs:341-358). A
        handful of entries per row: host-computed values added into a copy of the logits by a
        small kernel."""
        V = logits.shape[1]
        rows, cols, vals = [], [], []
        for r, (p, hist) in enumerate(zip(params, histories or [[]] * len(params))):
            delta: dict[int, float] = {}
            if p.has_penalties and hist:
                counts: dict[int, int] = {}
                for t in hist:
                    counts[t] = counts.get(t, 0) + 1
                for t, c in counts.items():
                    if t < V:
                        delta[t] = -(p.frequency_penalty * c + p.presence_penalty)
            for t, b in p.logit_bias:
                if t < V:
                    delta[t] = delta.get(t, 0.0) + b
            for t, d in delta.items():
                rows.append(r); cols.append(t); vals.append(d)
        if not rows:
            return logits
        out = logits.clone()
        n = len(rows)
        lists = torch.empty((3, n), dtype=torch.int32).pin_memory()     # read by the kernel; kept until it has run
        a = lists.numpy()
        a[0], a[1] = rows, cols
        lists[2].view(torch.float32).numpy()[:] = vals
        self.backend.add_at(out, lists[0], lists[1], lists[2].view(torch.float32))
        done = torch.cuda.Event()
        done.record()
        self._held = [(l, e) for l, e in self._held if not e.query()] + [(lists, done)]
        return out
