"""The Python entry point: `LLM` and `generate()`.

Shaped like the reference's commands (src/commands/run.rs, batch.rs): a model folder, a
prompt (token ids; text when the folder has a tokenizer.json and the `tokenizers` package
is importable), `max_tokens` 128, `temperature` 1.0 (0 = greedy), `top_p`. `LLM.step()`
mirrors the reference's `InferenceEngine::step` loop (src/engine/mod.rs:82-117):
`add_request`, `step`, `abort`, `has_work`.
"""
from __future__ import annotations

import os
import warnings

import time

import torch
from dataclasses import dataclass, replace

from .engine.factory import load_engine, parse_dtype, random_engine
from .engine.scheduler import Scheduler, StepOutput
from .sampling import Sampler, SamplingParams


@dataclass
class StepStats:
    """What the steps of an `LLM` have run and where the host's time went, added up since the last
    `reset()`. `host_*_s`: seconds the host spent planning (scheduler), launching (pages, metadata,
    kernel launches, sampling launches) and recording results; `wait_s`: seconds it waited for a
    step's tokens to arrive; `wall_s`: seconds inside `LLM.step`; `device_s`: seconds between the CUDA
    events that bracket each step's launches on the stream (read once the step is over). With a step launched ahead the
    host's work overlaps the device's, so `host_share` says how busy the host is, not how much it
    delays the device. The reference logs tok/s per run (src/commands/run.rs:82-119); this is the
    per-step account behind such a line."""
    steps: int = 0
    tokens: int = 0              # tokens run: prompt portions and decode tokens
    prefill_tokens: int = 0      # of these, tokens of prompt portions
    sampled: int = 0             # tokens drawn
    h2d_bytes: int = 0           # step metadata copied to the device
    kv_positions: int = 0        # sum over entries of the keys visible to the entry's last token
    attn_pairs: int = 0          # (query, key) pairs scored
    preemptions: int = 0
    host_plan_s: float = 0.0
    host_launch_s: float = 0.0
    host_record_s: float = 0.0
    wait_s: float = 0.0
    wall_s: float = 0.0
    device_s: float = 0.0        # seconds the device worked on the steps (CUDA events around each step's launches)

    def reset(self) -> None:
        self.__init__()

    @property
    def host_share(self) -> float:
        """Fraction of the time inside `LLM.step` that the host worked (did not wait for the device)."""
        return (self.host_plan_s + self.host_launch_s + self.host_record_s) / self.wall_s if self.wall_s else 0.0

    def line(self) -> str:
        w = self.wall_s or 1e-30
        return (f"{self.steps} steps, {self.tokens} tokens run ({self.prefill_tokens} of prompts), {self.sampled} drawn, "
                f"{self.sampled / w:.1f} tok/s; per step {w / max(self.steps, 1) * 1e3:.3f} ms of which host "
                f"{self.host_share:.1%} (plan {self.host_plan_s / w:.1%}, launch {self.host_launch_s / w:.1%}, "
                f"record {self.host_record_s / w:.1%}), waiting {self.wait_s / w:.1%}, device busy {self.device_s / w:.1%}; "
                f"{self.h2d_bytes / max(self.steps, 1):.0f} B of metadata a step; {self.preemptions} preemptions")


class LLM:
    """A loaded model with its cache, scheduler and sampler on one GPU."""

    def __init__(self, model: str | dict, dtype="bfloat16", device="cuda:0", seed: int = 0,
                 page_size: int = 16, num_pages: int | None = None, max_active: int = 64,
                 max_tokens_per_step: int = 2048, max_chunk: int | None = None,
                 weight_std: float = 0.02, norm_std: float = 0.0):
        """`model`: a folder with config.json + model.safetensors, or a raw config dict, which
        gets random weights from `seed`."""
        kw = dict(dtype=parse_dtype(dtype), device=device, page_size=page_size, num_pages=num_pages,
                  max_requests=max_active)
        if isinstance(model, dict):
            self.engine = random_engine(model, seed, std=weight_std, norm_std=norm_std, **kw)
            self.model_dir = None
        else:
            self.engine = load_engine(model, **kw)
            self.model_dir = model
        self.scheduler = Scheduler(self.engine.cache, max_active, max_tokens_per_step, max_chunk)
        self.sampler = Sampler(self.engine.backend)
        self._tokenizer = None
        # a step that was launched ahead: (plan, its drawn tokens: device tensor, host copy, event,
        # and the host copies of the log-probabilities where a request asked for them)
        self._ahead = None
        self._pinned = []                        # host buffers the drawn tokens are copied into, in turn
        self._timed = []                         # (begin, end) events of steps whose device time is not added up yet
        self._free_events = []
        self.run_ahead = os.environ.get("RLLM_B200_NO_RUN_AHEAD") != "1"
        self.steps_ahead = 0
        self._warned_positions = False
        self.stats = StepStats()
        self._since_report = 0

    # ---- the reference's engine loop
    def add_request(self, prompt_token_ids: list[int], params: SamplingParams | None = None) -> int:
        """A request ends at the model's own end-of-sequence ids (config.json's `eos_token_id`)
        unless its parameters name others or say `ignore_eos`, as the reference's engine stops
        at its tokenizer's list (src/engine/mod.rs:694-699)."""
        params = params or SamplingParams()
        # positions the configuration does not allow are not run: a prompt that is too long is
        # refused, a generation is cut where the positions end (finish reason "length")
        limit = getattr(self.engine.model.config, "max_position_embeddings", None)
        if limit is not None:
            if len(prompt_token_ids) >= limit:
                raise ValueError(f"the prompt has {len(prompt_token_ids)} tokens, the model's "
                                 f"max_position_embeddings is {limit}")
            if len(prompt_token_ids) + params.max_tokens > limit:
                if not self._warned_positions:
                    self._warned_positions = True
                    warnings.warn(f"prompt + max_tokens exceeds max_position_embeddings {limit}: "
                                  f"the generation is cut there", stacklevel=2)
                params = replace(params, max_tokens=limit - len(prompt_token_ids))
        eos = getattr(self.engine.model.config, "eos_token_ids", ())
        if eos and not params.eos_token_ids and not params.ignore_eos:
            params = replace(params, eos_token_ids=tuple(eos))
        return self.scheduler.add_request(prompt_token_ids, params)

    def abort(self, request_id: int) -> bool:
        return self.scheduler.abort(request_id, self.engine)

    def has_work(self) -> bool:
        return self.scheduler.has_work()

    def _launch(self, plan, feed=None, ahead: int = 0):
        """Run the plan's batch and draw its tokens. Returns None when nothing is sampled, else
        (tokens on the device, their pinned host copy, the event after which that copy is
        complete, log-probabilities on their way to the host or None).
        `ahead`: how many tokens each request is about to get that its `output` lacks."""
        st = self.stats
        for p in plan:
            q, start = len(p.tokens), p.request.num_stored + ahead
            st.tokens += q
            st.prefill_tokens += q if q > 1 or not p.request.decoding else 0
            st.kv_positions += start + q
            st.attn_pairs += q * start + q * (q + 1) // 2
        h2d0 = self.engine.h2d_bytes
        begin, end = self._event_pair()
        begin.record()
        logits = self.engine.step(self.scheduler.entries(plan), keep=False, feed=feed)
        st.h2d_bytes += self.engine.h2d_bytes - h2d0
        sampled = [p.request for p in plan if p.samples]
        if not sampled:
            end.record()
            self._timed.append((begin, end))
            return None
        drawn, lps = self.sampler.draw(logits, [r.params for r in sampled], [r.seed for r in sampled],
                                       [len(r.output) + ahead for r in sampled], [r.output for r in sampled],
                                       logprobs=True)
        # Their way to the host goes over a stream of its own, which waits for the draw only: the
        # step launched behind them on the main stream does not wait for a copy engine.
        if not self._pinned:
            n = max(self.scheduler.max_active, 1)
            self._pinned = [torch.zeros(n + 4, dtype=torch.int32).pin_memory() for _ in range(2)]
            self._copy_stream = torch.cuda.Stream(self.engine.device)
        self._pinned.reverse()
        buf = self._pinned[0]
        host = buf[: drawn.numel()]
        drawn_at = torch.cuda.Event()
        drawn_at.record()
        end.record()
        self._timed.append((begin, end))
        arrived = torch.cuda.Event()
        lp_host = None
        with torch.cuda.stream(self._copy_stream):
            self._copy_stream.wait_event(drawn_at)
            host.copy_(drawn, non_blocking=True)
            buf[-4:].copy_(self.engine.error_words, non_blocking=True)      # and the device's error words with them
            if lps is not None:                  # log-probabilities were asked for: they travel with the tokens
                rows, lp, ids = lps
                lp_host = (rows, torch.empty(lp.shape, dtype=lp.dtype).pin_memory(),
                           torch.empty(ids.shape, dtype=ids.dtype).pin_memory())
                lp_host[1].copy_(lp, non_blocking=True)
                lp_host[2].copy_(ids, non_blocking=True)
                lp.record_stream(self._copy_stream)
                ids.record_stream(self._copy_stream)
            arrived.record()
        return drawn, host, arrived, lp_host

    def _event_pair(self):
        return self._free_events.pop() if self._free_events else (torch.cuda.Event(enable_timing=True),
                                                                  torch.cuda.Event(enable_timing=True))

    def _settle_device_time(self) -> None:
        """Adds up the device time of the steps that are over (their end events have passed)."""
        while self._timed and self._timed[0][1].query():
            begin, end = self._timed.pop(0)
            self.stats.device_s += begin.elapsed_time(end) * 1e-3
            self._free_events.append((begin, end))

    def step(self) -> list[StepOutput]:
        """One scheduler step: plan, run the batch, sample, finish and free.

        In the steady state of decoding the step after this one is launched before this one's
        tokens are read (`Scheduler.plan_ahead`): its token ids go from the sampling kernel's
        output into the step's metadata on the device, so the GPU does not wait while the host
        reads the tokens, records them and plans. Each call still returns the tokens of exactly
        one step; a request that met its end token has one unused position computed for it."""
        st, clock = self.stats, time.perf_counter
        t_in = clock()
        plan_s = launch_s = wait_s = 0.0
        failed: list[StepOutput] = []
        if self._ahead is not None:
            plan, drawn = self._ahead
            self._ahead = None
        else:
            t0 = clock()
            pre0 = self.scheduler.preempted_total
            plan, failed = self.scheduler.schedule(self.engine)
            st.preemptions += self.scheduler.preempted_total - pre0
            t1 = clock()
            plan_s += t1 - t0
            if not plan:
                st.host_plan_s += plan_s
                st.wall_s += clock() - t_in
                return failed
            drawn = self._launch(plan)
            launch_s += clock() - t1
        if self.run_ahead and drawn is not None:
            t0 = clock()
            nxt = self.scheduler.plan_ahead(plan)
            t1 = clock()
            plan_s += t1 - t0
            if nxt is not None and self.engine.takes_feed(self.scheduler.entries(nxt)):
                self._ahead = (nxt, self._launch(nxt, feed=drawn[0], ahead=1))
                self.steps_ahead += 1
            launch_s += clock() - t1
        tokens, logprobs = [], None
        if drawn is not None:
            t0 = clock()
            drawn[2].synchronize()               # this step's tokens only; the step ahead keeps running
            wait_s = clock() - t0
            tokens = drawn[1].tolist()
            if drawn[3] is not None:
                logprobs = self._logprobs(plan, *drawn[3])
            if self._pinned[0][-4:].any() or self._pinned[1][-4:].any():
                self._ahead = None
                self.engine.check()              # raises: a kernel gave up waiting, or a token id was out of range
        self._settle_device_time()
        outs = failed + self.scheduler.advance(plan, tokens, self.engine, logprobs)
        if self._ahead is not None and all(p.request.finished for p in self._ahead[0]):
            self._ahead = None                   # nobody is left to take its tokens
        wall = clock() - t_in
        st.steps += 1
        st.sampled += len(tokens)
        st.host_plan_s += plan_s
        st.host_launch_s += launch_s
        st.wait_s += wait_s
        st.wall_s += wall
        st.host_record_s += wall - plan_s - launch_s - wait_s
        prof = getattr(self.engine.backend, "report", None)
        if prof is not None:                     # RLLM_B200_PROFILE=1: the per-operation table every 256 tokens drawn
            self._since_report += len(tokens)
            if self._since_report >= 256:
                self._since_report = 0
                prof()
        return outs

    @staticmethod
    def _logprobs(plan, rows, lp, ids) -> dict:
        """{index among the step's sampled requests: (ln p of its token, [(token, ln p), ...])}, each
        list cut to the request's own `top_logprobs` and to the tokens that exist."""
        sampled = [p.request for p in plan if p.samples]
        lp, ids = lp.tolist(), ids.tolist()
        out = {}
        for i, r in enumerate(rows):
            n = sampled[r].params.top_logprobs
            out[r] = (lp[i][0], [(t, v) for t, v in zip(ids[i][:n], lp[i][1: 1 + n]) if t >= 0])
        return out

    def warm_up(self, prompt_len: int = 2048) -> None:
        """Run a throw-away request (a prompt portion as long as the token budget allows, then a few
        decoded tokens) so that what happens once per process happens now: the kernels' modules
        are loaded, their attributes set, the first decode graph is captured. The first real
        request then costs what every later one costs."""
        vocab = self.engine.vocab
        limit = getattr(self.engine.model.config, "max_position_embeddings", None) or prompt_len + 8
        n = max(1, min(prompt_len, self.scheduler.max_tokens_per_step, limit - 8,
                       (min(self.engine.cache.free_pages()) - 1) * self.engine.cache.page_size - 8))
        prompt = [(7 * i + 1) % vocab for i in range(n)]
        self.generate([prompt], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
        self.generate([prompt[:5]], SamplingParams(temperature=0.8, top_p=0.9, max_tokens=2, ignore_eos=True, seed=0))

    # ---- whole generations
    def generate(self, prompts, params: SamplingParams | list[SamplingParams] | None = None,
                 details: bool = False, **overrides):
        """Token ids in, generated token ids out, one list per prompt (all prompts run
        concurrently, as `rllm batch` does). With `details` the requests themselves come back
        (`output`, `logprobs`, `finish_reason`, `preemptions`)."""
        if prompts and isinstance(prompts[0], int):
            prompts = [prompts]
        base = params or SamplingParams()
        plist = base if isinstance(base, list) else [base] * len(prompts)
        if overrides:
            plist = [replace(p, **overrides) for p in plist]
        ids = [self.add_request(list(p), sp) for p, sp in zip(prompts, plist)]
        while self.has_work():
            self.step()
        self.engine.check()
        reqs = [self.scheduler.requests.pop(i) for i in ids]
        return reqs if details else [r.output for r in reqs]

    # ---- optional text I/O
    def tokenizer(self):
        if self._tokenizer is None:
            path = os.path.join(self.model_dir or "", "tokenizer.json")
            if not self.model_dir or not os.path.isfile(path):
                raise RuntimeError("no tokenizer.json in the model folder: pass token ids")
            try:
                from tokenizers import Tokenizer
            except ImportError as e:
                raise RuntimeError("text prompts need the `tokenizers` package") from e
            self._tokenizer = Tokenizer.from_file(path)
        return self._tokenizer


def generate(model: str | dict, prompts, max_tokens: int = 128, temperature: float = 1.0,
             top_p: float = 1.0, top_k: int = 0, min_p: float = 0.0, seed: int | None = None,
             dtype="bfloat16", **engine_opts) -> list[list[int]]:
    """Load `model`, generate for every prompt (lists of token ids), return the new ids."""
    llm = LLM(model, dtype=dtype, **engine_opts)
    sp = SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p,
                        max_tokens=max_tokens, seed=seed)
    return llm.generate(prompts, sp)
