"""The generation loop: batches of unequal prompts, stop tokens, sequences that end early, batch after batch.

The reference generates one sequence: prefill, sample, then feed each token
back until `max_new_tokens` or the end-of-sequence token, which is kept in the
output and not fed (examples/common/llama/llama_engine.cpp:633-653;
`max_new_tokens == 0` returns after the prompt, :635-637).  The same rules
hold here for every sequence of a batch; a sequence that ends leaves the batch
at once and its slot and pages go back to the cache; requests that did not fit
into one batch run in the next.

The loop only needs `open() / close(slot) / step(entries) -> logits` and a
sampler, so its decisions can be tested without a GPU.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field
from typing import Callable, List, Optional, Sequence

from ..cache.pages import PAGE_TOKENS
from ..sampling.sampler import SamplingParams
from .step import Entry


@dataclass
class Request:
    prompt: Sequence[int]
    params: SamplingParams = SamplingParams()
    stream: int = 0                      # Philox stream of this request (its index, by default)


@dataclass
class Result:
    """What the reference returns per call (llama_engine.h:32-38), per sequence."""
    tokens: List[int] = field(default_factory=list)
    finish_reason: str = ""              # "stop" (a stop token, kept in `tokens`), "length", "empty"
    prompt_tokens: int = 0
    text: str = ""                       # the tokens as text (filled where a tokenizer is at hand; "[id]" pieces without one)
    elapsed_seconds: float = 0.0         # of the whole call that produced it (prompts and decoding of every batch)
    tokens_per_second: float = 0.0       # this sequence's tokens over that time


@dataclass
class Timing:
    prefill_seconds: float = 0.0
    decode_seconds: float = 0.0
    decode_steps: int = 0
    generated_tokens: int = 0

    @property
    def tokens_per_second(self) -> float:
        total = self.prefill_seconds + self.decode_seconds
        return self.generated_tokens / total if total > 0 else 0.0


def pages_for(request: Request) -> int:
    """Pages a request may come to hold: prompt plus every token it may feed back."""
    most = len(request.prompt) + max(request.params.max_tokens - 1, 0)
    return -(-max(most, 1) // PAGE_TOKENS)


def plan_batches(requests: Sequence[Request], total_pages: int, max_batch: int) -> List[List[int]]:
    """Cut the request list, in order, into batches that fit the cache (by pages) and `max_batch` slots.
    Raises ValueError for a request that cannot fit even alone."""
    batches: List[List[int]] = []
    cur: List[int] = []
    used = 0
    for i, r in enumerate(requests):
        need = pages_for(r)
        if need > total_pages:
            raise ValueError(f"request {i} may reach {need * PAGE_TOKENS} cached tokens; the cache holds {total_pages * PAGE_TOKENS}")
        if cur and (used + need > total_pages or len(cur) >= max_batch):
            batches.append(cur)
            cur, used = [], 0
        cur.append(i)
        used += need
    if cur:
        batches.append(cur)
    return batches


class GenerationLoop:
    """Runs requests through a stepper (`open`, `close`, `step`) with a sampler
    (`sample(logits, params, streams, steps) -> token per row`)."""

    def __init__(self, stepper, sampler, total_pages: int, max_batch: int, default_stop: Sequence[int] = (),
                 steps_per_sync: int = 1):
        self.stepper = stepper
        self.sampler = sampler
        # > 1: decode steps are queued in runs of up to this many, their tokens fed back on the device, and the host
        # looks at the tokens once per run (the stepper needs `decode_many`); a sequence that ends inside a run costs
        # the run's remaining steps for that sequence, nothing else
        self.steps_per_sync = max(1, int(steps_per_sync))
        self.total_pages = int(total_pages)
        self.max_batch = int(max_batch)
        self.default_stop = tuple(default_stop)
        self.timing = Timing()

    def run(self, requests: Sequence[Request],
            on_token: Optional[Callable[[int, int], None]] = None) -> List[Result]:
        """Generate for every request; `on_token(request_index, token)` is called as tokens appear."""
        requests = list(requests)
        results = [Result(prompt_tokens=len(r.prompt)) for r in requests]
        self.timing = Timing()
        for batch in plan_batches(requests, self.total_pages, self.max_batch):
            self._run_batch(requests, batch, results, on_token)
        return results

    def _run_length(self, requests, results, live, step_no) -> int:
        """How many decode steps to queue before looking at the tokens: 1 for the prompts' step, for steppers without
        `decode_many`, and when steps_per_sync is 1; never beyond what the sequence closest to its budget may still take."""
        if step_no == 0 or self.steps_per_sync <= 1 or not hasattr(self.stepper, "decode_many"):
            return 1
        room = min(requests[i].params.max_tokens - len(results[i].tokens) for i, _ in live)
        limit = getattr(self.stepper, "MAX_DECODE_RUN", self.steps_per_sync)
        return max(1, min(self.steps_per_sync, room, limit))

    def _run_batch(self, requests, batch, results, on_token) -> None:
        stepper = self.stepper
        live = []                        # (request index, slot)
        for i in batch:
            r = requests[i]
            if r.params.max_tokens <= 0:
                results[i].finish_reason = "length"      # llama_engine.cpp:635-637: nothing to generate
                continue
            if len(r.prompt) == 0:
                results[i].finish_reason = "empty"
                continue
            live.append((i, stepper.open()))
        try:
            t0 = time.perf_counter()
            feed = {i: list(requests[i].prompt) for i, _ in live}
            step_no = 0
            timing, default_stop = self.timing, self.default_stop
            # what the batch's live sequences bring to every step, kept while none of them ends
            live_params = [requests[i].params for i, _ in live]
            live_streams = [requests[i].stream for i, _ in live]
            live_tokens = [results[i].tokens for i, _ in live]
            while live:
                run = self._run_length(requests, results, live, step_no)
                drawn = [len(t) for t in live_tokens]
                if run > 1:
                    rows = stepper.decode_many([slot for _, slot in live], [feed[i][0] for i, _ in live], live_params,
                                               live_streams, drawn, run)
                else:
                    entries = [Entry(slot, feed[i], [len(feed[i]) - 1]) for i, slot in live]
                    logits = stepper.step(entries)
                    rows = [self.sampler.sample(logits, live_params, live_streams, drawn)]
                now = time.perf_counter()
                if step_no == 0:
                    timing.prefill_seconds += now - t0
                else:
                    timing.decode_seconds += now - t0
                    timing.decode_steps += len(rows)
                t0 = now
                ended = set()
                for tokens in rows:                      # one row of tokens per step of the run
                    tokens = tokens.tolist() if hasattr(tokens, "tolist") else tokens
                    for (i, slot), par, out, tok in zip(live, live_params, live_tokens, tokens):
                        if i in ended:
                            continue                     # the sequence ended earlier in this run: the rest is not its output
                        tok = int(tok)
                        out.append(tok)
                        timing.generated_tokens += 1
                        if on_token is not None:
                            on_token(i, tok)
                        reason = ""
                        if tok in (par.stop_tokens or default_stop):
                            reason = "stop"
                        elif len(out) >= par.max_tokens:
                            reason = "length"
                        elif tok < 0:
                            reason = "error"
                        if reason:
                            results[i].finish_reason = reason
                            ended.add(i)
                        else:
                            feed[i] = [tok]
                if ended:
                    still = []
                    for (i, slot) in live:
                        if i in ended:
                            stepper.close(slot)          # the slot and its pages are free for the next batch at once
                        else:
                            still.append((i, slot))
                    live = still
                    live_params = [requests[i].params for i, _ in live]
                    live_streams = [requests[i].stream for i, _ in live]
                    live_tokens = [results[i].tokens for i, _ in live]
                step_no += len(rows)
        except Exception:
            for _, slot in live:
                try:
                    stepper.close(slot)
                except Exception:
                    pass
            raise
