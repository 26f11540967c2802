"""Helpers shared by the engine tests: requests, the plain implementation's logits, and the three ways of
cutting requests into steps (whole; last tokens one by one; unequal batches one after another)."""
from __future__ import annotations

import functools
import json

import numpy as np

import plain_llama as P


def make_requests(vocab, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return {f"r{i}": [int(t) for t in rng.integers(0, vocab, n)] for i, n in enumerate(lengths)}


@functools.lru_cache(maxsize=None)
def _plain_cached(folder, tokens):
    cfg, w = P.read_model(folder)
    return P.forward_logits(cfg, w, list(tokens))


def plain_logits(folder, requests):
    return {rid: _plain_cached(folder, tuple(toks)) for rid, toks in requests.items()}


def steps_whole(requests):
    """Each request alone and whole, one after another."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}],
                      "end": [rid]})
    return steps


def steps_tail_one_by_one(requests, tail=32):
    """Each request alone: all but the last `tail` tokens in one step, then one token per step."""
    steps = []
    for rid, toks in requests.items():
        k = min(tail, len(toks) - 1)
        head = toks[: len(toks) - k]
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": head, "want": list(range(len(head)))}],
                      "end": [rid] if k == 0 else []})
        for j in range(len(head), len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[j]], "want": [0]}],
                          "end": [rid] if j == len(toks) - 1 else []})
    return steps


def steps_unequal_batches(requests, batch=3, tails=(3, 11, 6, 1, 8, 2)):
    """Batches of `batch` requests that start together: prompts (all but a request's tail) in one step, then one
    token each; requests with short tails end earlier; the next batch starts when the last has ended."""
    steps = []
    ids = list(requests)
    for b0 in range(0, len(ids), batch):
        group = ids[b0: b0 + batch]
        tail = {rid: min(tails[(b0 + i) % len(tails)], len(requests[rid]) - 1) for i, rid in enumerate(group)}
        head = {rid: len(requests[rid]) - tail[rid] for rid in group}
        ends = [rid for rid in group if tail[rid] == 0]
        steps.append({"step": len(steps), "end": ends,
                      "entries": [{"id": rid, "tokens": requests[rid][: head[rid]], "want": list(range(head[rid]))}
                                  for rid in group]})
        for j in range(max(tail.values())):
            live = [rid for rid in group if j < tail[rid]]
            steps.append({"step": len(steps), "end": [rid for rid in live if j == tail[rid] - 1],
                          "entries": [{"id": rid, "tokens": [requests[rid][head[rid] + j]], "want": [0]} for rid in live]})
    return steps


def steps_sparse_wants(requests, batch=3, tails=(3, 11, 6, 1, 8, 2)):
    """The batches of steps_unequal_batches, asking for few logits: none at all from the prompts' step, and from the
    decode steps only every other request's, so that some steps want nothing and others mix entries that do and do not."""
    steps = steps_unequal_batches(requests, batch, tails)
    first_of = {}
    for st in steps:
        for i, e in enumerate(st["entries"]):
            if e["id"] not in first_of:
                first_of[e["id"]] = st["step"]
                e["want"] = []                                    # the prompt
            elif (st["step"] + i) % 2:
                e["want"] = []
    return steps


def expected_rows(steps, requests, plain):
    """For every step with wanted places: the plain logits rows in the order trace replay writes them."""
    fed = {rid: 0 for rid in requests}
    out = {}
    for st in steps:
        rows = []
        for e in st["entries"]:
            base = fed[e["id"]]
            for w in e["want"]:
                rows.append(plain[e["id"]][base + w])
            fed[e["id"]] += len(e["tokens"])
        if rows:
            out[st["step"]] = np.stack(rows)
    return out


def run_steps_in_process(engine, steps):
    """Drive an Engine with the trace-replay step records; returns {step: logits as numpy}."""
    from velomind_b200 import Entry
    slots, out = {}, {}
    for st in steps:
        entries = []
        for e in st["entries"]:
            if e["id"] not in slots:
                slots[e["id"]] = engine.open()
            entries.append(Entry(slots[e["id"]], e["tokens"], e["want"]))
        logits = engine.step(entries)
        if logits.shape[0]:
            out[st["step"]] = logits.float().cpu().numpy().copy()
        for rid in st["end"]:
            engine.close(slots.pop(rid))
    engine.raise_if_error()
    engine.cache.check()
    return out


def to_jsonl(steps):
    return "".join(json.dumps(s) + "\n" for s in steps)
