"""The cache's bookkeeping, the activation arena, the step function's host side (with the kernels replaced by
CPU stand-ins) and the generation loop's decisions."""
import random

import numpy as np
import pytest
import torch

import plain_llama as P
import schedules as S
from tiny_configs import TINY_A, TINY_B
from velomind_b200.cache import PAGE_TOKENS, CacheError, CacheNeed, FreeList, SequenceCache
from velomind_b200.engine.arena import Workspace, plan_arena
from velomind_b200.engine.generate import GenerationLoop, Request, pages_for, plan_batches
from velomind_b200.sampling import SamplingParams


# ------------------------------------------------------------------------------------------ free list
def test_free_list_never_loses_or_doubles():
    fl = FreeList(5, "thing")
    got = [fl.take() for _ in range(5)]
    assert got == [0, 1, 2, 3, 4] and fl.free_count == 0
    with pytest.raises(CacheError, match="out of things"):
        fl.take()
    fl.give(3); fl.give(1)
    with pytest.raises(CacheError, match="freed twice"):
        fl.give(3)
    with pytest.raises(CacheError, match="does not exist"):
        fl.give(9)
    assert fl.take() == 1 and fl.take() == 3          # lowest first: what a batch gave back is used again
    fl.check()
    rnd = random.Random(0)
    held = set(range(5))
    for _ in range(2000):
        if held and rnd.random() < 0.5:
            i = rnd.choice(sorted(held)); held.remove(i); fl.give(i)
        elif len(held) < 5:
            i = fl.take(); assert i not in held; held.add(i)
        fl.check()
        assert fl.held_count == len(held)


def _cache(needs, max_tokens=64 * 8, shares=None, **kw):
    shares = shares or [None] * len(needs)
    return SequenceCache(needs, shares, max_tokens, 1024, torch.float32, "cpu", **kw)


def test_slots_and_pages_come_back():
    need = CacheNeed("all", 2, 16)
    c = _cache([need, need], max_slots=3)
    assert len(c.groups) == 1 and c.groups[0].k.shape == (2, 8, 2, PAGE_TOKENS, 16)
    a, b = c.open(), c.open()
    c.reserve(a, 65); c.commit(a, 65)
    c.reserve(b, 64); c.commit(b, 64)
    assert c.groups[0].pages.held_count == 3 and c.tokens_held() == 192
    c.reserve(a, 66); c.commit(a, 66)                          # same page
    assert c.groups[0].pages.held_count == 3
    c.check()
    with pytest.raises(CacheError, match="out of cache pages"):
        c.reserve(b, 64 * 7)
    assert c.groups[0].pages.held_count == 3                   # a refused reservation changes nothing
    c.close(a)
    with pytest.raises(CacheError, match="not open"):
        c.close(a)
    with pytest.raises(CacheError, match="not open"):
        c.reserve(a, 1)
    assert c.groups[0].pages.held_count == 1
    a2 = c.open()
    assert a2 == a and c.length[a2] == 0                        # the slot is used again, empty
    c.reserve(a2, 1)
    assert int(c.groups[0].block_table[a2, 0]) in (0, 1)       # and so are its pages
    c.close(a2); c.close(b)
    c.check()
    assert c.slots.held_count == 0 and c.tokens_held() == 0
    with pytest.raises(CacheError, match="model's limit"):
        s = c.open(); c.reserve(s, 2000)


def test_groups_with_different_needs_have_their_own_storage():
    full, win = CacheNeed("all", 2, 16), CacheNeed("window", 1, 32, window=70)
    c = _cache([full, win, full, None, CacheNeed("none", state_floats=5)], shares=[None, None, None, 1, None], max_tokens=64 * 16)
    assert len(c.groups) == 2
    assert c.where(0) == (0, 0) and c.where(2) == (0, 1) and c.where(1) == (1, 0) and c.where(3) == (1, 0) and c.where(4) is None
    assert c.groups[0].k.shape[2:] == (2, 64, 16) and c.groups[1].k.shape[2:] == (1, 64, 32)
    assert c.state[4].shape == (c.max_slots, 5) and c.state[0] is None
    s = c.open()
    c.state[4][s] = 7.0
    c.reserve(s, 300); c.commit(s, 300)
    assert c.groups[0].pages.held_count == 5
    # window 70: the next query (position 300) sees keys 231..300, so blocks 0..2 (keys < 192) are gone
    assert c.groups[1].pages.held_count == 2 and c.groups[1].blocks_begin[s] == 3
    assert list(c.groups[1].block_table[s, :3]) == [-1, -1, -1]
    c.check()
    c.close(s)
    s2 = c.open()
    assert s2 == s and float(c.state[4][s2].abs().sum()) == 0.0    # state is cleared for the next sequence
    c.close(s2)
    c.check()


# ------------------------------------------------------------------------------------------ arena
def test_arena_plan_packs_by_liveness():
    # a and b overlap in time, c lives after a died: c reuses a's bytes
    plan = plan_arena([(1000, 1, 4), (500, 2, 6), (900, 5, 8)])
    assert plan.peak_bytes == 1024 + 512 and plan.buffer_count == 3 and plan.reused_count >= 1
    for i, (oi, si) in enumerate(zip(plan.offsets, plan.sizes)):
        assert oi % 256 == 0
    ivs = [(int(random.Random(i).randrange(1, 5000)), i, i + random.Random(i + 7).randrange(0, 6)) for i in range(40)]
    plan = plan_arena(ivs)
    for i in range(40):
        for j in range(i):
            overlap_t = not (ivs[i][2] < ivs[j][1] or ivs[j][2] < ivs[i][1])
            overlap_m = plan.offsets[i] < plan.offsets[j] + plan.sizes[j] and plan.offsets[j] < plan.offsets[i] + plan.sizes[i]
            assert not (overlap_t and overlap_m)
    assert plan.bytes_saved == sum(plan.sizes) - plan.peak_bytes > 0


def test_workspace_records_then_replays():
    ws = Workspace("cpu")
    for round_ in range(3):
        ws.begin("k")
        a = ws.take((10, 8), torch.float32); b = ws.take((4,), torch.bfloat16)
        ws.give(a)
        c = ws.take((10, 8), torch.float32)
        if round_:
            assert c.data_ptr() == a.data_ptr()              # planned: c lies where a lay
            assert a.data_ptr() >= ws.arena.data_ptr()
        ws.give(b); ws.give(c)
        with pytest.raises(RuntimeError, match="given twice"):
            ws.give(c)
        ws.end()
    assert ws.plans["k"].buffer_count == 3 and ws.generation == 1
    ws.begin("k")
    with pytest.raises(RuntimeError, match="other buffers"):
        ws.take((100, 8), torch.float32)
    ws.abort()


# ------------------------------------------------------------------------------------------ step function, host side
@pytest.mark.parametrize("name,cfg", [("tiny_a", TINY_A), ("tiny_b", TINY_B)])
def test_step_function_with_stand_in_kernels(emulated, model_folders, name, cfg):
    import velomind_b200 as vm
    folder = model_folders[name]
    requests = S.make_requests(cfg["vocab_size"], (5, 70, 2, 130, 65, 1), seed=2)
    plain = S.plain_logits(folder, requests)
    model = vm.load_model(folder, torch.float32, "cpu")
    for cut in (S.steps_whole, S.steps_tail_one_by_one, S.steps_unequal_batches, S.steps_sparse_wants):
        engine = vm.Engine(model, 64 * 6, max_slots=3, max_step_tokens=100)    # 130-token prompts are cut in two
        steps = cut(requests) if cut is not S.steps_tail_one_by_one else cut(requests, tail=4)
        got = S.run_steps_in_process(engine, steps)
        want = S.expected_rows(steps, requests, plain)
        assert set(got) == set(want)
        assert max(float(np.abs(got[k] - want[k]).max()) for k in want) < 5e-6
        assert engine.cache.slots.held_count == 0 and engine.cache.tokens_held() == 0


def test_op_times_bracket_every_launch_and_restore_the_wrappers(emulated, model_folders):
    """The switchable per-operation timer: inside the block every launching function of `ops` is bracketed by two events,
    outside it the functions are the ones they were.  (Stand-in events with a counter as clock: no device here.)"""
    import velomind_b200 as vm
    from velomind_b200.kernels import ops
    from velomind_b200.kernels.optimes import OpTimes

    clock = [0.0]

    class Event:
        def record(self):
            clock[0] += 1.0
            self.at = clock[0]

        def synchronize(self):
            pass

        def elapsed_time(self, other):
            return other.at - self.at

    model = vm.load_model(model_folders["tiny_a"], torch.float32, "cpu")
    engine = vm.Engine(model, 64 * 2, max_slots=1)
    s = engine.open()
    before = {n: getattr(ops, n) for n in ("linear", "add_rmsnorm", "rope_kv_write", "swiglu")}
    with OpTimes(event=Event) as times:
        assert ops.linear is not before["linear"]
        engine.step([vm.Entry(s, [1, 2, 3], [2])])
    assert all(getattr(ops, n) is fn for n, fn in before.items())
    layers = TINY_A["num_hidden_layers"]
    assert times.calls["rope_kv_write"] == layers and times.calls["swiglu"] == layers
    assert times.calls["add_rmsnorm"] == 2 * layers + 1 and times.calls["linear"] == 4 * layers + 1
    assert all(ms > 0 for ms in times.ms.values()) and "operation" in times.table() and "linear" in times.table()
    engine.close(s)


def test_injected_failures_leave_the_engine_usable(emulated, model_folders, monkeypatch):
    """Failures made on the host (never on the device): a step whose N-th scratch buffer is refused raises, holds no
    workspace, and the same step run again gives the right logits; a kernel wrapper told to fail names its op."""
    import velomind_b200 as vm
    from velomind_b200.kernels import ops
    folder = model_folders["tiny_a"]
    tokens = [int(t) for t in np.random.default_rng(6).integers(0, TINY_A["vocab_size"], 40)]
    ref = P.forward_logits(*P.read_model(folder), tokens)
    model = vm.load_model(folder, torch.float32, "cpu")
    engine = vm.Engine(model, 64 * 2, max_slots=2)
    s = engine.open()
    engine.ws.fail_after = 3
    with pytest.raises(RuntimeError, match="injected failure: buffer 3"):
        engine.step([vm.Entry(s, tokens[:30], [29])])
    assert engine.length(s) == 0                                   # nothing was committed
    engine.ws.fail_after = None
    out = engine.step([vm.Entry(s, tokens[:30], [29])])            # the same step again
    assert np.abs(out.numpy()[0] - ref[29]).max() < 5e-6
    engine.ws.fail_after = 2                                       # ... and in a decode step
    with pytest.raises(RuntimeError, match="injected failure"):
        engine.step([vm.Entry(s, [tokens[30]], [0])])
    assert engine.length(s) == 30
    engine.ws.fail_after = None
    out = engine.step([vm.Entry(s, [tokens[30]], [0])])
    assert np.abs(out.numpy()[0] - ref[30]).max() < 5e-6
    engine.close(s)
    engine.cache.check()
    assert engine.cache.tokens_held() == 0
    # the kernel wrappers' own switch: the op of that name raises after its launch
    monkeypatch.setattr(ops, "FAIL_OP", "rope_kv_write")
    ops._check(0, "add_rmsnorm")
    with pytest.raises(ops.KernelError, match="rope_kv_write: injected failure"):
        ops._check(0, "rope_kv_write")


def test_sampler_keeps_its_parameter_block_while_requests_move_on_together(emulated):
    """The device sampler uploads (temperature, top-p, seed, stream, step) per row; while the same requests all move on
    by the same number of draws it leaves the block where it is and hands the kernel the offset.  The draws are the
    same either way, and anything else (other parameters, rows that move on unevenly, other rows) uploads again."""
    from velomind_b200.sampling.sampler import DeviceSampler, SamplingParams
    rng = np.random.default_rng(0)
    V = 50
    params = [SamplingParams(temperature=0.8, top_p=0.9, seed=7), SamplingParams(temperature=1.3, top_p=1.0, seed=9)]
    logits = [torch.from_numpy(rng.standard_normal((2, V)).astype(np.float32)) for _ in range(6)]

    def expected(row, p, stream, step):
        return P.sample_top_p(row.numpy(), p.temperature, p.top_p, P.uniform01(p.seed, stream, step))

    kept = DeviceSampler("cpu")
    for step, lg in enumerate(logits[:4]):                       # steps 0, 1, 2, 3: one upload, then offsets 1, 2, 3
        got = kept.sample(lg, params, [0, 1], [step, step])
        assert list(got) == [expected(lg[r], params[r], r, step) for r in range(2)]
        if step == 0:
            block = kept._uploaded
        assert kept._uploaded is block
    got = kept.sample(logits[4], params, [0, 1], [4, 6])          # the rows move on unevenly: a new upload
    assert kept._uploaded is not block and list(got) == [expected(logits[4][0], params[0], 0, 4), expected(logits[4][1], params[1], 1, 6)]
    block = kept._uploaded
    other = [params[0], SamplingParams(temperature=0.0)]           # other parameters (greedy row): a new upload
    got = kept.sample(logits[5], other, [0, 1], [5, 7])
    assert kept._uploaded is not block and int(got[1]) == int(logits[5][1].argmax())
    got = kept.sample(logits[5][:1], other[:1], [0], [6])          # fewer rows: a new upload
    assert list(got) == [expected(logits[5][0], params[0], 0, 6)]


def test_poisoned_scratch_changes_nothing(emulated, model_folders):
    """With `poison_freed` every scratch buffer is filled with NaN the moment a part gives it back: a part that gave a
    buffer back before its last reader ran, or read one it no longer holds, would show in the logits."""
    import velomind_b200 as vm
    folder = model_folders["tiny_b"]
    requests = S.make_requests(TINY_B["vocab_size"], (5, 70, 2, 33), seed=8)
    plain = S.plain_logits(folder, requests)
    model = vm.load_model(folder, torch.float32, "cpu")
    for cut in (S.steps_whole, S.steps_unequal_batches):
        engine = vm.Engine(model, 64 * 6, max_slots=3, poison_freed=True)
        steps = cut(requests)
        got = S.run_steps_in_process(engine, steps)
        want = S.expected_rows(steps, requests, plain)
        assert max(float(np.abs(got[k] - want[k]).max()) for k in want) < 5e-6
    # the poison itself: a buffer that was given back reads NaN
    ws = engine.ws
    ws.begin(("poison test",))
    t = ws.take((4, 8), torch.float32)
    t.zero_()
    ws.give(t)
    assert torch.isnan(t).all()
    ws.end()


def test_steps_that_want_no_logits(emulated, model_folders):
    """A prompt cut by the caller into steps of which only the last wants logits: the earlier steps return no rows (in
    whichever order steps with and without wanted rows first meet a capacity bucket) and leave the cache as a whole
    prompt does."""
    import velomind_b200 as vm
    folder = model_folders["tiny_a"]
    tokens = [int(t) for t in np.random.default_rng(4).integers(0, TINY_A["vocab_size"], 23)]
    ref = P.forward_logits(*P.read_model(folder), tokens)
    model = vm.load_model(folder, torch.float32, "cpu")
    for first_wants in (False, True):
        engine = vm.Engine(model, 64 * 2, max_slots=2)
        s = engine.open()
        if first_wants:                                            # a step of the same bucket that does want rows comes first
            w = engine.open()
            engine.step([vm.Entry(w, tokens[:9], [8])])
            engine.close(w)
        none = engine.step([vm.Entry(s, tokens[:9], [])])
        assert tuple(none.shape) == (0, TINY_A["vocab_size"])
        assert tuple(engine.step([vm.Entry(s, tokens[9:17], [])]).shape) == (0, TINY_A["vocab_size"])
        assert tuple(engine.step([vm.Entry(s, tokens[17:18], [])]).shape) == (0, TINY_A["vocab_size"])     # one token, nothing wanted
        out = engine.step([vm.Entry(s, tokens[18:], [0, 4])])
        assert np.abs(out.numpy() - ref[[18, 22]]).max() < 5e-6
        engine.close(s)


def test_step_described_ahead_is_dropped_when_a_slot_changes_hands(emulated, model_folders):
    """After a decode step the engine describes the next one ahead of its tokens.  If a sequence of the batch ends and
    another takes its slot and reaches the very same length, what was described ahead is stale (other pages): it has to
    be noticed, whatever the lengths say."""
    import velomind_b200 as vm
    folder = model_folders["tiny_b"]
    V = TINY_B["vocab_size"]
    rng = np.random.default_rng(9)
    a, b, c = ([int(t) for t in rng.integers(0, V, n)] for n in (70, 12, 13))
    weights = P.read_model(folder)
    model = vm.load_model(folder, torch.float32, "cpu")
    engine = vm.Engine(model, 64 * 6, max_slots=3)
    sa, sb, sd = engine.open(), engine.open(), engine.open()
    engine.step([vm.Entry(sa, a[:68], []), vm.Entry(sb, b[:11], [])])
    out = engine.step([vm.Entry(sa, [a[68]], [0]), vm.Entry(sb, [b[11]], [0])])           # lengths now 69 and 12
    assert np.abs(out.numpy() - np.stack([P.forward_logits(*weights, a[:69])[-1], P.forward_logits(*weights, b[:12])[-1]])).max() < 5e-6
    page_of_b = int(engine.cache.groups[0].block_table[sb, 0])
    engine.close(sb)
    engine.step([vm.Entry(sd, a[:5], [])])                                                # a third sequence takes the freed page
    sc = engine.open()
    assert sc == sb                                                                       # the same slot, another sequence
    engine.step([vm.Entry(sc, c[:12], [])])                                               # ... at the same length: 12
    assert int(engine.cache.groups[0].block_table[sc, 0]) != page_of_b                    # ... in another page
    out = engine.step([vm.Entry(sa, [a[69]], [0]), vm.Entry(sc, [c[12]], [0])])
    want = np.stack([P.forward_logits(*weights, a[:70])[-1], P.forward_logits(*weights, c[:13])[-1]])
    assert np.abs(out.numpy() - want).max() < 5e-6
    # and the plain case: the same two sequences go on, from what was described ahead
    a2, c2 = int(rng.integers(0, V)), int(rng.integers(0, V))
    out = engine.step([vm.Entry(sa, [a2], [0]), vm.Entry(sc, [c2], [0])])
    want = np.stack([P.forward_logits(*weights, a[:70] + [a2])[-1], P.forward_logits(*weights, c[:13] + [c2])[-1]])
    assert np.abs(out.numpy() - want).max() < 5e-6
    engine.close(sa); engine.close(sc); engine.close(sd)
    assert engine.cache.tokens_held() == 0


def test_step_refusals(emulated, model_folders):
    import velomind_b200 as vm
    model = vm.load_model(model_folders["tiny_a"], torch.float32, "cpu")
    engine = vm.Engine(model, 128, max_slots=2)
    s = engine.open()
    with pytest.raises(ValueError, match="outside the vocabulary"):
        engine.step([vm.Entry(s, [1, 256], [0])])
    with pytest.raises(ValueError, match="wanted place 2"):
        engine.step([vm.Entry(s, [1, 2], [2])])
    with pytest.raises(ValueError, match="twice"):
        engine.step([vm.Entry(s, [1], []), vm.Entry(s, [2], [])])
    with pytest.raises(CacheError, match="not open"):
        engine.step([vm.Entry(1, [1], [])])
    with pytest.raises(CacheError, match="max_tokens"):
        engine.step([vm.Entry(s, [1] * 129, [])])
    assert engine.length(s) == 0
    out = engine.step([vm.Entry(s, [1, 2, 3], [2, 0])])            # wanted places keep their order
    ref = P.forward_logits(*P.read_model(model_folders["tiny_a"]), [1, 2, 3])
    assert np.abs(out.numpy() - ref[[2, 0]]).max() < 5e-6
    with pytest.raises(CacheError, match="model's limit"):
        engine.step([vm.Entry(s, [1] * 600, [])])
    engine.close(s)


# ------------------------------------------------------------------------------------------ generation loop
class FakeStepper:
    """Logits that make the next token = (last token + 1) % vocab; records what it is asked to do."""

    def __init__(self, vocab=50, slots=4):
        self.vocab, self.free, self.open_slots, self.log, self.closed = vocab, list(range(slots)), set(), [], []

    def open(self):
        s = min(self.free); self.free.remove(s); self.open_slots.add(s); return s

    def close(self, slot):
        assert slot in self.open_slots, "closed twice"
        self.open_slots.remove(slot); self.free.append(slot); self.closed.append(slot)

    def step(self, entries):
        self.log.append([(e.slot, list(e.tokens)) for e in entries])
        out = torch.full((len(entries), self.vocab), -1.0)
        for r, e in enumerate(entries):
            assert e.slot in self.open_slots and list(e.want) == [len(e.tokens) - 1]
            out[r, (e.tokens[-1] + 1) % self.vocab] = 1.0
        return out


class GreedyHostSampler:
    def sample(self, logits, params, streams, steps):
        self.last = (list(streams), list(steps))
        return logits.argmax(-1).numpy()


def test_loop_unequal_prompts_stop_tokens_and_early_ends():
    st, sm = FakeStepper(), GreedyHostSampler()
    loop = GenerationLoop(st, sm, total_pages=100, max_batch=4, default_stop=(13,))
    reqs = [Request([1, 2, 3], SamplingParams(0.0, 0.9, 5)), Request([10], SamplingParams(0.0, 0.9, 9)),
            Request([40, 41], SamplingParams(0.0, 0.9, 2)), Request([7], SamplingParams(0.0, 0.9, 0)),
            Request([], SamplingParams(0.0, 0.9, 4))]
    seen = []
    res = loop.run(reqs, on_token=lambda i, t: seen.append((i, t)))
    assert res[0].tokens == [4, 5, 6, 7, 8] and res[0].finish_reason == "length"
    assert res[1].tokens == [11, 12, 13] and res[1].finish_reason == "stop"        # the stop token is kept, not fed
    assert res[2].tokens == [42, 43] and res[2].finish_reason == "length"
    assert res[3].tokens == [] and res[3].finish_reason == "length"               # max_tokens 0: nothing to do
    assert res[4].finish_reason == "empty"
    assert st.log[0] == [(0, [1, 2, 3]), (1, [10]), (2, [40, 41])]                # prompts whole, in one step
    assert st.log[1] == [(0, [4]), (1, [11]), (2, [42])]                          # then one token each
    assert st.log[2] == [(0, [5]), (1, [12])]                                     # request 2 ended earlier
    assert st.log[3] == [(0, [6])] and len(st.log) == 5                           # 13 was never fed
    assert not st.open_slots and sorted(st.closed) == [0, 1, 2]
    assert [t for i, t in seen if i == 1] == [11, 12, 13]
    assert loop.timing.generated_tokens == 10 and loop.timing.decode_steps == 4
    assert res[0].prompt_tokens == 3


def test_loop_runs_batch_after_batch_and_reuses_slots():
    st, sm = FakeStepper(slots=2), GreedyHostSampler()
    loop = GenerationLoop(st, sm, total_pages=100, max_batch=2)
    reqs = [Request([i], SamplingParams(0.0, 0.9, 2 + i), stream=i) for i in range(5)]
    res = loop.run(reqs)
    assert [r.tokens for r in res] == [[i + 1 + k for k in range(2 + i)] for i in range(5)]
    assert st.closed == [0, 1, 0, 1, 0] or sorted(st.closed) == [0, 0, 0, 1, 1]
    assert [e[0] for e in st.log[0]] == [0, 1] and not st.open_slots
    assert sm.last == ([4], [5])                        # request 4's stream and its own step count


def test_batches_are_cut_by_pages_and_slots():
    reqs = [Request([0] * 100, SamplingParams(max_tokens=29)), Request([0] * 10, SamplingParams(max_tokens=1)),
            Request([0] * 64, SamplingParams(max_tokens=2)), Request([0] * 300, SamplingParams(max_tokens=1))]
    assert [pages_for(r) for r in reqs] == [2, 1, 2, 5]
    assert plan_batches(reqs, total_pages=5, max_batch=8) == [[0, 1, 2], [3]]
    assert plan_batches(reqs, total_pages=100, max_batch=2) == [[0, 1], [2, 3]]
    with pytest.raises(ValueError, match="request 3"):
        plan_batches(reqs, total_pages=4, max_batch=8)


def test_loop_closes_slots_when_a_step_fails():
    class Failing(FakeStepper):
        def step(self, entries):
            if len(self.log) == 1:
                raise RuntimeError("boom")
            return super().step(entries)
    st = Failing()
    loop = GenerationLoop(st, GreedyHostSampler(), 100, 4)
    with pytest.raises(RuntimeError, match="boom"):
        loop.run([Request([1], SamplingParams(0.0, 0.9, 5)), Request([2], SamplingParams(0.0, 0.9, 5))])
    assert not st.open_slots


def test_generation_with_stand_in_kernels_matches_plain(emulated, model_folders):
    import velomind_b200 as vm
    folder = model_folders["tiny_b"]
    cfg, w = P.read_model(folder)
    prompts = [[1, 2, 3, 4, 5, 6, 7], [9, 8, 7, 6]]
    te = vm.TextEngine(vm.EngineConfig(model_path=folder, dtype="float32", device="cpu", max_tokens=512)).load()
    got = te.generate(prompts, temperature=0.8, top_p=0.95, max_tokens=4, seed=5, stop_tokens=())
    want = [P.generate(cfg, w, p, 4, temperature=0.8, top_p=0.95, seed=5, stream=i) for i, p in enumerate(prompts)]
    assert [r.tokens for r in got] == want
    assert got[0].text == "".join(f"[{t}]" for t in want[0]) and got[0].elapsed_seconds > 0 and got[0].tokens_per_second > 0
    pieces = []
    te.generate(prompts[:1], temperature=0.0, max_tokens=2, on_token=lambda i, t, piece: pieces.append(piece))
    assert all(p.startswith("[") for p in pieces)         # no tokenizer: ids in brackets
    logits = te.prefill(prompts[0][:-1])
    step = te.forward_step(prompts[0][-1])
    ref = P.forward_logits(cfg, w, prompts[0])
    assert te.session_length == 7
    assert np.abs(logits.numpy() - ref[-2]).max() < 5e-6 and np.abs(step.numpy() - ref[-1]).max() < 5e-6
    assert np.abs(te.forward_logits(prompts[0]).numpy() - ref[-1]).max() < 5e-6
    assert np.abs(te.forward_full_logits(prompts[0]).numpy() - ref).max() < 5e-6
    te.reset_session()
    assert te.session_length == 0 and te.engine.cache.slots.held_count == 0
    # the reference's own way of sampling: a host function of one row of logits (llama_engine.h:106-121)
    seen = []

    def second_best(row):
        seen.append(row.shape)
        return int(np.argsort(row)[-2])

    got = te.generate([prompts[1]], max_tokens=3, stop_tokens=(), sample_fn=second_best)[0].tokens
    want, ctx = [], list(prompts[1])
    for _ in range(3):
        want.append(int(np.argsort(P.forward_logits(cfg, w, ctx)[-1])[-2]))
        ctx.append(want[-1])
    assert got == want and seen == [(cfg["vocab_size"],)] * 3
    # forward_step with the reference's position argument: only the session's length is a valid place
    te.prefill(prompts[0][:3])
    with pytest.raises(ValueError, match="not the session's length 3"):
        te.forward_step(prompts[0][3], pos=5)
    step = te.forward_step(prompts[0][3], pos=3)
    assert np.abs(step.numpy() - P.forward_logits(cfg, w, prompts[0][:4])[-1]).max() < 5e-6
    te.reset_session()


def test_queued_decode_runs_with_stand_in_kernels_equal_single_steps(emulated, model_folders):
    """`Engine.decode_many` (several decode steps without the host in between, the tokens fed back by the device-side
    kernel's stand-in) against one step at a time and against the plain implementation, greedy and sampled, with a stop
    token that ends one sequence inside a run."""
    import velomind_b200 as vm
    folder = model_folders["tiny_a"]
    cfg, w = P.read_model(folder)
    prompts = [[3, 1, 4, 1, 5, 9, 2, 6], [2, 7], [1] * 62]          # the last one crosses a page while decoding
    te = vm.TextEngine(vm.EngineConfig(model_path=folder, dtype="float32", device="cpu", max_tokens=1024)).load()
    for temperature, top_p in ((0.0, 1.0), (0.9, 0.8)):
        one = te.generate(prompts, temperature=temperature, top_p=top_p, max_tokens=9, seed=3, stop_tokens=(), steps_per_sync=1)
        want = [P.generate(cfg, w, p, 9, temperature=temperature, top_p=top_p, seed=3, stream=i) for i, p in enumerate(prompts)]
        assert [r.tokens for r in one] == want
        stop = want[1][4]                                             # ends the second sequence in the middle of a run
        ref = te.generate(prompts, temperature=temperature, top_p=top_p, max_tokens=9, seed=3, stop_tokens=(stop,), steps_per_sync=1)
        for k in (2, 4, 8):
            got = te.generate(prompts, temperature=temperature, top_p=top_p, max_tokens=9, seed=3, stop_tokens=(stop,), steps_per_sync=k)
            assert [(r.tokens, r.finish_reason) for r in got] == [(r.tokens, r.finish_reason) for r in ref]
    assert te.engine.cache.slots.held_count == 0 and te.engine.cache.tokens_held() == 0


class FakeRunStepper(FakeStepper):
    """FakeStepper that can also queue several decode steps (next token = last + 1, like its logits say)."""
    MAX_DECODE_RUN = 5

    def __init__(self, *a, **kw):
        super().__init__(*a, **kw)
        self.runs = []

    def decode_many(self, slots, last_tokens, params, streams, draw_steps, k):
        assert all(s in self.open_slots for s in slots) and 1 <= k <= self.MAX_DECODE_RUN
        self.runs.append((list(slots), list(last_tokens), list(draw_steps), k))
        return np.array([[(t + 1 + j) % self.vocab for t in last_tokens] for j in range(k)], dtype=np.int32)


def test_loop_with_queued_decode_runs_gives_the_same_tokens():
    reqs = [Request([1, 2, 3], SamplingParams(0.0, 0.9, 9)), Request([10], SamplingParams(0.0, 0.9, 12)),
            Request([40, 41], SamplingParams(0.0, 0.9, 2))]
    base = GenerationLoop(FakeStepper(), GreedyHostSampler(), 100, 4, default_stop=(15,)).run(reqs)
    st = FakeRunStepper()
    loop = GenerationLoop(st, GreedyHostSampler(), 100, 4, default_stop=(15,), steps_per_sync=8)
    got = loop.run(reqs)
    assert [r.tokens for r in got] == [r.tokens for r in base] and [r.finish_reason for r in got] == [r.finish_reason for r in base]
    assert got[1].tokens == [11, 12, 13, 14, 15] and got[1].finish_reason == "stop"     # ended inside a run; the rest is dropped
    # request 2 may take only one more token after the prompts' step, so that step is a single one; then a run of the
    # stepper's cap (5), inside which request 1 stops; then what request 0's budget leaves (2)
    assert [k for *_, k in st.runs] == [5, 2]
    assert st.runs[0][0] == [0, 1] and st.runs[0][2] == [2, 2]      # slots and draw counters of the first run
    assert st.runs[1][0] == [0] and st.runs[1][1] == [10] and st.runs[1][2] == [7]
    assert not st.open_slots
    assert loop.timing.generated_tokens == sum(len(r.tokens) for r in got)
