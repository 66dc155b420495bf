"""The generation loop's decisions, on the CPU with a scripted backend: which sequences run in which
step, stop tokens, sequences that end earlier, what is yielded, when slots are given back, and how
requests are cut into batches."""

import pytest

from dryft_b200.engine.loop import ENDED, plan_batches, run_batch, run_requests
from dryft_b200.sampling.sampler import SamplingParams


class Scripted:
    """Sequence ``i`` emits script[i][0], script[i][1], ...; records every call."""

    def __init__(self, script, n_slots=8):
        self.script = script
        self.free = list(range(n_slots))
        self.calls = []
        self.pos = {}
        self.owner = {}

    def open(self, n):
        assert n <= len(self.free), "loop asked for more slots than exist"
        h = [self.free.pop(0) for _ in range(n)]
        self.calls.append(("open", tuple(h)))
        return h

    def prefill(self, handles, prompts, seq_ids, params):
        self.calls.append(("prefill", tuple(handles), tuple(len(p) for p in prompts), tuple(seq_ids)))
        out = []
        for h, s in zip(handles, seq_ids):
            self.owner[h] = s
            self.pos[h] = 1
            out.append(self.script[s][0])
        return out

    def decode(self, handles, seq_ids, step, params):
        self.calls.append(("decode", tuple(handles), tuple(seq_ids), step))
        out = []
        for h, s in zip(handles, seq_ids):
            assert self.owner[h] == s and self.pos[h] == step
            out.append(self.script[s][self.pos[h]])
            self.pos[h] += 1
        return out

    def close(self, handles):
        self.calls.append(("close", tuple(handles)))
        for h in handles:
            assert h not in self.free, "slot freed twice"
            self.free.append(h)
        self.free.sort()


GREEDY = SamplingParams()


def test_every_sequence_yields_max_new_tokens_without_stops():
    be = Scripted({0: [10, 11, 12], 1: [20, 21, 22]})
    out = list(run_batch(be, [[1, 2, 3], [4]], 3, GREEDY))
    assert out == [[10, 20], [11, 21], [12, 22]]
    kinds = [c[0] for c in be.calls]
    assert kinds == ["open", "prefill", "decode", "decode", "close"]
    assert be.calls[1][2] == (3, 1)  # unequal prompts in ONE step
    assert be.free == list(range(8))


def test_stop_token_is_yielded_then_the_sequence_is_left_out():
    be = Scripted({0: [5, 99, 7, 8], 1: [6, 6, 6, 6], 2: [99, 1, 1, 1]})
    out = list(run_batch(be, [[1], [2], [3]], 4, GREEDY, stop_token_ids=[99]))
    assert out == [[5, 6, 99], [99, 6, ENDED], [ENDED, 6, ENDED], [ENDED, 6, ENDED]]
    decodes = [c for c in be.calls if c[0] == "decode"]
    assert [c[2] for c in decodes] == [(0, 1), (1,), (1,)]  # who runs in each decode step
    assert [c[3] for c in decodes] == [1, 2, 3]


def test_loop_ends_when_every_sequence_has_ended():
    be = Scripted({0: [1, 99, 0, 0, 0], 1: [99, 0, 0, 0, 0]})
    out = list(run_batch(be, [[1], [2]], 5, GREEDY, stop_token_ids=[99]))
    assert out == [[1, 99], [99, ENDED]]
    assert be.calls[-1][0] == "close" and be.free == list(range(8))


def test_degenerate_requests():
    be = Scripted({0: [1]})
    assert list(run_batch(be, [], 4, GREEDY)) == [] and list(run_batch(be, [[1]], 0, GREEDY)) == []
    assert be.calls == []  # engine/engine.py:142-143: nothing happens
    with pytest.raises(ValueError, match="empty prompt"):
        list(run_batch(be, [[1], []], 2, GREEDY))
    assert be.calls == []  # refused before any slot is taken
    assert list(run_batch(be, [[3]], 1, GREEDY)) == [[1]]
    assert [c[0] for c in be.calls] == ["open", "prefill", "close"]  # max_new_tokens=1: no decode step


def test_slots_are_given_back_on_error_and_on_early_exit():
    class Failing(Scripted):
        def decode(self, *a):
            raise RuntimeError("boom")

    be = Failing({0: [1, 2]})
    with pytest.raises(RuntimeError):
        list(run_batch(be, [[1]], 2, GREEDY))
    assert be.free == list(range(8))
    be = Scripted({0: [1, 2, 3, 4]})
    gen = run_batch(be, [[1]], 4, GREEDY)
    next(gen)
    gen.close()  # the consumer stops early
    assert be.free == list(range(8))


def test_plan_batches():
    # at most 2 sequences and 256 cache tokens per batch, pages of 64
    assert plan_batches([10, 10, 10], 2, 256, 64, 128) == [[0, 1], [2]]
    assert plan_batches([100, 100, 100], 4, 256, 64, 128) == [[0, 1], [2]]   # 128 + 128 fills the cache
    assert plan_batches([65, 1, 1, 1], 4, 256, 64, 128) == [[0, 1, 2], [3]]
    assert plan_batches([], 4, 256, 64, 128) == []
    with pytest.raises(ValueError):
        plan_batches([129], 4, 256, 64, 128)
    with pytest.raises(ValueError):
        plan_batches([200], 4, 128, 64, 256)


def test_requests_run_batch_after_batch_and_reuse_slots():
    script = {i: [100 + i, 200 + i, 99 if i % 2 else 300 + i] for i in range(5)}
    be = Scripted(script, n_slots=2)
    res = run_requests(be, [[1]] * 5, 3, GREEDY, [99], [[0, 1], [2, 3], [4]])
    assert res == [[100, 200, 300], [101, 201, 99], [102, 202, 302], [103, 203, 99], [104, 204, 304]]
    opens = [c for c in be.calls if c[0] == "open"]
    assert [c[1] for c in opens] == [(0, 1), (0, 1), (0,)]  # the same slots again
    # a request samples as the same sequence index whatever batch it lands in
    prefills = [c for c in be.calls if c[0] == "prefill"]
    assert [c[3] for c in prefills] == [(0, 1), (2, 3), (4,)]


def test_sampling_params_are_validated():
    with pytest.raises(ValueError):
        SamplingParams(temperature=-1.0)
    with pytest.raises(ValueError):
        SamplingParams(top_k=-2)
    assert SamplingParams().greedy and not SamplingParams(temperature=0.7).greedy


class ScriptedInFlight(Scripted):
    """The same backend with the optional pair: a step is launched, and its tokens are fetched later."""

    def decode_launch(self, handles, seq_ids, step, params):
        self.calls.append(("launch", step))
        return (step, self.decode(handles, seq_ids, step, params))

    def decode_result(self, ticket):
        step, toks = ticket
        self.calls.append(("result", step))
        return toks


def test_one_step_is_kept_in_flight_when_nothing_can_stop_early():
    script = {0: [10, 11, 12, 13], 1: [20, 21, 22, 23]}
    plain = list(run_batch(Scripted(script), [[1, 2, 3], [4]], 4, GREEDY))
    be = ScriptedInFlight(script)
    seen = []
    for out in run_batch(be, [[1, 2, 3], [4]], 4, GREEDY):
        seen.append((out, [c for c in be.calls if c[0] in ("launch", "result")]))
    assert [o for o, _ in seen] == plain == [[10, 20], [11, 21], [12, 22], [13, 23]]
    assert seen[0][1] == []                                          # the first tokens go out before any decode step is launched
    order = [c for c in be.calls if c[0] in ("launch", "result")]
    assert order == [("launch", 1), ("launch", 2), ("result", 1), ("launch", 3), ("result", 2), ("result", 3)]
    assert be.calls[-1][0] == "close" and sorted(be.free) == list(range(8))
    # a single new token: no decode step at all
    be = ScriptedInFlight(script)
    assert list(run_batch(be, [[1], [2]], 1, GREEDY)) == [[10, 20]] and not [c for c in be.calls if c[0] == "launch"]


def test_stop_tokens_switch_the_flight_off():
    """With stop tokens the host must see a step's tokens before it can decide who runs the next one."""
    be = ScriptedInFlight({0: [10, 99, 12], 1: [20, 21, 22]})
    out = list(run_batch(be, [[1], [2]], 3, GREEDY, stop_token_ids=[99]))
    assert out == [[10, 20], [99, 21], [ENDED, 22]]
    assert not [c for c in be.calls if c[0] in ("launch", "result")]


def test_leaving_early_with_a_step_in_flight_gives_the_slots_back():
    be = ScriptedInFlight({0: [10, 11, 12, 13], 1: [20, 21, 22, 23]})
    gen = run_batch(be, [[1], [2]], 4, GREEDY)
    assert next(gen) == [10, 20] and next(gen) == [11, 21]
    gen.close()
    assert be.calls[-1][0] == "close" and sorted(be.free) == list(range(8))
