"""The generation loop's decisions, against a scripted stepper (no model, no GPU)."""
import pytest

from qwenforge_b200.engine.generate import GenerationLoop


class ScriptedStepper:
    """Chooses token = (sum of the fed tokens + sequence id + step) % 50, and records everything."""
    max_positions = 64

    def __init__(self, n_slots=3):
        self.free = list(range(n_slots))[::-1]
        self.held = set()
        self.calls = []
        self.reserved = []

    def open(self):
        if not self.free:
            raise RuntimeError("no free slot")
        s = self.free.pop()
        self.held.add(s)
        return s

    def close(self, slot):
        assert slot in self.held, "closed twice"
        self.held.remove(slot)
        self.free.append(slot)
        self.free.sort(reverse=True)

    def reserve(self, slot_totals):
        self.reserved.append(list(slot_totals))

    def step_and_choose(self, entries, seq_ids, steps):
        assert len({slot for slot, _ in entries}) == len(entries)
        self.calls.append(([(slot, list(t)) for slot, t in entries], list(seq_ids), list(steps)))
        return [(sum(t) + i + k) % 50 for (_, t), i, k in zip(entries, seq_ids, steps)]


def expected(prompt, index, budget, stops=()):
    out, fed = [], list(prompt)
    for k in range(budget):
        token = (sum(fed) + index + k) % 50
        out.append(token)
        if token in stops:
            break
        fed = [token]
    return out


def test_batches_start_together_and_run_one_after_another():
    st = ScriptedStepper(3)
    prompts = [[1, 2, 3], [4], [5, 6], [7, 8, 9, 10], [11]]
    results = GenerationLoop(st).run(prompts, 4, batch_size=3)
    assert [r.tokens for r in results] == [expected(p, i, 4) for i, p in enumerate(prompts)]
    assert all(r.finish_reason == "length" for r in results)
    first, second = st.calls[0], st.calls[4]
    assert [t for _, t in first[0]] == prompts[:3] and first[1] == [0, 1, 2] and first[2] == [0, 0, 0]
    assert [t for _, t in second[0]] == prompts[3:] and second[1] == [3, 4]
    assert len(st.calls) == 8                     # per batch: 1 prompt step + 3 single-token steps
    assert all(len(t) == 1 for call in st.calls[1:4] for _, t in call[0])
    assert {slot for slot, _ in second[0]} <= {0, 1, 2} and not st.held   # slots used again, none left held
    assert st.reserved[0] == [(0, 3 + 3), (1, 1 + 3), (2, 2 + 3)]


def test_sequences_end_on_their_own():
    st = ScriptedStepper(3)
    prompts = [[1, 2, 3], [4], [5, 6]]
    budgets = [2, 5, 3]
    results = GenerationLoop(st).run(prompts, budgets, batch_size=3)
    assert [len(r.tokens) for r in results] == budgets
    sizes = [len(call[0]) for call in st.calls]
    assert sizes == [3, 3, 2, 1, 1]               # the batch shrinks as requests end
    assert not st.held


def test_stop_tokens_end_a_sequence_and_are_kept():
    prompts = [[1, 2, 3], [4]]
    free_run = [expected(p, i, 6) for i, p in enumerate(prompts)]
    stop = free_run[0][2]
    st = ScriptedStepper(2)
    results = GenerationLoop(st, stop_token_ids=[stop]).run(prompts, 6, batch_size=2)
    assert results[0].tokens == expected(prompts[0], 0, 6, [stop]) and results[0].tokens[-1] == stop
    assert results[0].finish_reason == "stop"
    assert results[1].tokens == expected(prompts[1], 1, 6, [stop])
    ignoring = GenerationLoop(ScriptedStepper(2), stop_token_ids=[stop], ignore_eos=True).run(prompts, 6, batch_size=2)
    assert [r.tokens for r in ignoring] == free_run


def test_stop_on_the_first_token_needs_no_decode_step():
    st = ScriptedStepper(1)
    first = expected([9], 0, 1)[0]
    results = GenerationLoop(st, stop_token_ids=[first]).run([[9]], 5)
    assert results[0].tokens == [first] and len(st.calls) == 1 and not st.held


def test_budgets_and_limits():
    st = ScriptedStepper(2)
    results = GenerationLoop(st).run([[1], [2]], [0, 1], batch_size=2)
    assert results[0].tokens == [] and results[1].tokens == expected([2], 1, 1)
    assert len(st.calls) == 1 and len(st.calls[0][0]) == 1   # the request without budget never ran
    with pytest.raises(ValueError, match="exceeds model limit 64"):
        GenerationLoop(ScriptedStepper(1)).run([[1] * 60], 5)
    with pytest.raises(ValueError, match="one per prompt"):
        GenerationLoop(ScriptedStepper(1)).run([[1]], [1, 2])


def test_empty_prompt_takes_bos_or_fails():
    with pytest.raises(ValueError, match="empty prompt"):
        GenerationLoop(ScriptedStepper(1)).run([[]], 2)
    st = ScriptedStepper(1)
    results = GenerationLoop(st, bos_token_id=7).run([[]], 2)
    assert st.calls[0][0][0][1] == [7] and results[0].tokens == expected([7], 0, 2)


def test_slots_are_returned_after_a_failure():
    class Failing(ScriptedStepper):
        def step_and_choose(self, entries, seq_ids, steps):
            if len(self.calls) == 2:
                raise RuntimeError("boom")
            return super().step_and_choose(entries, seq_ids, steps)

    st = Failing(2)
    with pytest.raises(RuntimeError, match="boom"):
        GenerationLoop(st).run([[1], [2]], 5, batch_size=2)
    assert not st.held
