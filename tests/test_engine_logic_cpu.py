"""The step function, the cache and the loops above them on the CPU, with every CUDA kernel replaced by its plain
reference (tests/kernel_refs.py, through the `reference_kernels` fixture). This checks the host side: the batch
layout, positions, page tables, slot reuse, the order of the schedule. The kernels themselves are checked on a GPU."""
import io
import json

import numpy as np
import pytest
import torch

from tests import plain_qwen2 as plain
from tests.helpers import CONFIGS, make_model_dir, max_err, random_tokens


def build(config, tmp_path, seed=0):
    from qwenforge_b200.engine import Model
    folder, weights = make_model_dir(config, seed, tmp_path)
    return Model.from_dir(folder, "float32", "cpu"), weights, folder


@pytest.mark.parametrize("name", list(CONFIGS))
def test_every_cut_gives_the_plain_logits(reference_kernels, name, tmp_path):
    config = CONFIGS[name]
    model, weights, _ = build(config, tmp_path)
    cache = model.new_cache(64 * 8, 3)
    vocab = config["vocab_size"]
    seqs = [random_tokens(vocab, n, 10 + n) for n in (70, 5, 33, 101, 64)]
    refs = [plain.forward_logits(config, weights, s) for s in seqs]
    for round_ in range(2):                               # the second round runs in slots and pages used before
        for begin in range(0, len(seqs), 3):
            batch = list(range(begin, min(begin + 3, len(seqs))))
            slots = {i: cache.open() for i in batch}
            heads = {i: max(1, len(seqs[i]) - 4 - i) for i in batch}
            logits = model.step(cache, [(slots[i], seqs[i][:heads[i]]) for i in batch],
                                want=[list(range(heads[i])) for i in batch])
            got = {i: [] for i in batch}
            o = 0
            for i in batch:
                got[i].append(logits[o:o + heads[i]])
                o += heads[i]
            fed = dict(heads)
            live = [i for i in batch if fed[i] < len(seqs[i])]
            while live:
                logits = model.step(cache, [(slots[i], [seqs[i][fed[i]]]) for i in live])
                for row, i in enumerate(live):
                    got[i].append(logits[row:row + 1])
                    fed[i] += 1
                for i in [i for i in live if fed[i] == len(seqs[i])]:
                    cache.close(slots.pop(i))
                live = [i for i in live if fed[i] < len(seqs[i])]
            for i in list(slots):
                cache.close(slots.pop(i))
            for i in batch:
                assert max_err(torch.cat(got[i]), refs[i]) < 2e-6, (name, round_, i)
    assert cache.slots.n_free == cache.max_seqs and all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


def test_step_refuses_what_it_cannot_hold(reference_kernels, tmp_path):
    from qwenforge_b200.cache import CacheFull
    config = CONFIGS["tiny_a"]
    model, _, _ = build(config, tmp_path)
    cache = model.new_cache(128, 2)
    slot = cache.open()
    with pytest.raises(CacheFull):
        model.step(cache, [(slot, [1] * 129)])
    assert cache.lengths[slot] == 0 and cache.kv_groups[0].pages.n_free == 2   # nothing half-done
    with pytest.raises(ValueError, match="exceeds model limit"):
        big = model.new_cache(1024, 2)
        model.step(big, [(big.open(), [1] * 385)])
    with pytest.raises(ValueError, match="twice"):
        model.step(cache, [(slot, [1]), (slot, [2])])
    with pytest.raises(ValueError, match="brings no tokens"):
        model.step(cache, [(slot, [])])


def test_generation_through_the_entry_point(reference_kernels, tmp_path, monkeypatch):
    from qwenforge_b200.engine import StudentEngine
    config = CONFIGS["tiny_b"]
    folder, weights = make_model_dir(config, 4, tmp_path)
    engine = StudentEngine(str(folder), device="cpu", dtype="float32")
    prompts = [random_tokens(config["vocab_size"], n, 20 + n) for n in (3, 9, 1, 14)]
    got = engine.generate_ids(prompts, max_new_tokens=[5, 2, 6, 4], batch_size=3, ignore_eos=True)
    want = [plain.greedy_generate(config, weights, p, b) for p, b in zip(prompts, (5, 2, 6, 4))]
    assert got == want
    assert not engine.cache.live_slots()
    sampled = engine.generate_ids(prompts, 5, batch_size=2, temperature=0.8, seed=3, ignore_eos=True)
    again = engine.generate_ids(prompts, 5, batch_size=4, temperature=0.8, seed=3, ignore_eos=True)
    assert sampled == again and sampled != engine.generate_ids(prompts, 5, batch_size=4, ignore_eos=True)
    with pytest.raises(TypeError, match="list\\[str\\]"):
        engine.generate("not a list", 3)
    texts = engine.generate(["ab", "c"], 3, batch_size=2, suite_name="ignored")
    assert len(texts) == 2 and all(isinstance(t, str) and len(t) == 3 for t in texts)


def test_replay_in_process(reference_kernels, tmp_path):
    from qwenforge_b200.engine.replay import replay
    config = CONFIGS["tiny_a"]
    model, weights, _ = build(config, tmp_path / "m")
    cache = model.new_cache(128, 2)
    a, b = random_tokens(256, 20, 1), random_tokens(256, 7, 2)
    steps = [dict(step=0, entries=[dict(id="a", tokens=a[:19], want=[0, 18]), dict(id="b", tokens=b[:6], want=[])], end=[]),
             dict(step=1, entries=[dict(id="a", tokens=a[19:], want=[0]), dict(id="b", tokens=b[6:], want=[0])], end=["a", "b"]),
             dict(step=2, entries=[dict(id="c", tokens=b, want=[6])], end=["c"])]
    out = tmp_path / "o"
    out.mkdir()
    said = []
    dumps = tmp_path / "layers"
    dumps.mkdir()
    replay(model, cache, io.StringIO("".join(json.dumps(s) + "\n" for s in steps)), out, report=said.append, dump_dir=dumps)
    model.observer = None
    assert said == ["done 0", "done 1", "done 2"]
    # the dumped residual stream of the last step (request c, whole): the embedding, then every layer's output
    sizes = plain.read_sizes(config)
    w64 = {k: v.double() for k, v in weights.items()}
    h = w64["model.embed_tokens.weight"][torch.tensor(b)]
    cos, sin = plain.rope_cos_sin(torch.arange(len(b)), sizes["head_dim"], sizes["theta"], torch.float64)
    for k in range(sizes["layers"] + 1):
        dumped = torch.from_numpy(np.fromfile(dumps / f"2.layer{k}.f32", dtype="<f4").reshape(len(b), -1).copy())
        assert max_err(dumped, h) < 2e-6, f"residual stream after {k} layers"
        if k < sizes["layers"]:
            h = plain.decoder_layer(h, w64, k, sizes, cos, sin)
    ra, rb = plain.forward_logits(config, weights, a), plain.forward_logits(config, weights, b)
    read = lambda n: torch.from_numpy(np.fromfile(out / f"{n}.f32", dtype="<f4").reshape(-1, 256).copy())
    assert max_err(read(0), ra[[0, 18]]) < 2e-6
    assert max_err(read(1), torch.stack((ra[19], rb[6]))) < 2e-6
    assert max_err(read(2), rb[6:7]) < 2e-6
    assert not cache.live_slots()


def test_no_cpu_path_in_the_package(tmp_path):
    """Without the fixture the package refuses to compute anywhere but on a CUDA device."""
    from qwenforge_b200.engine import Model
    from qwenforge_b200.ops import KernelError
    folder, _ = make_model_dir(CONFIGS["tiny_a"], 0, tmp_path)
    with pytest.raises(KernelError, match="no CPU execution path|CUDA devices only"):
        Model.from_dir(folder, "float32", "cpu")


def test_pack_step_layout_and_shape_key():
    """The step's integers lie as ids | tok_seq | tok_pos | slots | cu_q | rows; steps of equal shape share a key
    whatever their tokens, slots and start positions are."""
    import numpy as np
    from qwenforge_b200.engine.step import pack_step
    a = pack_step([(3, 0, [5, 6, 7]), (-1, 0, [9]), (0, 10, [1, 2])], None)
    assert a.n_tokens == 6 and a.n_seqs == 3 and a.n_rows == 2 and a.max_q_len == 3 and a.max_kv_len == 12
    want = [5, 6, 7, 9, 1, 2] + [0, 0, 0, 1, 2, 2] + [0, 1, 2, 0, 10, 11] + [3, -1, 0] + [0, 3, 4, 6] + [2, 5]
    assert a.packed.dtype == np.int32 and a.packed.tolist() == want
    b = pack_step([(1, 40, [8, 8, 8]), (2, 7, [4]), (5, 0, [3, 3])], [[0], [], [1]])
    assert b.shape_key == a.shape_key
    c = pack_step([(1, 0, [8, 8, 8, 8]), (2, 0, [4, 4])], None)
    assert c.shape_key != a.shape_key
    import pytest
    with pytest.raises(ValueError, match="wants place 3"):
        pack_step([(0, 0, [1, 2, 3])], [[3]])


def test_prompt_graphs_decisions_without_a_gpu():
    """Which steps are replayed: not the first of a shape, every later one; other shapes and other caches have graphs
    of their own; only the newest `keep` stay; a shape whose capture fails is left alone from then on."""
    import types
    import torch
    from qwenforge_b200.engine.graphs import PrefillGraphs
    from qwenforge_b200.engine.step import pack_step

    class FakeGraph:
        def __init__(self):
            self.replayed = 0

        def replay(self):
            self.replayed += 1

    captured = []

    def fake_capture(self, cache, step):
        if step.host_q_lens[0] == 13:
            raise RuntimeError("no memory")
        graph = FakeGraph()
        captured.append((cache.serial, step.shape_key, graph))
        return graph, torch.zeros(step.packed.size, dtype=torch.int32), torch.full((step.n_rows, 4), float(len(captured))), 7

    graphs = PrefillGraphs(model=types.SimpleNamespace(), keep=2)
    graphs._capture = types.MethodType(fake_capture, graphs)
    cache_a, cache_b = types.SimpleNamespace(serial=1), types.SimpleNamespace(serial=2)
    triples = lambda lens, slot0=0: [(slot0 + i, 0, list(range(n))) for i, n in enumerate(lens)]
    step = lambda lens, slot0=0: pack_step(triples(lens, slot0), None)
    run = lambda cache, lens, slot0=0: graphs.run(cache, step(lens, slot0), triples(lens, slot0), None)

    assert not graphs.takes(step([1, 1])) and graphs.takes(step([2, 1])) and not graphs.takes(step([9000]))
    assert run(cache_a, [50, 30]) is None and not captured                       # first of its shape: launch by launch
    out = run(cache_a, [45, 33], slot0=4)                                        # second (other lengths, same rounded shape): captured and replayed
    assert out is not None and out.shape == (2, 4) and len(captured) == 1 and captured[0][2].replayed == 1
    assert captured[0][1] == (128, 3, 64, 2)
    held_integers = graphs.graphs[(1, 128, 3, 64, 2)][1]
    padded = pack_step(triples([45, 33], 4) + [(-1, 0, [0] * 50)], None)
    assert held_integers.tolist() == padded.packed.tolist()                      # the replay's own integers went in, padding entry last
    run(cache_a, [64, 1])
    assert captured[0][2].replayed == 2 and graphs.replays == 2 and len(captured) == 1
    assert run(cache_b, [50, 30]) is None                                        # another cache: its own count
    assert run(cache_a, [70, 10]) is None                                        # same tokens, a longer longest entry
    assert run(cache_a, [64, 64]) is None                                        # a full granule: no padding entry, a shape of its own
    for lens in ([130, 1], [200, 1]):
        run(cache_a, lens)
        run(cache_a, lens)
    assert len(graphs.graphs) == 2 and (1, 128, 3, 64, 2) not in graphs.graphs   # the oldest graph was dropped
    assert run(cache_a, [13]) is None and run(cache_a, [13]) is None
    assert run(cache_a, [13]) is None and len(captured) == 3                     # the failed capture is not tried again


def test_prompt_steps_are_rounded_to_shapes_that_come_back():
    """Prompt steps replay a graph when their rounded shape came before: token counts go up to the next multiple of
    the granule through ONE padding entry, the bound on the longest entry likewise, and nothing else changes."""
    from qwenforge_b200.engine.graphs import PrefillGraphs
    from qwenforge_b200.engine.step import pack_step
    assert [PrefillGraphs.granule(n) for n in (2, 512, 513, 2048, 2049, 4096, 4097, 8192)] == [64, 64, 128, 128, 256, 256, 512, 512]
    triples = [(3, 0, list(range(100))), (1, 7, list(range(30)))]
    want = [[0, 99], [29]]
    step = pack_step(triples, want)
    rounded = PrefillGraphs.rounded(step, triples, want)
    assert rounded.shape_key == (192, 3, 128, 3)
    assert rounded.host_slots == [3, 1, -1] and rounded.host_q_lens == [100, 30, 62] and rounded.max_kv_len == 128
    n = step.n_tokens
    assert list(rounded.packed[:n]) == list(step.packed[:n]) and not rounded.packed[n:192].any()      # ids, then zeros
    assert list(rounded.packed[-3:]) == list(step.packed[-3:])                                          # the wanted rows
    assert step.max_q_len == 100                                                                        # the step itself is left alone
    other = [(0, 0, list(range(90))), (2, 0, list(range(41)))]
    assert PrefillGraphs.rounded(pack_step(other, None), other, None).shape_key == (192, 3, 128, 2)
    exact = [(0, 0, list(range(128)))]
    same = PrefillGraphs.rounded(pack_step(exact, None), exact, None)
    assert same.shape_key == (128, 1, 128, 1) and same.host_slots == [0]


def test_decode_session_keeps_the_next_chunk_on_the_stream():
    """The graph session's order of events with a scripted graph: a chunk is enqueued once, the chunk after it goes
    onto the stream as soon as the device says that a row is live and before the caller sees a token, nothing is
    enqueued after every row has ended, and the cache learns how many tokens each slot was fed."""
    from qwenforge_b200.engine.engine import _GraphSession
    from qwenforge_b200.engine.graphs import CHUNK_STEPS

    events = []

    class ScriptedGraph:
        """Two rows: row 0 runs 40 steps, row 1 ends after 5 (a stop token)."""
        def __init__(self):
            self.done = 0
        def load(self, *state):
            events.append("load")
        def enqueue(self, n):
            n = min(n, CHUNK_STEPS)
            events.append(("enqueue", n))
            self.pending = n
            return n
        def collect(self, n):
            assert n == self.pending
            tokens = [[100 + self.done + i, 200 + self.done + i if self.done + i < 5 else -1] for i in range(n)]
            self.done += n
            events.append(("collect", n))
            return tokens, max(40 - self.done, 0), 0

    class Cache:
        lengths = {3: 10, 4: 7}
        advanced = {3: 0, 4: 0}
        def flush(self):
            pass
        def advance(self, slot, n):
            self.advanced[slot] += n

    class Decoder:
        def get(self, rows, longest, sampler):
            assert rows == 2 and longest == 10 + 40
            return ScriptedGraph()

    class Stepper:
        cache, graph_decoder, sampler, model = Cache(), Decoder(), None, None

    session = _GraphSession(Stepper(), [(3, 9, 0, 0, 40), (4, 8, 1, 0, 40)], (2,))
    first = session.run(40)
    assert events == ["load", ("enqueue", 32), ("collect", 32), ("enqueue", 8)]   # the next chunk is out before we look
    assert len(first) == 32 and first[0] == [100, 200] and first[5] == [105, -1]
    second = session.run(8)
    assert events[4:] == [("collect", 8)] and len(second) == 8 and second[-1] == [139, -1]   # nothing after the end
    assert session.in_flight == 0
    assert Cache.advanced == {3: 40, 4: 5}
