"""The engine against the plain implementation on a GPU, in float32 and in bfloat16: each request alone and
whole; with the last 32 tokens one by one; in batches of unequal lengths whose shorter requests end earlier,
one batch after another so that slots and pages are used again; long decoding; the first tokens of a
sequence; greedy generation through the entry point."""
import pytest
import torch

from tests import plain_qwen2 as plain
from tests.helpers import CONFIGS, SMALL_64, SMALL_128, assert_logits_close, make_model_dir, random_tokens

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
ALL_CONFIGS = dict(CONFIGS, small_64=SMALL_64, small_128=SMALL_128)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for i, (name, config) in enumerate(ALL_CONFIGS.items()):
        out[name] = make_model_dir(config, seed=i, folder=tmp_path_factory.mktemp(name))
    return out


_models = {}


def get_model(folders, name, dtype, attention="auto"):
    from qwenforge_b200.engine import Model
    key = (name, dtype, attention)
    if key not in _models:
        _models[key] = Model.from_dir(folders[name][0], dtype, "cuda", attention)
    return _models[key]


def plain_logits(folders, name, tokens):
    return plain.forward_logits(ALL_CONFIGS[name], folders[name][1], tokens)


def lengths_for(name):
    limit = ALL_CONFIGS[name]["max_position_embeddings"]
    return [n for n in (1, 5, 33, 64, 65, 130, 200) if n <= limit]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ALL_CONFIGS))
def test_whole_requests_alone(folders, name, dtype):
    model = get_model(folders, name, dtype)
    cache = model.new_cache(1024, 4)
    vocab = ALL_CONFIGS[name]["vocab_size"]
    for i, n in enumerate(lengths_for(name)):
        tokens = random_tokens(vocab, n, 100 + i)
        slot = cache.open()
        logits = model.step(cache, [(slot, tokens)], want=[list(range(n))])
        model.raise_on_kernel_error()
        assert_logits_close(logits, plain_logits(folders, name, tokens), dtype, f"{name} whole {n}")
        cache.close(slot)
    assert cache.slots.n_free == cache.max_seqs and all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ALL_CONFIGS))
def test_last_32_one_by_one(folders, name, dtype):
    model = get_model(folders, name, dtype)
    cache = model.new_cache(1024, 4)
    vocab = ALL_CONFIGS[name]["vocab_size"]
    for i, n in enumerate([40, 97, 130]):
        tokens = random_tokens(vocab, n, 200 + i)
        ref = plain_logits(folders, name, tokens)
        slot = cache.open()
        head = n - 32
        got = [model.step(cache, [(slot, tokens[:head])], want=[list(range(head))])]
        for t in range(head, n):
            got.append(model.step(cache, [(slot, tokens[t:t + 1])]))
        model.raise_on_kernel_error()
        got = torch.cat(got)
        assert_logits_close(got, ref, dtype, f"{name} last-32 of {n}")
        if dtype == torch.float32:
            # the same positions computed whole: equal beyond the plain comparison's tolerance
            slot2 = cache.open()
            whole = model.step(cache, [(slot2, tokens)], want=[list(range(n))])
            assert float((whole - got).abs().max()) <= 1e-5 * float(ref.abs().max())
            cache.close(slot2)
        cache.close(slot)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", list(ALL_CONFIGS))
def test_unequal_batches_with_slot_reuse(folders, name, dtype):
    """Three batches one after another in a cache with 4 slots and few pages; in each, prompts of unequal
    lengths start together, then decode one token each; shorter requests end earlier."""
    model = get_model(folders, name, dtype)
    cache = model.new_cache(64 * 9, 4)
    vocab = ALL_CONFIGS[name]["vocab_size"]
    batches = [[(5, 9), (70, 3), (17, 12), (1, 6)], [(33, 4), (64, 8), (2, 2)], [(100, 5), (63, 7), (9, 1), (40, 10)]]
    seed = 300
    for batch in batches:
        seqs = []
        for prompt_len, n_decode in batch:
            seed += 1
            tokens = random_tokens(vocab, prompt_len + n_decode, seed)
            seqs.append(dict(tokens=tokens, prompt=prompt_len, total=prompt_len + n_decode, fed=0, got=[],
                             slot=cache.open()))
        logits = model.step(cache, [(s["slot"], s["tokens"][:s["prompt"]]) for s in seqs],
                            want=[list(range(s["prompt"])) for s in seqs])
        offset = 0
        for s in seqs:
            s["got"].append(logits[offset:offset + s["prompt"]])
            offset += s["prompt"]
            s["fed"] = s["prompt"]
        live = list(seqs)
        while live:
            logits = model.step(cache, [(s["slot"], [s["tokens"][s["fed"]]]) for s in live])
            for row, s in enumerate(live):
                s["got"].append(logits[row:row + 1])
                s["fed"] += 1
            for s in [s for s in live if s["fed"] == s["total"]]:
                cache.close(s["slot"])
            live = [s for s in live if s["fed"] < s["total"]]
        model.raise_on_kernel_error()
        for s in seqs:
            assert_logits_close(torch.cat(s["got"]), plain_logits(folders, name, s["tokens"]), dtype,
                                f"{name} batch request {s['prompt']}+{s['total'] - s['prompt']}")
    assert cache.slots.n_free == cache.max_seqs and all(g.pages.n_free == g.pages.n_pages for g in cache.kv_groups)


@pytest.mark.parametrize("dtype", DTYPES)
def test_padding_entries_change_nothing(folders, dtype):
    name = "tiny_b"
    model = get_model(folders, name, dtype)
    cache = model.new_cache(1024, 4)
    tokens = random_tokens(ALL_CONFIGS[name]["vocab_size"], 20, 7)
    a, b = cache.open(), cache.open()
    alone = model.step(cache, [(a, tokens)], want=[list(range(20))])
    padded = model.step(cache, [(-1, [0, 0, 0]), (b, tokens), (-1, [1])], want=[[], list(range(20)), []])
    model.raise_on_kernel_error()
    assert torch.equal(alone, padded) if dtype == torch.float32 else float((alone - padded).abs().max()) < 1e-2
    d1 = model.step(cache, [(a, [5])])
    d2 = model.step(cache, [(-1, [9]), (b, [5])], want=[[], [0]])
    assert torch.equal(d1, d2) if dtype == torch.float32 else float((d1 - d2).abs().max()) < 1e-2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["tiny_a", "tiny_w", "small_64"])
def test_long_decoding(folders, name, dtype):
    """A short prompt, then token after token across several pages (and, for tiny_w, far beyond the window)."""
    model = get_model(folders, name, dtype)
    cache = model.new_cache(512, 2)
    total = min(300, ALL_CONFIGS[name]["max_position_embeddings"])
    tokens = random_tokens(ALL_CONFIGS[name]["vocab_size"], total, 11)
    slot = cache.open()
    got = [model.step(cache, [(slot, tokens[:3])], want=[[0, 1, 2]])]
    for t in range(3, total):
        got.append(model.step(cache, [(slot, [tokens[t]])]))
    model.raise_on_kernel_error()
    assert_logits_close(torch.cat(got), plain_logits(folders, name, tokens), dtype, f"{name} long decode")
    if name == "tiny_w":  # pages that left the window were given back
        group = [g for g in cache.kv_groups if g.need.window > 0][0]
        assert group.pages_held(slot) <= (37 + 63) // 64 + 1


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens(folders, dtype):
    """Positions 0, 1, 2 of a sequence fed one by one, and a one-token prompt in a batch."""
    for name in CONFIGS:
        model = get_model(folders, name, dtype)
        cache = model.new_cache(512, 4)
        tokens = random_tokens(ALL_CONFIGS[name]["vocab_size"], 4, 13)
        slot, other = cache.open(), cache.open()
        got = []
        for t in range(4):
            entries = [(slot, [tokens[t]])] + ([(other, [1, 2, 3])] if t == 0 else [(other, [4])])
            got.append(model.step(cache, entries)[0:1])
        model.raise_on_kernel_error()
        assert_logits_close(torch.cat(got), plain_logits(folders, name, tokens), dtype, f"{name} first tokens")


@pytest.mark.parametrize("dtype", DTYPES)
def test_far_key_among_hundreds(folders, dtype, tmp_path):
    """Random weights spread attention thinly over hundreds of keys, which would hide a key that is lost or read
    from the wrong place. Here the query and key projections are scaled up so that the softmax is sharp and single
    keys decide the result; the plain implementation itself confirms that replacing ONE far token moves the last
    position's logits by much more than the tolerance, so an engine that misreads that key cannot pass."""
    import json

    from qwenforge_b200.engine import Model
    from qwenforge_b200.weights import save_safetensors
    name = "tiny_a"
    config = ALL_CONFIGS[name]
    weights = {k: v.clone() for k, v in folders[name][1].items()}
    for key in weights:
        if any(part in key for part in ("q_proj", "k_proj")):
            weights[key] *= 15.0
    n = 330
    tokens = random_tokens(config["vocab_size"], n, 17)
    ref = plain.forward_logits(config, weights, tokens)
    rel, abs_ = (2e-5, 2e-6) if dtype == torch.float32 else (4e-2, 2e-2)
    bound = abs_ + rel * float(ref.abs().max())
    sensitivity = 0.0
    for far in range(0, 128, 4):
        moved = list(tokens)
        moved[far] = (moved[far] + 1) % config["vocab_size"]
        sensitivity = max(sensitivity, float((plain.forward_logits(config, weights, moved)[-1] - ref[-1]).abs().max()))
    assert sensitivity > 2.5 * bound, f"no far key matters enough ({sensitivity:.3e} vs {bound:.3e}) for this test to see a fault"
    (tmp_path / "config.json").write_text(json.dumps(config))
    save_safetensors(tmp_path / "model.safetensors", weights)
    model = Model.from_dir(tmp_path, dtype, "cuda")
    cache = model.new_cache(512, 2)
    slot = cache.open()
    got = [model.step(cache, [(slot, tokens[:200])], want=[list(range(200))])]
    for t in range(200, n):
        got.append(model.step(cache, [(slot, [tokens[t]])]))
    model.raise_on_kernel_error()
    assert_logits_close(torch.cat(got), ref, dtype, "sharp attention over far keys")


SMALL_64W = dict(SMALL_64, use_sliding_window=True, sliding_window=100, max_window_layers=1)
# configuration, seed of the weights, seed of the tokens: chosen so that one token far back (or near the window's far
# edge) moves the last logits by several times the tolerance once queries and keys are scaled by 3
SHARP_CASES = {"small_64": (SMALL_64, 3, 18), "small_128": (SMALL_128, 4, 21), "small_64w": (SMALL_64W, 3, 22)}


@pytest.mark.parametrize("tcgen05", [False, True], ids=["mma", "tcgen05"])
@pytest.mark.parametrize("case", list(SHARP_CASES))
def test_far_key_through_the_tensor_core_kernels(case, tcgen05, tmp_path, monkeypatch):
    """The sharp-softmax test at the head sizes of the real models, in bfloat16: a 300-token prompt through the
    tensor-core prefill attention (mma.sync, or tcgen05 when forced), continuations of 2 and of 60 tokens across a page
    end (and, windowed, across the window's edge), single tokens through the fused decode kernels, and the last 20
    from a captured decode graph over a cache whose windowed pages are given back meanwhile."""
    import json

    from qwenforge_b200.engine import Model
    from qwenforge_b200.engine.graphs import DecodeGraph
    from qwenforge_b200.parts import attention
    from qwenforge_b200.sampling import Sampler
    from qwenforge_b200.weights import save_safetensors
    config, weight_seed, token_seed = SHARP_CASES[case]
    weights = plain.random_weights(config, weight_seed)
    for key in weights:
        if "q_proj" in key or "k_proj" in key:
            weights[key] = weights[key] * 3.0
    n = 420
    tokens = random_tokens(config["vocab_size"], n, token_seed)
    ref = plain.forward_logits(config, weights, tokens)
    bound = 2e-2 + 4e-2 * float(ref.abs().max())
    first = n - 100 if config.get("use_sliding_window") else 0
    sensitivity = 0.0
    for far in range(first, first + 64, 2):
        moved = list(tokens)
        moved[far] = (moved[far] + 1) % config["vocab_size"]
        sensitivity = max(sensitivity, float((plain.forward_logits(config, weights, moved)[-1] - ref[-1]).abs().max()))
    assert sensitivity > 2.5 * bound, f"no far key matters enough ({sensitivity:.3e} vs {bound:.3e}) for this test to see a fault"
    (tmp_path / "config.json").write_text(json.dumps(config))
    save_safetensors(tmp_path / "model.safetensors", weights)
    if tcgen05:
        monkeypatch.setattr(attention, "TC_PREFILL_MIN_TOKENS", {64: 1, 128: 1})
    model = Model.from_dir(tmp_path, torch.bfloat16, "cuda")
    cache = model.new_cache(1024, 2)
    slot = cache.open()
    cache.reserve([(slot, n)])
    got = [model.step(cache, [(slot, tokens[:300])], want=[list(range(300))]),
           model.step(cache, [(slot, tokens[300:302])], want=[[0, 1]]),
           model.step(cache, [(slot, tokens[302:362])], want=[list(range(60))])]
    for t in range(362, 400):
        got.append(model.step(cache, [(slot, [tokens[t]])]))
    graph = DecodeGraph(model, cache, 1, 512, Sampler())
    cache.flush()
    graph.capture()
    for t in range(400, n):
        cache.flush()   # a windowed group gave pages back at the last advance
        graph.load([slot], [tokens[t]], [t], [1], [1 << 30], [0], [])
        graph.run(1)
        got.append(graph.last_logits.clone())
        cache.advance(slot, 1)
    model.raise_on_kernel_error()
    if config.get("use_sliding_window"):
        group = [g for g in cache.kv_groups if g.need.window > 0][0]
        assert group.pages_held(slot) <= (100 + 63) // 64 + 1
    assert_logits_close(torch.cat(got), ref, torch.bfloat16, f"{case}: sharp attention over far keys")


def test_prompts_of_new_lengths_replay_a_rounded_shape(folders):
    """A prompt whose length never came before replays the graph of its rounded shape (a padding entry fills it up):
    the logits are the plain implementation's, the padding leaves no trace in the cache, and a continuation over the
    same slots reads what the replays wrote."""
    from qwenforge_b200.engine import Model
    name = "small_64"
    model = Model.from_dir(folders[name][0], torch.bfloat16, "cuda")
    model.enable_prefill_graphs()
    vocab = ALL_CONFIGS[name]["vocab_size"]
    cache = model.new_cache(4096, 4)
    held = []
    for turn, (na, nb) in enumerate([(150, 70), (133, 101), (158, 49), (140, 97)]):   # 220 .. 237 tokens: all 256 rounded
        a, b = random_tokens(vocab, na, 1200 + turn), random_tokens(vocab, nb, 1210 + turn)
        sa, sb = cache.open(), cache.open()
        places = [[0, na // 3, na - 1], [0, nb // 2, nb - 2, nb - 1]]
        logits = model.step(cache, [(sa, a), (sb, b)], want=places)
        model.raise_on_kernel_error()
        assert_logits_close(logits[:3], plain_logits(folders, name, a)[places[0]], torch.bfloat16, f"rounded turn {turn} a")
        assert_logits_close(logits[3:], plain_logits(folders, name, b)[places[1]], torch.bfloat16, f"rounded turn {turn} b")
        assert cache.lengths[sa] == na and cache.lengths[sb] == nb
        if turn < 3:
            cache.close(sa)
            cache.close(sb)
        else:
            held = [(sa, a), (sb, b)]
    assert model.prefill_graphs.replays == 3 and len(model.prefill_graphs.graphs) == 1
    more = [random_tokens(vocab, 5, 1230), random_tokens(vocab, 9, 1231)]
    logits = model.step(cache, [(held[0][0], more[0]), (held[1][0], more[1])])
    model.raise_on_kernel_error()
    for row, ((_, first), rest) in enumerate(zip(held, more)):
        assert_logits_close(logits[row:row + 1], plain_logits(folders, name, first + rest)[-1:], torch.bfloat16, f"rounded continuation {row}")


def test_a_capture_survives_the_cycle_collector(folders):
    """An older graph that sits in a reference cycle is destroyed when Python's cycle collector runs; CUDA forbids that
    call while a stream captures and ends the capture with an error. Here such a cycle is made and dropped in the
    middle of a capture, and enough young objects follow it for the collector to run: the capture must hold it off."""
    import gc

    from qwenforge_b200.engine import Model
    from qwenforge_b200.engine.graphs import DecodeGraph
    from qwenforge_b200.sampling import Sampler
    model = Model.from_dir(folders["tiny_a"][0], torch.bfloat16, "cuda")
    cache = model.new_cache(512, 2)
    old = torch.cuda.CUDAGraph()
    counter = torch.zeros(8, device="cuda")
    with torch.cuda.graph(old, stream=torch.cuda.Stream()):
        counter += 1
    holder = [old]
    del old
    graph = DecodeGraph(model, cache, 2, 256, Sampler())
    calls, young = [], []

    def let_go(index, hidden, delta):
        calls.append(index)
        if len(calls) == 2 * (len(model.spec.schedule) + 1) + 1:   # the first call of the third step: the captured one
            ring = [holder.pop()]
            ring.append(ring)   # a cycle: only the collector frees it
            del ring
        young.extend([] for _ in range(200))

    saved = gc.get_threshold()
    model.observer = let_go
    try:
        gc.set_threshold(50, 1000, 1000)
        graph.capture()
    finally:
        gc.set_threshold(*saved)
        model.observer = None
    assert not holder and len(calls) == 3 * (len(model.spec.schedule) + 1)
    slot = cache.open()
    cache.reserve([(slot, 8)])
    model.step(cache, [(slot, [3, 1, 4])])
    cache.flush()
    graph.load([slot], [5], [3], [1], [1 << 30], [0], [])
    graph.run(1)
    model.raise_on_kernel_error()
    assert torch.isfinite(graph.last_logits).all()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_a", "tiny_b"])
def test_greedy_generation_through_entry_point(folders, name, dtype):
    from qwenforge_b200.engine import StudentEngine
    engine = StudentEngine(str(folders[name][0]), device="cuda", dtype=dtype)
    vocab = ALL_CONFIGS[name]["vocab_size"]
    prompts = [random_tokens(vocab, n, 400 + n) for n in (5, 11, 17, 1, 30)]
    got = engine.generate_ids(prompts, max_new_tokens=12, batch_size=3, ignore_eos=True)
    assert [len(t) for t in got] == [12] * 5
    assert engine.graph_decoder.graphs, "a budget of 12 tokens must decode from a captured graph"
    if dtype == "float32":
        want = [plain.greedy_generate(ALL_CONFIGS[name], folders[name][1], p, 12) for p in prompts]
        assert got == want
    else:  # bfloat16 may legitimately leave the greedy path at a near-tie: check every step's choice against the
        for p, out in zip(prompts, got):  # plain logits of the sequence the engine actually produced
            ref = plain.forward_logits(ALL_CONFIGS[name], folders[name][1], p + out)[len(p) - 1:-1]
            for r, token in zip(ref, out):
                assert float(r.max() - r[token]) <= 2e-2 + 4e-2 * float(r.abs().max())
    # stop tokens: generation ends with the first stop token, which is kept
    stop = got[0][2]
    again = engine.generate_ids(prompts[:1], max_new_tokens=12, stop_token_ids=[stop])
    assert again[0] == got[0][:got[0].index(stop) + 1]
    # strings in, strings out, in the reference's contract
    texts = engine.generate(["hello", "a b c"], max_new_tokens=4, batch_size=2)
    assert isinstance(texts, list) and len(texts) == 2 and all(isinstance(t, str) and t for t in texts)
    assert engine.generate([], 4) == [] and engine.generate(["x"], 0) == [""]


@pytest.mark.parametrize("preset,seed,lengths,steps", [("tiny-a", 0, (5, 11, 17), 8), ("tiny-b", 1, (1, 7, 19, 33), 12)])
def test_the_two_tiny_workloads_as_they_are_written(preset, seed, lengths, steps, tmp_path):
    """The two tiny configurations exactly as the package's presets hold them (maximum positions 128 and 256), weights
    from the package's random mode with the workload's seed, the workload's batch of unequal prompts and decode steps,
    float32: the tokens and the logits of the plain implementation."""
    from qwenforge_b200.config import preset_config
    from qwenforge_b200.engine import Model, StudentEngine
    from qwenforge_b200.weights import SafetensorsFile, write_random_model
    config = preset_config(preset)
    write_random_model(config, seed, tmp_path, torch.float32)
    with SafetensorsFile(tmp_path / "model.safetensors") as f:
        weights = {name: f.tensor(name) for name in f.names()}
    data = config.to_dict()
    prompts = [random_tokens(config.vocab_size, n, 40 + n) for n in lengths]
    engine = StudentEngine(str(tmp_path), device="cuda", dtype="float32")
    got = engine.generate_ids(prompts, steps + 1, batch_size=len(prompts), ignore_eos=True)
    want = [plain.greedy_generate(data, weights, p, steps + 1) for p in prompts]
    assert got == want
    model = Model.from_dir(tmp_path, torch.float32, "cuda")
    cache = model.new_cache(64 * len(prompts), len(prompts))
    slots = [cache.open() for _ in prompts]
    logits = model.step(cache, list(zip(slots, prompts)))
    for row, p in enumerate(prompts):
        assert_logits_close(logits[row:row + 1], plain.forward_logits(data, weights, p)[-1:], torch.float32, f"{preset} prompt {len(p)}")


def test_temperature_sampling_is_independent_of_batching(folders):
    from qwenforge_b200.engine import StudentEngine
    engine = StudentEngine(str(folders["tiny_a"][0]), device="cuda", dtype="float32", seed=5)
    prompts = [random_tokens(256, n, 500 + n) for n in (4, 9, 2, 13)]
    together = engine.generate_ids(prompts, 10, batch_size=4, temperature=0.9, ignore_eos=True)
    apart = engine.generate_ids(prompts, 10, batch_size=1, temperature=0.9, ignore_eos=True)
    assert together == apart
    other_seed = engine.generate_ids(prompts, 10, batch_size=4, temperature=0.9, seed=6, ignore_eos=True)
    assert other_seed != together
    greedy = engine.generate_ids(prompts, 10, batch_size=4, ignore_eos=True)
    assert greedy != together


def check_choices(name, folders, prompts, results, temperature, seed, what):
    """Every token that a bfloat16 run chose must be (within the logits' tolerance) the best choice by the plain
    implementation's logits of the sequence that the run actually produced: the argmax when greedy, else the best
    Gumbel-perturbed score of (seed, request index, step)."""
    config, weights = ALL_CONFIGS[name], folders[name][1]
    for index, (prompt, result) in enumerate(zip(prompts, results)):
        out = result.tokens
        ref = plain.forward_logits(config, weights, prompt + out)[len(prompt) - 1:-1]
        margin = 2e-2 + 4e-2 * float(ref.abs().max())
        for step, (row, token) in enumerate(zip(ref, out)):
            _, scores = plain.sample_token(row, temperature, seed, index, step)
            lost = float(scores.max() - scores[token]) * (temperature if temperature > 0 else 1.0)
            assert lost <= margin, f"{what}: request {index} step {step} chose {token}, {lost:.3e} below the best"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["tiny_b", "tiny_w", "small_64", "small_128"])
def test_graph_decoding_equals_stepping(folders, name, dtype):
    """Decode steps replayed from CUDA graphs give the tokens of step-by-step decoding: unequal prompts, budgets that
    end at different steps, a stop token, several chunks of replays, and a second batch that reuses the graph. In
    bfloat16, where two attention split shapes may break a near-tie differently, every chosen token of both runs is
    checked against the plain implementation's logits instead."""
    from qwenforge_b200.engine import StudentEngine
    vocab = ALL_CONFIGS[name]["vocab_size"]
    prompts = [random_tokens(vocab, n, 600 + n) for n in (5, 70, 17, 1, 64)]
    budgets = [80, 12, 45, 9, 33]
    eager = StudentEngine(str(folders[name][0]), device="cuda", dtype=dtype, cuda_graphs=False)
    graphed = StudentEngine(str(folders[name][0]), device="cuda", dtype=dtype, cuda_graphs=True)
    for temperature in (0.0, 0.8):
        want = eager.generate_results(prompts, budgets, batch_size=5, temperature=temperature, ignore_eos=True)
        got = graphed.generate_results(prompts, budgets, batch_size=5, temperature=temperature, ignore_eos=True)
        assert graphed.graph_decoder.graphs, "no graph was captured"
        assert [len(r.tokens) for r in got] == budgets
        if dtype == "float32":
            assert [r.tokens for r in got] == [r.tokens for r in want]
        else:
            check_choices(name, folders, prompts, got, temperature, 0, f"{name} graph T={temperature}")
            check_choices(name, folders, prompts, want, temperature, 0, f"{name} stepping T={temperature}")
    stop = want[0].tokens[20]
    a = eager.generate_results(prompts, budgets, batch_size=5, temperature=0.8, stop_token_ids=[stop])
    b = graphed.generate_results(prompts, budgets, batch_size=5, temperature=0.8, stop_token_ids=[stop])
    if dtype == "float32":
        assert [(r.tokens, r.finish_reason) for r in a] == [(r.tokens, r.finish_reason) for r in b]
        assert b[0].finish_reason == "stop" and b[0].tokens[-1] == stop
    assert not graphed.cache.live_slots()
    assert all(g.pages.n_free == g.pages.n_pages for g in graphed.cache.kv_groups)
    n_graphs = len(graphed.graph_decoder.graphs)
    graphed.generate_results(prompts, budgets, batch_size=5, temperature=0.8, ignore_eos=True)
    assert len(graphed.graph_decoder.graphs) == n_graphs       # the same key: replayed, not captured again


@pytest.mark.parametrize("preset,layers", [("qwen2.5-0.5b", 2), ("qwen2.5-3b", 1), ("qwen2.5-7b", 1)])
def test_real_layer_sizes(preset, layers, tmp_path):
    """The layer sizes of the three Qwen2.5 models (head size 64 and 128, groups of 7, 8 and 7, widths 896/2048/3584,
    intermediate 4864/11008/18944) with few layers and a small vocabulary, in float32 and bfloat16, against the plain
    implementation: a whole prompt, a batch of unequal prompts, and tokens decoded one by one."""
    import json

    from qwenforge_b200.config import preset_dict
    from qwenforge_b200.engine import Model
    from qwenforge_b200.weights import save_safetensors
    config = dict(preset_dict(preset), num_hidden_layers=layers, vocab_size=1000, max_position_embeddings=512)
    weights = plain.random_weights(config, 9)
    (tmp_path / "config.json").write_text(json.dumps(config))
    save_safetensors(tmp_path / "model.safetensors", weights)
    seqs = [random_tokens(1000, n, 700 + n) for n in (70, 9)]
    refs = [plain.forward_logits(config, weights, s, dtype=torch.float32) for s in seqs]
    for dtype in DTYPES:
        model = Model.from_dir(tmp_path, dtype, "cuda")
        cache = model.new_cache(512, 4)
        slots = [cache.open() for _ in seqs]
        heads = [len(s) - 6 for s in seqs]
        got = [[] for _ in seqs]
        logits = model.step(cache, [(slot, s[:h]) for slot, s, h in zip(slots, seqs, heads)],
                            want=[list(range(h)) for h in heads])
        got[0].append(logits[:heads[0]])
        got[1].append(logits[heads[0]:])
        for t in range(6):
            logits = model.step(cache, [(slot, [s[h + t]]) for slot, s, h in zip(slots, seqs, heads)])
            got[0].append(logits[0:1])
            got[1].append(logits[1:2])
        model.raise_on_kernel_error()
        for pieces, ref in zip(got, refs):
            rel, abs_ = (1e-4, 1e-5) if dtype == torch.float32 else (4e-2, 2e-2)   # the oracle is float32 here
            bound = abs_ + rel * float(ref.abs().max())
            err = float((torch.cat(pieces).double().cpu() - ref.double()).abs().max())
            assert err <= bound, f"{preset} {dtype}: {err:.3e} > {bound:.3e}"
        del model, cache
        torch.cuda.empty_cache()


def test_long_prompt_through_the_persistent_gate_product(tmp_path):
    """A prompt long enough that the gate/up product has tiles for every SM runs it on the persistent tcgen05 kernel
    with the gate in its epilogue (Qwen2.5-0.5B layer sizes, one layer): launch by launch, then replayed from a graph
    of its rounded shape with other tokens, against the plain implementation."""
    import json

    from qwenforge_b200 import ops
    from qwenforge_b200.config import preset_dict
    from qwenforge_b200.engine import Model
    from qwenforge_b200.weights import save_safetensors
    config = dict(preset_dict("qwen2.5-0.5b"), num_hidden_layers=1, vocab_size=1000, max_position_embeddings=1024)
    weights = plain.random_weights(config, 11)
    (tmp_path / "config.json").write_text(json.dumps(config))
    save_safetensors(tmp_path / "model.safetensors", weights)
    model = Model.from_dir(tmp_path, torch.bfloat16, "cuda")
    model.enable_prefill_graphs()
    cache = model.new_cache(2048, 2)
    places = [0, 1, 63, 64, 127, 128, 300, 511, 512, 640]
    for turn, n in enumerate((700, 690, 650)):
        assert ops.tc_gemm_is_persistent(ops.TC_SWIGLU, n, 2 * config["intermediate_size"])
        tokens = random_tokens(1000, n, 800 + turn)
        slot = cache.open()
        logits = model.step(cache, [(slot, tokens)], want=[places + [n - 1]])
        model.raise_on_kernel_error()
        ref = plain.forward_logits(config, weights, tokens, dtype=torch.float32)[places + [n - 1]]
        bound = 2e-2 + 4e-2 * float(ref.abs().max())
        err = float((logits.double().cpu() - ref.double()).abs().max())
        assert err <= bound, f"turn {turn}: {err:.3e} > {bound:.3e}"
        cache.close(slot)
    assert model.prefill_graphs.replays == 2


def test_own_tensor_core_products_in_the_model(folders):
    """With the library's own tcgen05 products switched on, a 200-token prompt gives the plain implementation's logits."""
    from qwenforge_b200 import ops
    model = get_model(folders, "small_64", torch.bfloat16)
    tokens = random_tokens(ALL_CONFIGS["small_64"]["vocab_size"], 200, 900)
    ref = plain_logits(folders, "small_64", tokens)
    ops.use_own_tensor_core_products(True)
    try:
        cache = model.new_cache(512, 2)
        slot = cache.open()
        before = ops.kernels.launches
        logits = model.step(cache, [(slot, tokens)], want=[list(range(200))])
        model.raise_on_kernel_error()
    finally:
        ops.use_own_tensor_core_products(False)
    assert_logits_close(logits, ref, torch.bfloat16, "own tcgen05 products")


@pytest.mark.parametrize("name", ["small_64", "small_128"])
def test_tcgen05_prefill_attention_in_the_model(folders, name, monkeypatch):
    """With the tcgen05 prefill attention chosen for every step of 128 rows or more: a batch of unequal prompts, then a
    continuation over the cache it left, give the plain implementation's logits."""
    from qwenforge_b200.parts import attention
    monkeypatch.setattr(attention, "TC_PREFILL_MIN_TOKENS", {64: 1, 128: 1})
    model = get_model(folders, name, torch.bfloat16)
    vocab = ALL_CONFIGS[name]["vocab_size"]
    limit = ALL_CONFIGS[name]["max_position_embeddings"]
    long_n = min(200, limit - 140)
    a, b = random_tokens(vocab, long_n, 910), random_tokens(vocab, 130, 911)
    more = random_tokens(vocab, 135, 912)
    cache = model.new_cache(1024, 4)
    sa, sb = cache.open(), cache.open()
    logits = model.step(cache, [(sa, a), (sb, b)], want=[list(range(long_n)), list(range(130))])
    model.raise_on_kernel_error()
    assert_logits_close(logits[:long_n], plain_logits(folders, name, a), torch.bfloat16, f"{name} tcgen05 prefill a")
    assert_logits_close(logits[long_n:], plain_logits(folders, name, b), torch.bfloat16, f"{name} tcgen05 prefill b")
    cache.close(sb)
    logits = model.step(cache, [(sa, more)], want=[list(range(135))])
    model.raise_on_kernel_error()
    whole = plain_logits(folders, name, a + more)
    assert_logits_close(logits, whole[long_n:], torch.bfloat16, f"{name} tcgen05 continuation")
    cache.close(sa)


def test_prefill_graphs_replay_equals_the_plain_implementation(folders):
    """Steps of whole prompts are captured the second time their shape comes and replayed from then on: other
    tokens, other slots, other start positions through the same graph give the plain implementation's logits."""
    from qwenforge_b200.engine import Model
    name = "small_64"
    model = Model.from_dir(folders[name][0], torch.bfloat16, "cuda")
    model.enable_prefill_graphs()
    assert model.prefill_graphs is not None
    vocab = ALL_CONFIGS[name]["vocab_size"]
    cache = model.new_cache(2048, 4)
    for turn in range(4):
        a, b = random_tokens(vocab, 70, 950 + turn), random_tokens(vocab, 130, 960 + turn)
        slots = [cache.open(), cache.open()]
        if turn % 2:
            slots.reverse()   # the same shape with the sequences in other slots
        logits = model.step(cache, [(slots[0], a), (slots[1], b)], want=[[0, 69], list(range(130))])
        model.raise_on_kernel_error()
        assert_logits_close(logits[:2], plain_logits(folders, name, a)[[0, 69]], torch.bfloat16, f"graph turn {turn} a")
        assert_logits_close(logits[2:], plain_logits(folders, name, b), torch.bfloat16, f"graph turn {turn} b")
        if turn == 3:  # a continuation of the same shape: 70 and 130 further tokens after 70 and 130
            more_a, more_b = random_tokens(vocab, 70, 970), random_tokens(vocab, 130, 971)
            logits = model.step(cache, [(slots[0], more_a), (slots[1], more_b)], want=[[0, 69], list(range(130))])
            model.raise_on_kernel_error()
            assert_logits_close(logits[:2], plain_logits(folders, name, a + more_a)[[70, 139]], torch.bfloat16, "graph continuation a")
            assert_logits_close(logits[2:], plain_logits(folders, name, b + more_b)[130:], torch.bfloat16, "graph continuation b")
        for slot in slots:
            cache.close(slot)
    assert model.prefill_graphs.replays == 4   # turns 1, 2, 3 and the continuation; turn 0 ran launch by launch
