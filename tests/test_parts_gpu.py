"""Each part of a layer alone against the plain implementation's function for it; the schedule as data (a layer
run twice, an entry that reads another entry's cache); and parts defined HERE (a mixer with state of its own,
another position encoding, a whole toy architecture) registered, built and stepped without touching the package."""
import json
from dataclasses import dataclass

import pytest
import torch

from tests import plain_qwen2 as plain
from tests.helpers import TINY_B, max_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 3e-5 if dtype == torch.float32 else 3e-2


def rand(shape, seed, scale=1.0):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)) * scale


def bind(part, tensors, dtype):
    from qwenforge_b200.csrc import prepare
    libs = set()
    stack = [part]
    while stack:
        p = stack.pop()
        libs |= p.kernel_libraries(dtype)
        stack += p.sub_parts()
    prepare(libs)
    on_device = {k: v.to(DEV, dtype) for k, v in tensors.items()}
    stack = [part]
    while stack:
        p = stack.pop()
        p.bind(on_device, dtype, DEV)
        stack += p.sub_parts()
    return part


def context(entries, dtype, want=None):
    from qwenforge_b200.engine import build_context
    err = torch.zeros(1, dtype=torch.int32, device=DEV)
    return build_context(entries, want, err, dtype, DEV)


@pytest.mark.parametrize("dtype", DTYPES)
def test_rms_norm_part(dtype):
    from qwenforge_b200.config import PartSpec
    from qwenforge_b200.parts import build_part
    w = 1 + rand((120,), 0, 0.1)
    part = bind(build_part("norm", PartSpec("rms_norm", {"width": 120, "eps": 1e-5}, {"weight": "n.w"})), {"n.w": w}, dtype)
    hidden = rand((7, 120), 1, 2.0).to(DEV)
    delta = rand((7, 120), 2).to(DEV, dtype)
    want = plain.rms_norm(hidden.double().cpu() + delta.double().cpu(), w.to(dtype).double(), 1e-5)
    got = part.forward(hidden, delta)
    assert got.dtype == dtype and max_err(got, want) <= tol(dtype) * float(want.abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu_part(dtype):
    from qwenforge_b200.config import PartSpec
    from qwenforge_b200.parts import build_part
    t = {"g": rand((200, 120), 3, 0.05), "u": rand((200, 120), 4, 0.05), "d": rand((120, 200), 5, 0.05)}
    part = bind(build_part("feed_forward", PartSpec("swiglu", {"hidden_size": 120, "intermediate_size": 200},
                                                    {"gate_weight": "g", "up_weight": "u", "down_weight": "d"})), t, dtype)
    x = rand((9, 120), 6).to(DEV, dtype)
    w = {"p.gate_proj.weight": t["g"].to(dtype).double(), "p.up_proj.weight": t["u"].to(dtype).double(),
         "p.down_proj.weight": t["d"].to(dtype).double()}
    want = plain.swiglu_mlp(x.double().cpu(), w, "p.")
    assert max_err(part.forward(x, None), want) <= tol(dtype) * max(1.0, float(want.abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding_and_head_parts(dtype):
    from qwenforge_b200.config import PartSpec
    from qwenforge_b200.parts import build_part
    table = rand((50, 24), 7)
    emb = bind(build_part("embedding", PartSpec("token_embedding", {"vocab_size": 50, "width": 24}, {"weight": "e"})),
               {"e": table}, dtype)
    head = bind(build_part("head", PartSpec("linear_head", {"vocab_size": 50, "width": 24, "tied": True}, {"weight": "e"})),
                {"e": table}, dtype)
    ctx = context([(0, 0, [3, 49, 0])], dtype)
    hidden = emb.forward(ctx.token_ids, ctx)
    assert hidden.dtype == torch.float32 and torch.equal(hidden.cpu(), table.to(dtype).float()[[3, 49, 0]])
    x = rand((4, 24), 8).to(DEV, dtype)
    logits = head.forward(x)
    want = x.double().cpu() @ table.to(dtype).double().T
    assert logits.dtype == torch.float32 and max_err(logits, want) <= tol(dtype) * float(want.abs().max())


def attention_tensors(hidden, nh, kvh, d, seed):
    return {"q.w": rand((nh * d, hidden), seed, 0.2), "q.b": rand((nh * d,), seed + 1, 0.2),
            "k.w": rand((kvh * d, hidden), seed + 2, 0.2), "k.b": rand((kvh * d,), seed + 3, 0.2),
            "v.w": rand((kvh * d, hidden), seed + 4, 0.2), "v.b": rand((kvh * d,), seed + 5, 0.2),
            "o.w": rand((hidden, nh * d), seed + 6, 0.2)}


def attention_spec(hidden, nh, kvh, d, window, theta):
    from qwenforge_b200.config import PartSpec
    return PartSpec("gqa_attention",
                    {"hidden_size": hidden, "num_heads": nh, "num_kv_heads": kvh, "head_dim": d, "qkv_bias": True,
                     "scale": d ** -0.5, "window": window,
                     "position": PartSpec("rotary_half", {"head_dim": d, "theta": theta})},
                    {"q_weight": "q.w", "q_bias": "q.b", "k_weight": "k.w", "k_bias": "k.b", "v_weight": "v.w",
                     "v_bias": "v.b", "o_weight": "o.w"})


def plain_attention_part(x, t, nh, kvh, d, window, theta, dtype):
    w = {"a.q_proj.weight": t["q.w"], "a.q_proj.bias": t["q.b"], "a.k_proj.weight": t["k.w"], "a.k_proj.bias": t["k.b"],
         "a.v_proj.weight": t["v.w"], "a.v_proj.bias": t["v.b"]}
    w = {k: v.to(dtype).double() for k, v in w.items()}
    q, k, v = plain.project_qkv(x, w, "a.", nh, kvh, d)
    cos, sin = plain.rope_cos_sin(torch.arange(x.shape[0]), d, theta, torch.float64)
    ctx = plain.attention(plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin), v, window)
    return ctx.transpose(0, 1).reshape(x.shape[0], nh * d) @ t["o.w"].to(dtype).double().T


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,nh,kvh,d,window", [(40, 6, 2, 8, 0), (33, 3, 3, 24, 0), (64, 8, 1, 16, 21)])
def test_attention_part_whole_and_in_pieces(dtype, hidden, nh, kvh, d, window):
    from qwenforge_b200.cache import SequenceCache
    from qwenforge_b200.parts import build_part
    t = attention_tensors(hidden, nh, kvh, d, 20)
    part = bind(build_part("mixer", attention_spec(hidden, nh, kvh, d, window, 777.0)), t, dtype)
    cache = SequenceCache([part.cache_need()], 1024, 4, 512, dtype, DEV)
    n = 90
    x = rand((n, hidden), 30).to(dtype)
    want = plain_attention_part(x.double(), t, nh, kvh, d, window, 777.0, dtype)
    bound = tol(dtype) * float(want.abs().max()) * 2
    slot = cache.open()
    cache.reserve([(slot, n)])
    cache.flush()
    got = part.forward(x.to(DEV), context([(slot, 0, [0] * n)], dtype), cache.site(0), True)
    assert max_err(got, want) <= bound
    # the same tokens in pieces of 64 + 25 + 1, beside another sequence
    other, again = cache.open(), cache.open()
    cache.reserve([(other, 10), (again, n)])
    cache.flush()
    pieces = []
    start = 0
    for size in (64, 25, 1):
        ctx = context([(other, start % 5, [0]), (again, start, [0] * size)], dtype)
        xs = torch.cat((x[:1], x[start:start + size])).to(DEV)
        pieces.append(part.forward(xs, ctx, cache.site(0), True)[1:])
        cache.advance(again, size)
        start += size
    assert max_err(torch.cat(pieces), want) <= bound
    assert int(ctx.err) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_pre_norm_block(dtype):
    from qwenforge_b200.cache import SequenceCache
    from qwenforge_b200.config import config_from_dict
    from qwenforge_b200.parts import build_block
    config = dict(TINY_B, num_hidden_layers=1)
    spec = config_from_dict(config).model_spec()
    weights = plain.random_weights(config, 3)
    block = bind(build_block(spec.layers[0]), weights, dtype)
    cache = SequenceCache([block.cache_need()], 512, 2, 256, dtype, DEV)
    n = 21
    h0 = rand((n, 120), 40)
    delta0 = rand((n, 120), 41, 0.1).to(dtype)
    sizes = plain.read_sizes(config)
    cos, sin = plain.rope_cos_sin(torch.arange(n), sizes["head_dim"], sizes["theta"], torch.float64)
    w64 = {k: v.to(dtype).double() for k, v in weights.items()}
    want = plain.decoder_layer(h0.double() + delta0.double(), w64, 0, sizes, cos, sin)
    slot = cache.open()
    cache.reserve([(slot, n)])
    cache.flush()
    hidden = h0.to(DEV)
    delta = block.forward(hidden, delta0.to(DEV), context([(slot, 0, [0] * n)], dtype), cache.site(0), True)
    got = hidden.double() if delta is None else hidden.double() + delta.double()   # a part may have added in place
    assert max_err(got, want) <= tol(dtype) * float(want.abs().max()) * 2


# ------------------------------------------------------------------------------------------------ the schedule as data

def plain_schedule_model(config, weights, tokens, schedule):
    """Plain forward for a schedule of (layer, cache_from) entries: an entry with cache_from attends with its own
    queries to the keys and values that entry `cache_from` computed."""
    sizes = plain.read_sizes(config)
    w = {k: v.double() for k, v in weights.items()}
    h = w["model.embed_tokens.weight"][torch.tensor(tokens)]
    cos, sin = plain.rope_cos_sin(torch.arange(len(tokens)), sizes["head_dim"], sizes["theta"], torch.float64)
    kept = {}
    for pos, (layer, cache_from) in enumerate(schedule):
        p = f"model.layers.{layer}."
        n = plain.rms_norm(h, w[p + "input_layernorm.weight"], sizes["eps"])
        q, k, v = plain.project_qkv(n, w, p + "self_attn.", sizes["heads"], sizes["kv_heads"], sizes["head_dim"])
        q, k = plain.apply_rope(q, cos, sin), plain.apply_rope(k, cos, sin)
        if cache_from is None:
            kept[pos] = (k, v)
        else:
            k, v = kept[cache_from]
        ctx = plain.attention(q, k, v).transpose(0, 1).reshape(len(tokens), -1)
        h = h + ctx @ w[p + "self_attn.o_proj.weight"].T
        n = plain.rms_norm(h, w[p + "post_attention_layernorm.weight"], sizes["eps"])
        h = h + plain.swiglu_mlp(n, w, p + "mlp.")
    h = plain.rms_norm(h, w["model.norm.weight"], sizes["eps"])
    return h @ w["lm_head.weight"].T


def test_schedule_names_a_layer_twice_and_shares_a_cache():
    import dataclasses

    from qwenforge_b200.config import ScheduleEntry, config_from_dict
    from qwenforge_b200.engine import Model
    config = dict(TINY_B, num_hidden_layers=2)
    weights = plain.random_weights(config, 5)
    schedule = [(0, None), (1, None), (0, None), (1, 1)]   # layer 0 twice (own caches); the last run reads entry 1's cache
    spec = dataclasses.replace(config_from_dict(config).model_spec(),
                               schedule=tuple(ScheduleEntry(a, b) for a, b in schedule))
    model = Model(spec, torch.float32, DEV)
    assert [n is not None for n in model.cache_needs()] == [True, True, True, False]
    model.bind({k: v.to(DEV) for k, v in weights.items()})
    cache = model.new_cache(512, 2)
    assert cache.kv_groups[0].storage.shape[0] == 3       # three caches for four runs
    tokens = [int(t) for t in torch.randint(0, 384, (75,), generator=torch.Generator().manual_seed(6))]
    want = plain_schedule_model(config, weights, tokens, schedule)
    slot = cache.open()
    got = [model.step(cache, [(slot, tokens[:70])], want=[list(range(70))])]
    for t in tokens[70:]:
        got.append(model.step(cache, [(slot, [t])]))
    model.raise_on_kernel_error()
    assert max_err(torch.cat(got), want) <= 3e-5 * float(want.abs().max())
    with pytest.raises(ValueError, match="does not run before"):
        dataclasses.replace(spec, schedule=(ScheduleEntry(0, 1), ScheduleEntry(1))).validate()


# ------------------------------------------------------------------------------------------------ toy parts, defined here

def register_toy_parts():
    """A mixer with state of its own (an exponentially decayed sum of projected inputs), another position encoding
    (queries and keys scaled by a function of the position: no fused form, so the mixer calls `apply`), and an
    architecture that uses them in some layers and the stock attention in others. Nothing of the package is edited."""
    from qwenforge_b200.cache import StateNeed
    from qwenforge_b200.config import (LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry, register_architecture)
    from qwenforge_b200.parts import Mixer, PositionEncoding, TensorSpec, register_part

    class DecayedSum(Mixer):
        graph_safe = False   # its forward plans on the host, so decode steps are not captured into CUDA graphs

        def __init__(self, spec):
            super().__init__(spec)
            self.width, self.inner, self.decay = self.params["width"], self.params["inner"], self.params["decay"]

        def tensor_specs(self):
            return [TensorSpec(self.file_name("in"), (self.inner, self.width)),
                    TensorSpec(self.file_name("out"), (self.width, self.inner)),
                    TensorSpec(self.file_name("gain"), (self.inner,), init="norm", keep="stored")]

        def cache_need(self):
            return StateNeed((self.inner,), torch.float32)

        def bind(self, tensors, dtype, device):
            self.w_in, self.w_out = tensors[self.file_name("in")], tensors[self.file_name("out")]
            self.gain = tensors[self.file_name("gain")]
            assert self.gain.dtype == torch.float32   # stored in 32 bits: stays so, also on the bfloat16 path

        def forward(self, x, ctx, site, writes_cache):
            from qwenforge_b200 import ops
            u = ops.linear(x, self.w_in).float() * self.gain
            states = torch.empty_like(u)
            begin = 0
            for slot, q_len in zip(ctx.host_slots, ctx.host_q_lens):
                state = site.storage[slot] if slot >= 0 else torch.zeros(self.inner, device=x.device)
                for t in range(begin, begin + q_len):       # in order over the span: whole and piecewise agree
                    state = self.decay * state + u[t]
                    states[t] = state
                if slot >= 0:
                    site.storage[slot] = state
                begin += q_len
            return ops.linear(states.to(x.dtype), self.w_out)

    class PositionGain(PositionEncoding):
        def apply(self, q, k, ctx):
            gain = (1.0 + self.params["slope"] * ctx.tok_pos.float()).view(-1, 1, 1)
            q.copy_((q.float() * gain).to(q.dtype))
            k.copy_((k.float() / gain).to(k.dtype))

    register_part("mixer", "toy_decayed_sum", DecayedSum)
    register_part("position", "toy_position_gain", PositionGain)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        vocab_size: int
        width: int
        inner: int
        decay: float
        slope: float
        eps: float
        n_layers: int
        architecture = "ToyMixedForCausalLM"

        @classmethod
        def from_dict(cls, data):
            return cls(*(data[k] for k in ("vocab_size", "width", "inner", "decay", "slope", "eps", "n_layers")))

        def to_dict(self):
            return dict(architectures=[self.architecture], vocab_size=self.vocab_size, width=self.width, inner=self.inner,
                        decay=self.decay, slope=self.slope, eps=self.eps, n_layers=self.n_layers)

        def model_spec(self):
            def norm(name):
                return PartSpec("rms_norm", {"width": self.width, "eps": self.eps}, {"weight": name})
            layers = []
            for i in range(self.n_layers):
                p = f"blocks.{i}."
                if i % 2 == 0:
                    mixer = PartSpec("toy_decayed_sum", {"width": self.width, "inner": self.inner, "decay": self.decay},
                                     {"in": p + "mix.in", "out": p + "mix.out", "gain": p + "mix.gain"})
                else:
                    mixer = PartSpec("gqa_attention",
                                     {"hidden_size": self.width, "num_heads": 4, "num_kv_heads": 2, "head_dim": 8,
                                      "qkv_bias": False, "window": 0,
                                      "position": PartSpec("toy_position_gain", {"slope": self.slope})},
                                     {"q_weight": p + "q", "k_weight": p + "k", "v_weight": p + "v", "o_weight": p + "o"})
                ffn = PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": 2 * self.width},
                               {"gate_weight": p + "ff.g", "up_weight": p + "ff.u", "down_weight": p + "ff.d"})
                layers.append(LayerSpec("pre_norm", {"mixer_norm": norm(p + "n1"), "mixer": mixer,
                                                    "feed_forward_norm": norm(p + "n2"), "feed_forward": ffn}))
            return ModelSpec("ToyMixedForCausalLM", self.vocab_size, self.width, 4096,
                             PartSpec("token_embedding", {"vocab_size": self.vocab_size, "width": self.width}, {"weight": "emb"}),
                             tuple(layers), tuple(ScheduleEntry(i) for i in range(self.n_layers)), norm("final"),
                             PartSpec("linear_head", {"vocab_size": self.vocab_size, "width": self.width, "tied": True},
                                      {"weight": "emb"}))

    try:
        register_architecture("ToyMixedForCausalLM", ToyConfig)
    except ValueError:
        pass
    return ToyConfig


def plain_toy_model(cfg, w, tokens, dtype):
    """The toy architecture on a whole sequence, in float64, with `dtype`-rounded weights."""
    w = {k: (v if v.dtype == torch.float32 and k.endswith("gain") else v.to(dtype)).double() for k, v in w.items()}
    n = len(tokens)
    h = w["emb"][torch.tensor(tokens)]
    pos = torch.arange(n, dtype=torch.float64)
    for i in range(cfg.n_layers):
        p = f"blocks.{i}."
        x = plain.rms_norm(h, w[p + "n1"], cfg.eps)
        if i % 2 == 0:
            u = (x @ w[p + "mix.in"].T) * w[p + "mix.gain"]
            state = torch.zeros(cfg.inner, dtype=torch.float64)
            states = []
            for t in range(n):
                state = cfg.decay * state + u[t]
                states.append(state)
            h = h + torch.stack(states) @ w[p + "mix.out"].T
        else:
            gain = (1.0 + cfg.slope * pos).view(1, n, 1)
            q = (x @ w[p + "q"].T).view(n, 4, 8).transpose(0, 1) * gain
            k = (x @ w[p + "k"].T).view(n, 2, 8).transpose(0, 1) / gain
            v = (x @ w[p + "v"].T).view(n, 2, 8).transpose(0, 1)
            h = h + plain.attention(q, k, v).transpose(0, 1).reshape(n, 32) @ w[p + "o"].T
        x = plain.rms_norm(h, w[p + "n2"], cfg.eps)
        g, u2 = x @ w[p + "ff.g"].T, x @ w[p + "ff.u"].T
        h = h + (g * torch.sigmoid(g) * u2) @ w[p + "ff.d"].T
    return plain.rms_norm(h, w["final"], cfg.eps) @ w["emb"].T


@pytest.mark.parametrize("dtype", DTYPES)
def test_toy_architecture_registers_builds_and_steps(dtype, tmp_path):
    from qwenforge_b200.engine import Model, StudentEngine
    from qwenforge_b200.weights import SafetensorsFile, write_random_model
    ToyConfig = register_toy_parts()
    cfg = ToyConfig(vocab_size=97, width=32, inner=20, decay=0.9, slope=0.01, eps=1e-5, n_layers=3)
    write_random_model(cfg, 4, tmp_path, torch.float32)        # the package's random mode knows the toy's tensors
    with SafetensorsFile(tmp_path / "model.safetensors") as f:
        weights = {n: f.tensor(n) for n in f.names()}
    assert "blocks.0.mix.gain" in weights and "blocks.1.q" in weights
    model = Model.from_dir(tmp_path, dtype, DEV)               # chosen by config.json's architecture name
    cache = model.new_cache(1024, 3)
    assert len(cache.state_groups) == 1 and len(cache.kv_groups) == 1
    g = torch.Generator().manual_seed(9)
    seqs = [torch.randint(0, 97, (n,), generator=g).tolist() for n in (70, 9, 33)]
    refs = [plain_toy_model(cfg, weights, s, dtype) for s in seqs]
    bound = [tol(dtype) * float(r.abs().max()) * 2 for r in refs]
    # whole, in one unequal batch
    slots = [cache.open() for _ in seqs]
    logits = model.step(cache, list(zip(slots, seqs)), want=[list(range(len(s))) for s in seqs])
    o = 0
    for s, r, b in zip(seqs, refs, bound):
        assert max_err(logits[o:o + len(s)], r) <= b
        o += len(s)
    for s in slots:
        cache.close(s)
    # a prompt, then token by token, in slots that were used before: the state must have been reset
    slots = [cache.open() for _ in seqs]
    got = [[model.step(cache, [(slot, s[:5])], want=[list(range(5))])] for slot, s in zip(slots, seqs)]
    for t in range(5, 70):
        live = [(i, slot) for i, (slot, s) in enumerate(zip(slots, seqs)) if t < len(s)]
        out = model.step(cache, [(slot, [seqs[i][t]]) for i, slot in live])
        for row, (i, _) in enumerate(live):
            got[i].append(out[row:row + 1])
    model.raise_on_kernel_error()
    for pieces, r, b in zip(got, refs, bound):
        assert max_err(torch.cat(pieces), r) <= b
    # and through the entry point
    engine = StudentEngine(str(tmp_path), device=DEV, dtype="float32" if dtype == torch.float32 else "bfloat16")
    out = engine.generate_ids([seqs[1]], 5, ignore_eos=True)
    assert len(out[0]) == 5
