"""More toy parts, defined here and registered from outside the package, to show what the parts' interfaces carry:
a feed-forward with routing (top-2 of 4 small experts, router logits in 32-bit from a tensor kept in 32-bit), a position
encoding that reads positions on two axes from the step's side inputs (`ctx.extras`), and another block arrangement
(one norm, mixer and feed-forward side by side: a parallel residual) that reads other part names from its layer spec.
They are toys: they never become a model of the package's. The package's files are not edited; loader, random
weights, cache, step function and the entry point work from the specs."""
from dataclasses import dataclass

import pytest
import torch

from tests import plain_qwen2 as plain
from tests.helpers import max_err

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]
HEADS, KV_HEADS, HEAD_DIM = 4, 2, 16
WEIGHT_SEED = 7   # of seeds 1..59 the one whose router decisions stay furthest from a tie (3.8e-3), found once on the CPU


def register_toys():
    from qwenforge_b200 import ops
    from qwenforge_b200.config import LayerSpec, ModelConfig, ModelSpec, PartSpec, ScheduleEntry, register_architecture
    from qwenforge_b200.parts import FeedForward, Part, PositionEncoding, TensorSpec, build_part, register_part

    class RoutedExperts(FeedForward):
        """out = sum over the top_k experts e of softmax(router logits of those)_e * W_out_e silu(W_in_e x)."""
        graph_safe = False   # which rows go to which expert is decided on the host

        def __init__(self, spec):
            super().__init__(spec)
            self.width, self.inner = self.params["width"], self.params["inner"]
            self.experts, self.top_k = self.params["experts"], self.params["top_k"]

        def tensor_specs(self):
            specs = [TensorSpec(self.file_name("router"), (self.experts, self.width), keep="stored")]
            for e in range(self.experts):
                specs += [TensorSpec(self.file_name("in").format(e), (self.inner, self.width)),
                          TensorSpec(self.file_name("out").format(e), (self.width, self.inner))]
            return specs

        def kernel_libraries(self, dtype):
            return {"gemm_f32"}

        def bind(self, tensors, dtype, device):
            self.router = tensors[self.file_name("router")]
            assert self.router.dtype == torch.float32
            self.w_in = [tensors[self.file_name("in").format(e)] for e in range(self.experts)]
            self.w_out = [tensors[self.file_name("out").format(e)] for e in range(self.experts)]

        def forward(self, x, ctx):
            logits = ops.linear(x.float(), self.router)                       # router logits in 32-bit
            top, chosen = torch.topk(logits, self.top_k, dim=-1)
            gates = torch.softmax(top, dim=-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e in range(self.experts):
                rows, which = (chosen == e).nonzero(as_tuple=True)
                if rows.numel() == 0:
                    continue
                inner = ops.linear(x[rows].contiguous(), self.w_in[e]).float()
                y = ops.linear((inner * torch.sigmoid(inner)).to(x.dtype), self.w_out[e]).float()
                out.index_add_(0, rows, y * gates[rows, which].unsqueeze(-1))
            return out.to(x.dtype)

    class TwoAxisRotary(PositionEncoding):
        """Half of each head is rotated by the token's row, the other half by its column (`ctx.extras["axes"]`,
        int [T, 2]); no fused form, so the mixer calls `apply`."""
        graph_safe = False   # needs the step's side inputs

        def apply(self, q, k, ctx):
            axes = ctx.extras["axes"].float()
            half, quarter = q.shape[-1] // 2, q.shape[-1] // 4
            freq = 1.0 / (self.params["theta"] ** (torch.arange(quarter, device=q.device, dtype=torch.float32) / quarter))
            for t in (q, k):
                v = t.float()
                for axis in range(2):
                    angle = axes[:, axis, None, None] * freq
                    a = v[..., axis * half:axis * half + quarter].clone()
                    b = v[..., axis * half + quarter:(axis + 1) * half].clone()
                    v[..., axis * half:axis * half + quarter] = a * angle.cos() - b * angle.sin()
                    v[..., axis * half + quarter:(axis + 1) * half] = b * angle.cos() + a * angle.sin()
                t.copy_(v.to(t.dtype))

    class ParallelBlock(Part):
        """h += mixer(norm(h)) + feed_forward(norm(h)): reads the layer spec's parts `norm`, `mixer`, `feed_forward`."""

        def __init__(self, layer_spec):
            self.kind = "toy_parallel"
            self.norm = build_part("norm", layer_spec.part("norm"))
            self.mixer = build_part("mixer", layer_spec.part("mixer"))
            self.feed_forward = build_part("feed_forward", layer_spec.part("feed_forward"))

        def sub_parts(self):
            return [self.norm, self.mixer, self.feed_forward]

        def cache_need(self):
            return self.mixer.cache_need()

        def forward(self, hidden, delta, ctx, site, writes_cache):
            x = self.norm.forward(hidden, delta)
            mixed = self.mixer.forward(x, ctx, site, writes_cache)
            return (mixed.float() + self.feed_forward.forward(x, ctx).float()).to(mixed.dtype)

    register_part("feed_forward", "toy_routed_experts", RoutedExperts)
    register_part("position", "toy_two_axis_rotary", TwoAxisRotary)
    register_part("block", "toy_parallel", ParallelBlock)

    @dataclass(frozen=True)
    class ToyRoutedConfig(ModelConfig):
        vocab_size: int
        width: int
        inner: int
        experts: int
        eps: float
        theta: float
        n_layers: int
        architecture = "ToyRoutedForCausalLM"

        @classmethod
        def from_dict(cls, data):
            return cls(*(data[k] for k in ("vocab_size", "width", "inner", "experts", "eps", "theta", "n_layers")))

        def to_dict(self):
            return dict(architectures=[self.architecture], vocab_size=self.vocab_size, width=self.width, inner=self.inner,
                        experts=self.experts, eps=self.eps, theta=self.theta, n_layers=self.n_layers)

        def model_spec(self):
            def norm(name):
                return PartSpec("rms_norm", {"width": self.width, "eps": self.eps}, {"weight": name})
            layers = []
            for i in range(self.n_layers):
                p = f"l{i}."
                mixer = PartSpec("gqa_attention",
                                 {"hidden_size": self.width, "num_heads": HEADS, "num_kv_heads": KV_HEADS, "head_dim": HEAD_DIM,
                                  "qkv_bias": False, "window": 0,
                                  "position": PartSpec("toy_two_axis_rotary", {"theta": self.theta})},
                                 {"q_weight": p + "q", "k_weight": p + "k", "v_weight": p + "v", "o_weight": p + "o"})
                routed = PartSpec("toy_routed_experts",
                                  {"width": self.width, "inner": self.inner, "experts": self.experts, "top_k": 2},
                                  {"router": p + "router", "in": p + "e{}.in", "out": p + "e{}.out"})
                dense = PartSpec("swiglu", {"hidden_size": self.width, "intermediate_size": 2 * self.width},
                                 {"gate_weight": p + "g", "up_weight": p + "u", "down_weight": p + "d"})
                if i % 2 == 0:   # a parallel-residual layer with the routed feed-forward
                    layers.append(LayerSpec("toy_parallel", {"norm": norm(p + "n"), "mixer": mixer, "feed_forward": routed}))
                else:            # the stock arrangement with a dense feed-forward
                    layers.append(LayerSpec("pre_norm", {"mixer_norm": norm(p + "n1"), "mixer": mixer,
                                                        "feed_forward_norm": norm(p + "n2"), "feed_forward": dense}))
            return ModelSpec(self.architecture, self.vocab_size, self.width, 1024,
                             PartSpec("token_embedding", {"vocab_size": self.vocab_size, "width": self.width}, {"weight": "emb"}),
                             tuple(layers), tuple(ScheduleEntry(i) for i in range(self.n_layers)), norm("final"),
                             PartSpec("linear_head", {"vocab_size": self.vocab_size, "width": self.width, "tied": False},
                                      {"weight": "head"}))

    try:
        register_architecture("ToyRoutedForCausalLM", ToyRoutedConfig)
    except ValueError:
        pass
    return ToyRoutedConfig


def plain_two_axis(t, axes, theta):
    """t [heads, n, D] float64, axes [n, 2]."""
    half, quarter = t.shape[-1] // 2, t.shape[-1] // 4
    freq = 1.0 / (theta ** (torch.arange(quarter, dtype=torch.float32) / quarter)).double()
    out = t.clone()
    for axis in range(2):
        angle = axes[:, axis].double()[None, :, None] * freq
        a, b = t[..., axis * half:axis * half + quarter], t[..., axis * half + quarter:(axis + 1) * half]
        out[..., axis * half:axis * half + quarter] = a * angle.cos() - b * angle.sin()
        out[..., axis * half + quarter:(axis + 1) * half] = b * angle.cos() + a * angle.sin()
    return out


def plain_toy(cfg, w, tokens, axes, dtype):
    """Logits [n, vocab] in float64 from `dtype`-rounded weights, and the smallest gap between the second and the third
    router logit of any token (how far the choice of experts is from a tie)."""
    w = {k: (v if k.endswith("router") else v.to(dtype)).double() for k, v in w.items()}
    n = len(tokens)
    h = w["emb"][torch.tensor(tokens)]
    closest = float("inf")

    def attend(x, p):
        q = plain_two_axis((x @ w[p + "q"].T).view(n, HEADS, HEAD_DIM).transpose(0, 1), axes, cfg.theta)
        k = plain_two_axis((x @ w[p + "k"].T).view(n, KV_HEADS, HEAD_DIM).transpose(0, 1), axes, cfg.theta)
        v = (x @ w[p + "v"].T).view(n, KV_HEADS, HEAD_DIM).transpose(0, 1)
        return plain.attention(q, k, v).transpose(0, 1).reshape(n, HEADS * HEAD_DIM) @ w[p + "o"].T

    for i in range(cfg.n_layers):
        p = f"l{i}."
        if i % 2 == 0:
            x = plain.rms_norm(h, w[p + "n"], cfg.eps)
            ranked = torch.sort(x @ w[p + "router"].T, dim=-1, descending=True).values
            closest = min(closest, float((ranked[:, 1] - ranked[:, 2]).min()))
            top, chosen = torch.topk(x @ w[p + "router"].T, 2, dim=-1)
            gates = torch.softmax(top, dim=-1)
            routed = torch.zeros_like(h)
            for t in range(n):
                for slot in range(2):
                    e = int(chosen[t, slot])
                    inner = w[p + f"e{e}.in"] @ x[t]
                    routed[t] += gates[t, slot] * (w[p + f"e{e}.out"] @ (inner * torch.sigmoid(inner)))
            h = h + attend(x, p) + routed
        else:
            h = h + attend(plain.rms_norm(h, w[p + "n1"], cfg.eps), p)
            x = plain.rms_norm(h, w[p + "n2"], cfg.eps)
            g, u = x @ w[p + "g"].T, x @ w[p + "u"].T
            h = h + (g * torch.sigmoid(g) * u) @ w[p + "d"].T
    return plain.rms_norm(h, w["final"], cfg.eps) @ w["head"].T, closest


@pytest.mark.parametrize("dtype", DTYPES)
def test_routed_feed_forward_two_axis_positions_and_a_parallel_block(dtype, tmp_path):
    from qwenforge_b200.engine import Model
    from qwenforge_b200.engine.graphs import GraphDecoder
    from qwenforge_b200.weights import SafetensorsFile, write_random_model
    ToyRoutedConfig = register_toys()
    cfg = ToyRoutedConfig(vocab_size=101, width=64, inner=24, experts=4, eps=1e-5, theta=100.0, n_layers=3)
    write_random_model(cfg, WEIGHT_SEED, tmp_path, torch.float32)
    with SafetensorsFile(tmp_path / "model.safetensors") as f:
        weights = {n: f.tensor(n) for n in f.names()}
    assert weights["l0.router"].dtype == torch.float32 and "l0.e3.out" in weights and "l1.g" in weights
    model = Model.from_dir(tmp_path, dtype, DEV)
    assert not GraphDecoder.supported(model)   # the toys plan on the host: such a model steps, it does not replay graphs
    cache = model.new_cache(512, 3)
    g = torch.Generator().manual_seed(3)
    seqs = [torch.randint(0, 101, (n,), generator=g).tolist() for n in (40, 7, 21)]
    axes = [torch.stack((torch.arange(len(s)) // 8, torch.arange(len(s)) % 8), dim=1).int() for s in seqs]   # rows of 8
    refs, gaps = zip(*(plain_toy(cfg, weights, s, a, dtype) for s, a in zip(seqs, axes)))
    # the seed is one under which no token's choice of experts is near a tie: which experts run is then not a matter of
    # rounding, and the comparison sees the arithmetic
    assert min(gaps) > 2e-3, f"a router decision is {min(gaps):.1e} from a tie: take another WEIGHT_SEED"
    bound = [(4e-5 if dtype == torch.float32 else 5e-2) * float(r.abs().max()) for r in refs]
    slots = [cache.open() for _ in seqs]
    logits = model.step(cache, list(zip(slots, seqs)), want=[list(range(len(s))) for s in seqs], extras={"axes": axes})
    o = 0
    for s, r, b in zip(seqs, refs, bound):
        assert max_err(logits[o:o + len(s)], r) <= b
        o += len(s)
    for slot in slots:
        cache.close(slot)
    # a prompt, then token by token, with each step's own side inputs
    slots = [cache.open() for _ in seqs]
    got = [[] for _ in seqs]
    out = model.step(cache, [(slot, s[:4]) for slot, s in zip(slots, seqs)], want=[list(range(4))] * 3,
                     extras={"axes": [a[:4] for a in axes]})
    for i in range(3):
        got[i].append(out[4 * i:4 * i + 4])
    for t in range(4, 40):
        live = [i for i, s in enumerate(seqs) if t < len(s)]
        out = model.step(cache, [(slots[i], [seqs[i][t]]) for i in live], extras={"axes": [axes[i][t:t + 1] for i in live]})
        for row, i in enumerate(live):
            got[i].append(out[row:row + 1])
    model.raise_on_kernel_error()
    for pieces, r, b in zip(got, refs, bound):
        assert max_err(torch.cat(pieces), r) <= b
    with pytest.raises(ValueError, match="one row per token"):
        model.step(cache, [(slots[0], [1, 2])], extras={"axes": [axes[0][:1]]})
