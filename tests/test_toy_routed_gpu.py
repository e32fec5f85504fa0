"""Two more toy parts, defined here and run by the unchanged framework: a feed-forward
that routes every token over several small experts (router scores in float32, the
experts' outputs mixed by their softmax weights), and a position encoding that is
not the model's own (neighbouring pairs rotated, applied through
``PositionEncoding.apply`` instead of the fused rotary kernel).  The layers differ:
layer 0 has the routed feed-forward and a sliding window, layer 1 a dense one."""

import math
import random

import pytest
import torch

from tests import helpers
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

H, NQ, NKV, D, I, E, V, EPS, THETA, WINDOW = 40, 4, 2, 32, 56, 3, 61, 3e-6, 500.0, 24


def register_routed():
    from llm_runtime_study_b200.config import Architecture, register_architecture
    from llm_runtime_study_b200.models import LayerDescription, ModelDescription
    from llm_runtime_study_b200.parts import FEED_FORWARDS, POSITION_ENCODINGS, FeedForward, PositionEncoding, Projection
    from llm_runtime_study_b200.weights import TensorSpec

    class MixtureOfSmallExperts(FeedForward):
        """y = sum_e softmax(x R^T)_e * W2_e gelu(W1_e x): every expert sees every token, the
        router decides the weights.  Router scores and their softmax are float32."""

        def __init__(self, *, hidden_size: int, expert_size: int, experts: int) -> None:
            self.hidden_size, self.expert_size, self.experts = hidden_size, expert_size, experts

        def tensor_specs(self):
            specs = {"router.weight": TensorSpec((self.experts, self.hidden_size), init="normal", std=0.5)}
            for e in range(self.experts):
                specs[f"experts.{e}.up.weight"] = TensorSpec((self.expert_size, self.hidden_size), init="normal", std=0.2)
                specs[f"experts.{e}.down.weight"] = TensorSpec((self.hidden_size, self.expert_size), init="normal", std=0.2)
            return specs

        def load(self, tensors, runtime):
            self.runtime = runtime
            self.router = tensors["router.weight"].to(device=runtime.device, dtype=torch.float32)
            self.up = [Projection([tensors[f"experts.{e}.up.weight"]], None, runtime) for e in range(self.experts)]
            self.down = [Projection([tensors[f"experts.{e}.down.weight"]], None, runtime) for e in range(self.experts)]

        def forward(self, x, ctx):
            weights = torch.softmax(x.float() @ self.router.T, dim=-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e in range(self.experts):
                hidden = torch.nn.functional.gelu(self.up[e](x).float()).to(x.dtype)
                out += weights[:, e : e + 1] * self.down[e](hidden, torch.float32)
            return out

    class PairRotary(PositionEncoding):
        """Rotates the pairs (2i, 2i+1) of every head by position * theta^(-2i/d): the layout of
        the original rotary paper, not the half-split one the model's own encoding uses."""

        def __init__(self, *, head_dim: int, theta: float) -> None:
            self.head_dim, self.theta = head_dim, theta

        def load(self, tensors, runtime):
            self.runtime = runtime
            self.inv_freq = 1.0 / (self.theta ** (torch.arange(0, self.head_dim, 2, dtype=torch.float32) / self.head_dim))
            self.inv_freq = self.inv_freq.to(runtime.device)

        def apply(self, q, k, ctx):
            angle = ctx.positions.float()[:, None] * self.inv_freq[None, :]
            cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
            for t in (q, k):
                if t is None:
                    continue
                even, odd = t[..., 0::2].float(), t[..., 1::2].float()
                new_even, new_odd = even * cos - odd * sin, odd * cos + even * sin     # both before either is stored
                t[..., 0::2] = new_even.to(t.dtype)
                t[..., 1::2] = new_odd.to(t.dtype)

    FEED_FORWARDS.register("toy_mixture", MixtureOfSmallExperts, replace=True)
    POSITION_ENCODINGS.register("toy_pair_rotary", PairRotary, replace=True)

    def describe(cfg):
        norm = {"kind": "rms_norm", "dim": H, "eps": EPS}

        def attention(window):
            return {"kind": "gqa_attention", "hidden_size": H, "num_heads": NQ, "num_kv_heads": NKV, "head_dim": D,
                    "bias": True, "window": window, "position": {"kind": "toy_pair_rotary", "head_dim": D, "theta": THETA}}

        def block(mixer, ffn):
            return {"kind": "pre_norm", "mixer": mixer, "feed_forward": ffn, "mixer_norm": norm, "ffn_norm": norm}

        layers = (
            LayerDescription(block(attention(WINDOW), {"kind": "toy_mixture", "hidden_size": H, "expert_size": I, "experts": E}),
                             "net.layers.0"),
            LayerDescription(block(attention(None), {"kind": "swiglu", "hidden_size": H, "intermediate_size": 2 * I}), "net.layers.1"),
        )
        return ModelDescription(
            architecture="ToyRouted", vocab_size=V, hidden_size=H, max_positions=160, eos_token_ids=(0,),
            embedding={"prefix": "net.embed", "vocab_size": V, "hidden_size": H}, layers=layers,
            order=(0, 1), cache_of=(None, None),
            final_norm={"prefix": "net.norm", **norm},
            head={"prefix": "net.head", "vocab_size": V, "hidden_size": H, "tied": False},
        )

    class ToyConfig:
        def validate_context_length(self, n):
            assert n <= 160

    register_architecture(Architecture("ToyRouted", "toy_routed", lambda raw: ToyConfig(), describe), replace=True)


def plain_routed(w, tokens):
    """The same model, whole sequence, float64."""

    w = {n: t.double() for n, t in w.items()}
    T = len(tokens)
    h = w["net.embed.weight"][torch.tensor(tokens)]
    inv_freq = 1.0 / (THETA ** (torch.arange(0, D, 2, dtype=torch.float64) / D))
    angle = torch.arange(T, dtype=torch.float64)[:, None] * inv_freq[None, :]
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]

    def pair_rotate(t):
        even, odd = t[..., 0::2], t[..., 1::2]
        out = torch.empty_like(t)
        out[..., 0::2] = even * cos - odd * sin
        out[..., 1::2] = odd * cos + even * sin
        return out

    def attention(h, p, window):
        x = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], EPS)
        q = pair_rotate((x @ w[f"{p}.self_attn.q_proj.weight"].T + w[f"{p}.self_attn.q_proj.bias"]).view(T, NQ, D))
        k = pair_rotate((x @ w[f"{p}.self_attn.k_proj.weight"].T + w[f"{p}.self_attn.k_proj.bias"]).view(T, NKV, D))
        v = (x @ w[f"{p}.self_attn.v_proj.weight"].T + w[f"{p}.self_attn.v_proj.bias"]).view(T, NKV, D)
        o = plain.causal_attention(q, k, v, 1 / math.sqrt(D), window=window)
        return h + o.reshape(T, NQ * D) @ w[f"{p}.self_attn.o_proj.weight"].T

    h = attention(h, "net.layers.0", WINDOW)
    x = plain.rms_norm(h, w["net.layers.0.post_attention_layernorm.weight"], EPS)
    weights = torch.softmax(x @ w["net.layers.0.mlp.router.weight"].T, dim=-1)
    mixed = torch.zeros_like(h)
    for e in range(E):
        hidden = torch.nn.functional.gelu(x @ w[f"net.layers.0.mlp.experts.{e}.up.weight"].T)
        mixed += weights[:, e : e + 1] * (hidden @ w[f"net.layers.0.mlp.experts.{e}.down.weight"].T)
    h = h + mixed
    h = attention(h, "net.layers.1", None)
    x = plain.rms_norm(h, w["net.layers.1.post_attention_layernorm.weight"], EPS)
    h = h + plain.swiglu(x, w, "net.layers.1.mlp")
    return plain.rms_norm(h, w["net.norm.weight"], EPS) @ w["net.head.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_routed_feed_forward_and_foreign_position_encoding(tmp_path, dtype):
    from llm_runtime_study_b200.engine.replay import TraceReplayer
    from llm_runtime_study_b200.engine.runtime import load
    from llm_runtime_study_b200.weights import Checkpoint, write_random_model

    register_routed()
    raw = {"model_type": "toy_routed", "architectures": ["ToyRouted"], "torch_dtype": dtype}
    write_random_model(tmp_path / "net", raw, seed=11)
    weights = Checkpoint.from_model_dir(tmp_path / "net").get_tensors()
    assert "net.layers.0.mlp.experts.2.down.weight" in weights and "net.layers.1.mlp.gate_proj.weight" in weights
    loaded = load(tmp_path / "net", device="cuda:0", dtype=dtype)
    layout = loaded.model.cache_layout()
    assert sorted(g.requirement.window or 0 for g in layout.groups) == [0, WINDOW]   # a full group and a windowed one

    rng = random.Random(9)
    requests = {f"t{i}": helpers.random_tokens(rng, V, n) for i, n in enumerate([3, 31, 70, 150, 25, 49])}
    want = {rid: plain_routed(weights, toks) for rid, toks in requests.items()}
    tol = dict(atol=3e-5, rtol=1e-4) if dtype == "float32" else dict(atol=5e-2, rtol=3e-2)
    for steps in (helpers.trace_whole(requests), helpers.trace_chunked(requests, random.Random(1)),
                  helpers.trace_mixed(requests, random.Random(2), live_max=3)):
        replayer = TraceReplayer(loaded, max_tokens=helpers.pool_tokens(steps), page_size=8)
        outputs = {}
        for record in steps:
            rows = replayer.run_step(record)
            if rows is not None:
                outputs[record["step"]] = torch.from_numpy(rows.copy())
        got = helpers.collect_logits(steps, outputs)
        for rid, toks in requests.items():
            rows = torch.stack([got[rid][p] for p in range(len(toks))]).double()
            torch.testing.assert_close(rows, want[rid], **tol)
        replayer.runner.manager.check()
