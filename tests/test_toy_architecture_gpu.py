"""A toy architecture defined here, in the test, and run by the unchanged
framework: a mixer with per-request state of fixed size, a layer that runs twice
(shared weights, two caches), and a layer that reads the keys and values another
run wrote.  It is registered, built from a description, given random weights from
its own schema, and stepped under different cuts of the batch."""

import math
import random

import pytest
import torch

from tests import helpers
from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

H, NQ, NKV, D, I, V, EPS, THETA = 48, 3, 1, 16, 80, 97, 1e-5, 1e4


def register_toy():
    from llm_runtime_study_b200.config import Architecture, register_architecture
    from llm_runtime_study_b200.models import LayerDescription, ModelDescription
    from llm_runtime_study_b200.parts import MIXERS, FixedState, Mixer, Projection
    from llm_runtime_study_b200.weights import TensorSpec

    class DecaySum(Mixer):
        """s_t = sigmoid(a) * s_{t-1} + x_t per channel, y_t = W s_t; the state s is
        kept per request in a slot of fixed size."""

        def __init__(self, *, hidden_size: int) -> None:
            self.hidden_size = hidden_size

        def tensor_specs(self):
            return {"a": TensorSpec((self.hidden_size,), init="normal", std=1.0),
                    "out.weight": TensorSpec((self.hidden_size, self.hidden_size))}

        def load(self, tensors, runtime):
            self.runtime = runtime
            self.decay = torch.sigmoid(tensors["a"].to(device=runtime.device, dtype=torch.float32))
            self.out = Projection([tensors["out.weight"]], None, runtime)

        def cache_requirement(self):
            return FixedState((self.hidden_size,), torch.float32)

        def forward(self, x, ctx, cache):
            sums = torch.empty(x.shape, dtype=torch.float32, device=x.device)
            at = 0
            for slot, n in zip(ctx.entry_slots, ctx.q_lens):
                s = cache.state[slot]
                for t in range(at, at + n):
                    s = self.decay * s + x[t].float()
                    sums[t] = s
                cache.state[slot] = s
                at += n
            return self.out(sums.to(x.dtype), torch.float32)

    class DecaySumOnDevice(DecaySum):
        """The same mixer, written so that a decode step may be replayed from a CUDA graph: for a
        batch of single tokens it finds its rows of the state through the device-side ``ctx.slots``
        (rows that pad the batch point at the padding slot's row) and never looks at the host lists."""

        graph_safe = True

        def forward(self, x, ctx, cache):
            if not ctx.all_decode:
                return super().forward(x, ctx, cache)
            slots = ctx.slots.long()
            s = self.decay * cache.state.index_select(0, slots) + x.float()
            cache.state.index_copy_(0, slots, s)
            return self.out(s.to(x.dtype), torch.float32)

    MIXERS.register("toy_decay_sum", DecaySum, replace=True)
    MIXERS.register("toy_decay_sum_on_device", DecaySumOnDevice, replace=True)

    def describe(cfg):
        norm = {"kind": "rms_norm", "dim": H, "eps": EPS}
        attention = {"kind": "gqa_attention", "hidden_size": H, "num_heads": NQ, "num_kv_heads": NKV, "head_dim": D,
                     "qk_norm": {"kind": "rms_norm", "dim": D, "eps": EPS},
                     "position": {"kind": "rope", "head_dim": D, "theta": THETA}}
        ffn = {"kind": "swiglu", "hidden_size": H, "intermediate_size": I}

        def block(mixer):
            return {"kind": "pre_norm", "mixer": mixer, "feed_forward": ffn, "mixer_norm": norm, "ffn_norm": norm,
                    "names": {"mixer": "mix"}}

        layers = (
            LayerDescription(block(attention), "toy.layers.0"),
            LayerDescription(block({"kind": cfg.state_mixer, "hidden_size": H}), "toy.layers.1"),
            LayerDescription(block({**attention, "shares_kv": True}), "toy.layers.2"),
        )
        return ModelDescription(
            architecture="ToyHybrid", vocab_size=V, hidden_size=H, max_positions=128, eos_token_ids=(0,),
            embedding={"prefix": "toy.embed", "vocab_size": V, "hidden_size": H}, layers=layers,
            order=(0, 1, 0, 2), cache_of=(None, None, None, 2),
            final_norm={"prefix": "toy.norm", **norm},
            head={"prefix": "toy.head", "vocab_size": V, "hidden_size": H, "tied": True},
        )

    class ToyConfig:
        def __init__(self, raw):
            self.state_mixer = raw.get("state_mixer", "toy_decay_sum")

        def validate_context_length(self, n):
            assert n <= 128

    register_architecture(Architecture("ToyHybrid", "toy_hybrid", ToyConfig, describe), replace=True)


def plain_toy(w, tokens):
    """The same model, whole sequence, float64, from the plain functions."""

    w = {n: t.double() for n, t in w.items()}
    ids = torch.tensor(tokens)
    T = len(tokens)
    h = w["toy.embed.weight"][ids]
    cos, sin = plain.rotary_tables(torch.arange(T), D, THETA, torch.float64)
    cfg = {"num_attention_heads": NQ, "num_key_value_heads": NKV, "head_dim": D, "rms_norm_eps": EPS}

    def ffn(h, p):
        x = plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], EPS)
        return h + plain.swiglu(x, w, f"{p}.mlp")

    def attention_layer(h, p, shared_kv=None):
        x = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], EPS)
        q = plain.rotate(plain.rms_norm((x @ w[f"{p}.mix.q_proj.weight"].T).view(T, NQ, D), w[f"{p}.mix.q_norm.weight"], EPS), cos, sin)
        if shared_kv is None:
            k = plain.rotate(plain.rms_norm((x @ w[f"{p}.mix.k_proj.weight"].T).view(T, NKV, D), w[f"{p}.mix.k_norm.weight"], EPS), cos, sin)
            v = (x @ w[f"{p}.mix.v_proj.weight"].T).view(T, NKV, D)
        else:
            k, v = shared_kv
        o = plain.causal_attention(q, k, v, 1 / math.sqrt(D)).reshape(T, NQ * D) @ w[f"{p}.mix.o_proj.weight"].T
        return ffn(h + o, p), (k, v)

    h, _ = attention_layer(h, "toy.layers.0")
    x = plain.rms_norm(h, w["toy.layers.1.input_layernorm.weight"], EPS)
    decay, s, sums = torch.sigmoid(w["toy.layers.1.mix.a"]), torch.zeros(H, dtype=torch.float64), []
    for t in range(T):
        s = decay * s + x[t]
        sums.append(s)
    h = ffn(h + torch.stack(sums) @ w["toy.layers.1.mix.out.weight"].T, "toy.layers.1")
    h, kv = attention_layer(h, "toy.layers.0")                # the same weights again, a cache of its own
    h, _ = attention_layer(h, "toy.layers.2", shared_kv=kv)   # reads what the run before wrote
    return plain.rms_norm(h, w["toy.norm.weight"], EPS) @ w["toy.embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_architecture_is_built_and_stepped(tmp_path, dtype):
    from llm_runtime_study_b200.engine.replay import TraceReplayer
    from llm_runtime_study_b200.engine.runtime import load
    from llm_runtime_study_b200.weights import Checkpoint, write_random_model

    register_toy()
    raw = {"model_type": "toy_hybrid", "architectures": ["ToyHybrid"], "torch_dtype": dtype}
    write_random_model(tmp_path / "toy", raw, seed=5)
    weights = Checkpoint.from_model_dir(tmp_path / "toy").get_tensors()
    assert "toy.layers.2.mix.k_proj.weight" not in weights and "toy.layers.1.mix.a" in weights
    loaded = load(tmp_path / "toy", device="cuda:0", dtype=dtype)
    layout = loaded.model.cache_layout()
    assert [g.layers for g in layout.groups] == [(0, 2)] and [s.layer for s in layout.states] == [1]

    rng = random.Random(8)
    requests = {f"t{i}": helpers.random_tokens(rng, V, n) for i, n in enumerate([5, 23, 64, 41, 17, 9])}
    want = {rid: plain_toy(weights, toks) for rid, toks in requests.items()}
    tol = dict(atol=3e-5, rtol=1e-4) if dtype == "float32" else dict(atol=4e-2, rtol=3e-2)
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


@pytest.mark.parametrize("state_mixer,captured", [("toy_decay_sum", False), ("toy_decay_sum_on_device", True)])
def test_toy_architecture_generates_through_the_engine(tmp_path, state_mixer, captured):
    """The same toy model through ``Engine.generate`` with CUDA graphs asked for.  A mixer from outside the
    package that reads the host-side lists of the batch is not replayed from a graph (it does not say it
    may be), one that says so and keeps to the device-side slots is; both give the plain model's tokens,
    with requests joining and leaving the batch so that slots change hands between replays."""

    from llm_runtime_study_b200.engine.engine import Engine
    from llm_runtime_study_b200.weights import Checkpoint, write_random_model

    register_toy()
    raw = {"model_type": "toy_hybrid", "architectures": ["ToyHybrid"], "torch_dtype": "float32", "state_mixer": state_mixer}
    write_random_model(tmp_path / "toy", raw, seed=5)
    weights = Checkpoint.from_model_dir(tmp_path / "toy").get_tensors()
    engine = Engine.from_model_dir(tmp_path / "toy", device="cuda:0", dtype="float32", max_seq_len=64, max_batch_size=3,
                                   page_size=8, max_tokens_per_step=16, use_cuda_graph=True)
    assert engine.model.graph_safe() is captured
    rng = random.Random(12)
    prompts = [helpers.random_tokens(rng, V - 1, n) for n in (4, 11, 7, 19, 2)]
    new_tokens = [9, 5, 12, 6, 10]
    scheduler = engine.create_scheduler()
    for prompt, n in zip(prompts, new_tokens):
        scheduler.add_request([t + 1 for t in prompt], max_new_tokens=n)       # token 0 is the EOS
    got = {i: [] for i in range(len(prompts))}
    while scheduler.has_unfinished:
        for index, event in scheduler.step():
            got[index].append(event.token_id)
    assert (engine.runner._graphs is not None and len(engine.runner._graphs._graphs) > 0) is captured
    for i, (prompt, n) in enumerate(zip(prompts, new_tokens)):
        tokens = [t + 1 for t in prompt]
        for k in range(n):
            logits = plain_toy(weights, tokens)[-1]
            top = torch.topk(logits, 2).values
            if got[i][k] != int(logits.argmax()):
                assert float(top[0] - top[1]) < 1e-5, (i, k)
                break
            tokens.append(got[i][k])
            if got[i][k] == 0:
                break
    engine.cache_manager.check()
    assert engine.cache_manager.active_sequences == 0


def register_memo_toy():
    """A second toy: a mixer that keeps one vector per token in pages of its own (its own tensor, its own page
    size) and answers each token with the mean of what it has kept up to there."""

    from llm_runtime_study_b200.config import Architecture, register_architecture
    from llm_runtime_study_b200.models import LayerDescription, ModelDescription
    from llm_runtime_study_b200.parts import MIXERS, Mixer, Projection
    from llm_runtime_study_b200.parts.base import PagedTensors
    from llm_runtime_study_b200.weights import TensorSpec

    class RunningMean(Mixer):
        def __init__(self, *, hidden_size: int, width: int, page_size: int) -> None:
            self.hidden_size, self.width, self.page = hidden_size, width, page_size

        def tensor_specs(self):
            return {"in.weight": TensorSpec((self.width, self.hidden_size)), "out.weight": TensorSpec((self.hidden_size, self.width))}

        def load(self, tensors, runtime):
            self.runtime = runtime
            self.inp = Projection([tensors["in.weight"]], None, runtime)
            self.out = Projection([tensors["out.weight"]], None, runtime)

        def cache_requirement(self):
            return PagedTensors(tensors=(("memo", (self.width,)),), page_size=self.page)

        def forward(self, x, ctx, cache):
            memo = cache.tensors["memo"]                       # [pages, page, width]
            assert cache.page_size == self.page and memo.shape[1:] == (self.page, self.width)
            kept = self.inp(x).float()
            table = ctx.block_table(cache.group).cpu()
            means = torch.empty_like(kept)
            at = 0
            for entry, (n, after) in enumerate(zip(ctx.q_lens, ctx.kv_lens)):
                for i in range(n):
                    pos = after - n + i
                    memo[table[entry, pos // self.page], pos % self.page] = kept[at + i].to(memo.dtype)
                pages = table[entry, : -(-after // self.page)].to(x.device).long()
                history = memo[pages].reshape(-1, self.width)[:after].float()
                sums = history.cumsum(dim=0)[after - n:]
                means[at : at + n] = sums / torch.arange(after - n + 1, after + 1, device=x.device)[:, None]
                at += n
            return self.out(means.to(x.dtype), torch.float32)

    MIXERS.register("toy_running_mean", RunningMean, replace=True)

    def describe(cfg):
        norm = {"kind": "rms_norm", "dim": H, "eps": EPS}
        attention = {"kind": "gqa_attention", "hidden_size": H, "num_heads": NQ, "num_kv_heads": NKV, "head_dim": D,
                     "position": {"kind": "rope", "head_dim": D, "theta": THETA}}
        ffn = {"kind": "swiglu", "hidden_size": H, "intermediate_size": I}
        block = lambda mixer: {"kind": "pre_norm", "mixer": mixer, "feed_forward": ffn, "mixer_norm": norm, "ffn_norm": norm,
                               "names": {"mixer": "mix"}}
        layers = (LayerDescription(block({"kind": "toy_running_mean", "hidden_size": H, "width": 24, "page_size": 4}), "toy.layers.0"),
                  LayerDescription(block(attention), "toy.layers.1"))
        return ModelDescription(
            architecture="ToyMemo", vocab_size=V, hidden_size=H, max_positions=128, eos_token_ids=(0,),
            embedding={"prefix": "toy.embed", "vocab_size": V, "hidden_size": H}, layers=layers, order=(0, 1),
            final_norm={"prefix": "toy.norm", **norm}, head={"prefix": "toy.head", "vocab_size": V, "hidden_size": H, "tied": True})

    class Config:
        def validate_context_length(self, n):
            assert n <= 128

    register_architecture(Architecture("ToyMemo", "toy_memo", lambda raw: Config(), describe), replace=True)


def plain_memo_toy(w, tokens):
    w = {n: t.double() for n, t in w.items()}
    T = len(tokens)
    h = w["toy.embed.weight"][torch.tensor(tokens)]
    cos, sin = plain.rotary_tables(torch.arange(T), D, THETA, torch.float64)

    def ffn(h, p):
        return h + plain.swiglu(plain.rms_norm(h, w[f"{p}.post_attention_layernorm.weight"], EPS), w, f"{p}.mlp")

    x = plain.rms_norm(h, w["toy.layers.0.input_layernorm.weight"], EPS)
    kept = x @ w["toy.layers.0.mix.in.weight"].T
    means = kept.cumsum(dim=0) / torch.arange(1, T + 1)[:, None]
    h = ffn(h + means @ w["toy.layers.0.mix.out.weight"].T, "toy.layers.0")
    p = "toy.layers.1"
    x = plain.rms_norm(h, w[f"{p}.input_layernorm.weight"], EPS)
    q = plain.rotate((x @ w[f"{p}.mix.q_proj.weight"].T).view(T, NQ, D), cos, sin)
    k = plain.rotate((x @ w[f"{p}.mix.k_proj.weight"].T).view(T, NKV, D), cos, sin)
    v = (x @ w[f"{p}.mix.v_proj.weight"].T).view(T, NKV, D)
    o = plain.causal_attention(q, k, v, 1 / math.sqrt(D)).reshape(T, NQ * D) @ w[f"{p}.mix.o_proj.weight"].T
    h = ffn(h + o, p)
    return plain.rms_norm(h, w["toy.norm.weight"], EPS) @ w["toy.embed.weight"].T


def test_a_mixer_with_pages_of_its_own_kind():
    """Two page groups in one model: the attention layer's keys and values in pages of 8, the toy mixer's one
    vector per token in pages of 4; replayed whole, in portions and mixed, with pages of both groups reused."""

    import tempfile

    from llm_runtime_study_b200.engine.replay import TraceReplayer
    from llm_runtime_study_b200.engine.runtime import load
    from llm_runtime_study_b200.weights import Checkpoint, write_random_model

    register_memo_toy()
    with tempfile.TemporaryDirectory() as tmp:
        write_random_model(f"{tmp}/toy", {"model_type": "toy_memo", "architectures": ["ToyMemo"], "torch_dtype": "float32"}, seed=9)
        weights = Checkpoint.from_model_dir(f"{tmp}/toy").get_tensors()
        loaded = load(f"{tmp}/toy", device="cuda:0", dtype="float32")
    layout = loaded.model.cache_layout()
    assert len(layout.groups) == 2 and [g.requirement.page_size for g in layout.groups] == [4, None]
    rng = random.Random(4)
    requests = {f"m{i}": helpers.random_tokens(rng, V, n) for i, n in enumerate([3, 21, 40, 9, 17])}
    want = {rid: plain_memo_toy(weights, toks) for rid, toks in requests.items()}
    for steps in (helpers.trace_whole(requests), helpers.trace_chunked(requests, random.Random(1)),
                  helpers.trace_mixed(requests, random.Random(2), live_max=3)):
        replayer = TraceReplayer(loaded, max_tokens=helpers.pool_tokens(steps), page_size=8)
        manager = replayer.runner.manager
        assert [pool.page_size for pool in manager.groups] == [4, 8]
        outputs = {}
        for record in steps:
            rows = replayer.run_step(record)
            if rows is not None:
                outputs[record["step"]] = torch.from_numpy(rows.copy())
            manager.check()
        got = helpers.collect_logits(steps, outputs)
        for rid, toks in requests.items():
            rows = torch.stack([got[rid][p] for p in range(len(toks))]).double()
            torch.testing.assert_close(rows, want[rid], atol=3e-5, rtol=1e-4)
        assert manager.all_free and manager.active_sequences == 0
