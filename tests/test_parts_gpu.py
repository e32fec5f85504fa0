"""Each part alone, built from its registry with sizes unlike the tiny models',
against the plain functions."""

import math

import pytest
import torch

from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu


def runtime(dtype):
    from llm_runtime_study_b200.parts import Runtime

    return Runtime(torch.device("cuda:0"), dtype)


TOL = {torch.float32: dict(atol=3e-5, rtol=1e-4), torch.bfloat16: dict(atol=3e-2, rtol=3e-2)}


class OnePart:
    """Stands where a model stands, so that the real step function builds the
    batch metadata for a part under test."""

    def __init__(self, fn):
        self.fn = fn

    def bind_cache(self, manager):
        self.cache = manager.layer_cache(0)

    def forward(self, ctx):
        return self.fn(ctx, self.cache)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rms_norm_part(dtype):
    from llm_runtime_study_b200.parts import NORMS

    norm = NORMS.build({"kind": "rms_norm", "dim": 40, "eps": 2e-5})
    assert norm.tensor_specs()["weight"].shape == (40,)
    w = 1 + 0.1 * torch.randn(40)
    norm.load({"weight": w}, runtime(dtype))
    resid, delta = torch.randn(6, 40).cuda(), torch.randn(6, 40).cuda()
    want = plain.rms_norm((resid + delta).double().cpu(), w.double(), 2e-5)
    out = norm.add_norm(resid, delta)
    assert out.dtype == dtype
    torch.testing.assert_close(out.double().cpu(), want, **TOL[dtype])


def test_rope_part_frequencies():
    from llm_runtime_study_b200.parts import POSITION_ENCODINGS

    rope = POSITION_ENCODINGS.build({"kind": "rope", "head_dim": 48, "theta": 5e4})
    rope.load({}, runtime(torch.float32))
    inv_freq, rot = rope.rotary_parameters()
    assert rot == 48 and inv_freq.shape == (24,)
    want = 1.0 / (5e4 ** (torch.arange(0, 48, 2, dtype=torch.float32) / 48))
    assert torch.equal(inv_freq.cpu(), want)
    with pytest.raises(ValueError):
        POSITION_ENCODINGS.build({"kind": "rope", "head_dim": 48, "theta": 1.0, "rotary_dim": 50})


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_part(dtype):
    from llm_runtime_study_b200.parts import FEED_FORWARDS

    ffn = FEED_FORWARDS.build({"kind": "swiglu", "hidden_size": 72, "intermediate_size": 200})
    specs = ffn.tensor_specs()
    assert specs["gate_proj.weight"].shape == (200, 72) and specs["down_proj.weight"].shape == (72, 200)
    w = {n: (torch.randn(s.shape) * 0.1).to(dtype) for n, s in specs.items()}
    ffn.load(w, runtime(dtype))
    x = torch.randn(9, 72).to(dtype)
    out = ffn.forward(x.cuda(), None)
    assert out.dtype == torch.float32
    want = plain.swiglu(x.double(), {f"m.{n}": t.double() for n, t in w.items()}, "m")
    torch.testing.assert_close(out.double().cpu(), want, **TOL[dtype])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("bias,qk_norm,heads", [(False, True, (8, 2, 32)), (True, False, (3, 3, 16)), (True, True, (4, 1, 64))])
def test_attention_part_whole_and_in_portions(dtype, bias, qk_norm, heads):
    from llm_runtime_study_b200.cache import CacheLayout, CacheManager
    from llm_runtime_study_b200.engine.step import StepEntry, StepRunner
    from llm_runtime_study_b200.parts import MIXERS

    nq, nkv, d = heads
    hidden, eps, theta, T = 56, 1e-5, 1e4, 45
    desc = {"kind": "gqa_attention", "hidden_size": hidden, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d,
            "bias": bias, "position": {"kind": "rope", "head_dim": d, "theta": theta}}
    if qk_norm:
        desc["qk_norm"] = {"kind": "rms_norm", "dim": d, "eps": eps}
    mixer = MIXERS.build(desc)
    torch.manual_seed(0)
    w = {n: ((1 + 0.1 * torch.randn(s.shape)) if "norm" in n else torch.randn(s.shape) * 0.15).to(dtype)
         for n, s in mixer.tensor_specs().items()}
    rt = runtime(dtype)
    mixer.load(w, rt)
    x = torch.randn(T, hidden).to(dtype)
    # plain: whole sequence
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d, "rms_norm_eps": eps, "attention_bias": bias}
    pw = {f"a.{n}": t.double() for n, t in w.items()}
    if not qk_norm:
        pw["a.q_norm.weight"] = pw["a.k_norm.weight"] = None
    cos, sin = plain.rotary_tables(torch.arange(T), d, theta, torch.float64)
    if qk_norm:
        want = plain.attention_block(x.double(), pw, "a", cfg, cos, sin)
    else:
        q = (x.double() @ pw["a.q_proj.weight"].T + pw["a.q_proj.bias"]).view(T, nq, d)
        k = (x.double() @ pw["a.k_proj.weight"].T + pw["a.k_proj.bias"]).view(T, nkv, d)
        v = (x.double() @ pw["a.v_proj.weight"].T + pw["a.v_proj.bias"]).view(T, nkv, d)
        o = plain.causal_attention(plain.rotate(q, cos, sin), plain.rotate(k, cos, sin), v, 1 / math.sqrt(d))
        want = o.reshape(T, nq * d) @ pw["a.o_proj.weight"].T
    manager = CacheManager(CacheLayout.from_requirements([mixer.cache_requirement()]), max_tokens=64, page_size=8,
                           max_requests=2, dtype=dtype, device="cuda:0")
    xd = x.cuda()
    offset = {"at": 0}

    def run(ctx, cache):
        n = ctx.num_tokens
        out = mixer.forward(xd[offset["at"] : offset["at"] + n], ctx, cache)
        offset["at"] += n
        return out

    runner = StepRunner(OnePart(run), manager, rt, vocab_size=10, max_positions=64)
    for cuts in ([T], [20, 1, 1, 2, 21]):
        request = manager.admit()
        offset["at"] = 0
        outs = [runner.step([StepEntry(request, [0] * n, [])]) for n in cuts]
        manager.release(request)
        torch.testing.assert_close(torch.cat(outs).double().cpu(), want, **TOL[dtype])


def test_unknown_kind_and_bad_sizes():
    from llm_runtime_study_b200.errors import RegistryError
    from llm_runtime_study_b200.parts import FEED_FORWARDS, MIXERS

    with pytest.raises(RegistryError, match="unknown mixer kind"):
        MIXERS.build({"kind": "nothing"})
    with pytest.raises(ValueError, match="multiple of 16"):
        MIXERS.build({"kind": "gqa_attention", "hidden_size": 8, "num_heads": 2, "num_kv_heads": 1, "head_dim": 24})
    with pytest.raises(ValueError, match="multiple of num_kv_heads"):
        MIXERS.build({"kind": "gqa_attention", "hidden_size": 8, "num_heads": 3, "num_kv_heads": 2, "head_dim": 16})
    with pytest.raises(ValueError):
        FEED_FORWARDS.build({"kind": "swiglu", "hidden_size": 0, "intermediate_size": 4})


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_and_head_parts(dtype):
    from llm_runtime_study_b200.parts import OutputHead, TokenEmbedding

    torch.manual_seed(3)
    rt = runtime(dtype)
    emb = TokenEmbedding(vocab_size=37, hidden_size=24, scale=2.0)
    table = torch.randn(37, 24).to(dtype)
    emb.load({"weight": table}, rt)
    ids = torch.tensor([5, 0, 36, 5], dtype=torch.int32)
    out = emb.forward(ids.cuda())
    assert out.dtype == torch.float32
    torch.testing.assert_close(out.cpu(), table[ids.long()].float() * 2.0, atol=0, rtol=0)

    x = torch.randn(4, 24).to(dtype)
    untied = OutputHead(vocab_size=37, hidden_size=24, tied=False)
    assert not untied.tensor_specs()["weight"].optional
    w = (torch.randn(37, 24) * 0.2).to(dtype)
    untied.load({"weight": w}, rt, embedding=emb)
    logits = untied.forward(x.cuda())
    assert logits.dtype == torch.float32
    torch.testing.assert_close(logits.cpu().double(), x.double() @ w.double().T, **TOL[dtype])
    tied = OutputHead(vocab_size=37, hidden_size=24, tied=True)
    assert tied.tensor_specs()["weight"].optional
    tied.load({}, rt, embedding=emb)
    torch.testing.assert_close(tied.forward(x.cuda()).cpu().double(), x.double() @ table.double().T, **TOL[dtype])
    tied.load({"weight": w}, rt, embedding=emb)          # a stored head wins over the tie
    torch.testing.assert_close(tied.forward(x.cuda()).cpu().double(), x.double() @ w.double().T, **TOL[dtype])
    with pytest.raises(KeyError):
        untied.load({}, rt, embedding=emb)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pre_norm_block_composition(dtype):
    """h = h + mixer(norm1(h)); h = h + ffn(norm2(h)), the additions carried in float32 by the next norm."""

    from llm_runtime_study_b200.cache import CacheLayout, CacheManager
    from llm_runtime_study_b200.engine.step import StepEntry, StepRunner
    from llm_runtime_study_b200.parts import BLOCKS, ResidualStream

    hidden, nq, nkv, d, inter, eps, theta, T = 40, 2, 1, 16, 56, 1e-5, 1e4, 9
    norm = {"kind": "rms_norm", "dim": hidden, "eps": eps}
    block = BLOCKS.build({
        "kind": "pre_norm", "mixer_norm": norm, "ffn_norm": norm,
        "mixer": {"kind": "gqa_attention", "hidden_size": hidden, "num_heads": nq, "num_kv_heads": nkv, "head_dim": d,
                  "qk_norm": {"kind": "rms_norm", "dim": d, "eps": eps}, "position": {"kind": "rope", "head_dim": d, "theta": theta}},
        "feed_forward": {"kind": "swiglu", "hidden_size": hidden, "intermediate_size": inter},
    })
    torch.manual_seed(4)
    w = {n: ((1 + 0.1 * torch.randn(s.shape)) if "norm" in n else torch.randn(s.shape) * 0.2).to(dtype)
         for n, s in block.tensor_specs().items()}
    assert "self_attn.q_proj.weight" in w and "post_attention_layernorm.weight" in w and "mlp.down_proj.weight" in w
    rt = runtime(dtype)
    block.load(w, rt)
    h0 = torch.randn(T, hidden)
    cfg = {"num_attention_heads": nq, "num_key_value_heads": nkv, "head_dim": d, "rms_norm_eps": eps,
           "num_hidden_layers": 1, "rope_theta": theta}
    pw = {f"model.layers.0.{n}": t.double() for n, t in w.items()}
    cos, sin = plain.rotary_tables(torch.arange(T), d, theta, torch.float64)
    want = plain.decoder_layer(h0.double(), pw, 0, cfg, cos, sin)
    manager = CacheManager(CacheLayout.from_requirements([block.mixer.cache_requirement()]), max_tokens=32, page_size=4,
                           max_requests=1, dtype=dtype, device="cuda:0")

    def run(ctx, cache):
        stream = ResidualStream(h0.cuda().clone())
        block.forward(stream, ctx, cache)
        return stream.resid + stream.delta

    runner = StepRunner(OnePart(run), manager, rt, vocab_size=10, max_positions=32)
    got = runner.step([StepEntry(manager.admit(), [0] * T, [])])
    torch.testing.assert_close(got.double().cpu(), want, **TOL[dtype])
