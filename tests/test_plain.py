"""The plain implementation against the reference's own model (golden files made
by tests/golden/make_golden.py), and its parts against explicit formulas."""

import json
import math
from pathlib import Path

import pytest
import torch

from llm_runtime_study_b200.config import architecture_for
from llm_runtime_study_b200.models.description import tensor_schema
from llm_runtime_study_b200.weights import random_state
from tests.helpers import TINY
from tests.plain import qwen3_plain as plain

GOLDEN = Path(__file__).parent / "golden"


@pytest.mark.parametrize("name", sorted(TINY))
def test_plain_matches_reference_model(name):
    raw, seed, _ = TINY[name]
    golden = json.loads((GOLDEN / f"tiny_{name}.json").read_text())
    arch = architecture_for(raw)
    schema = tensor_schema(arch.describe(arch.config_from_dict(raw)))
    state = random_state(schema, seed, dtype=torch.float32, include_optional=False)
    want = torch.tensor(golden["logits"], dtype=torch.float64).view(golden["shape"])
    got32 = plain.forward(state, raw, golden["token_ids"], dtype=torch.float32)
    got64 = plain.forward(state, raw, golden["token_ids"], dtype=torch.float64)
    assert got32.shape == want.shape
    torch.testing.assert_close(got64, want, atol=3e-6, rtol=1e-5)   # reference ran in float32
    torch.testing.assert_close(got32.double(), want, atol=5e-6, rtol=1e-5)


def test_rms_norm_formula():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    w = torch.tensor([2.0, 0.5], dtype=torch.float64)
    r = 1.0 / math.sqrt((9 + 16) / 2 + 1e-6)
    torch.testing.assert_close(plain.rms_norm(x, w, 1e-6), torch.tensor([[6 * r, 2 * r]], dtype=torch.float64))


def test_rotation_pairs_and_norm():
    d, theta = 8, 100.0
    x = torch.randn(5, 3, d, dtype=torch.float64)
    cos, sin = plain.rotary_tables(torch.arange(5), d, theta, torch.float64)
    y = plain.rotate(x, cos, sin)
    torch.testing.assert_close(y[0], x[0])  # position 0: no rotation
    torch.testing.assert_close(y.norm(dim=-1), x.norm(dim=-1))
    p, i = 3, 1
    angle = float(torch.tensor(p, dtype=torch.float32) * (1.0 / (theta ** (torch.tensor(2.0 * i) / d))))
    a, b = x[p, 0, i], x[p, 0, i + d // 2]
    assert abs(float(y[p, 0, i]) - float(a * math.cos(angle) - b * math.sin(angle))) < 1e-9
    assert abs(float(y[p, 0, i + d // 2]) - float(b * math.cos(angle) + a * math.sin(angle))) < 1e-9


def test_attention_is_causal_and_groups_heads():
    torch.manual_seed(0)
    T, nq, nkv, d = 6, 4, 2, 8
    q, k, v = (torch.randn(T, n, d, dtype=torch.float64) for n in (nq, nkv, nkv))
    out = plain.causal_attention(q, k, v, 1 / math.sqrt(d))
    torch.testing.assert_close(out[0, 0], v[0, 0])          # first token sees itself only
    torch.testing.assert_close(out[0, 3], v[0, 1])          # heads 2, 3 read kv head 1
    k2, v2 = k.clone(), v.clone()
    k2[4:], v2[4:] = 0, 0                                   # the future does not matter
    torch.testing.assert_close(plain.causal_attention(q, k2, v2, 1 / math.sqrt(d))[:4], out[:4])
    win = plain.causal_attention(q, k, v, 1 / math.sqrt(d), window=1)
    torch.testing.assert_close(win[:, 0], v[:, 0])          # window 1: own value


def test_swiglu_formula():
    torch.manual_seed(1)
    x = torch.randn(3, 4, dtype=torch.float64)
    w = {"m.gate_proj.weight": torch.randn(6, 4, dtype=torch.float64),
         "m.up_proj.weight": torch.randn(6, 4, dtype=torch.float64),
         "m.down_proj.weight": torch.randn(4, 6, dtype=torch.float64)}
    g = x @ w["m.gate_proj.weight"].T
    want = (torch.nn.functional.silu(g) * (x @ w["m.up_proj.weight"].T)) @ w["m.down_proj.weight"].T
    torch.testing.assert_close(plain.swiglu(x, w, "m"), want)
