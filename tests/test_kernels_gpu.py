"""Each CUDA kernel alone against a plain float64 computation of the same
operation, at sizes other than the engine's tiny models."""

import math
import random

import pytest
import torch

from tests.plain import qwen3_plain as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def F():
    from llm_runtime_study_b200.ops import functional

    return functional


def tol(dtype):
    return dict(atol=2e-6, rtol=2e-6) if dtype == torch.float32 else dict(atol=1e-2, rtol=1e-2)


def dev(t, dtype=None):
    return t.to(device="cuda", dtype=dtype or t.dtype).contiguous()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden,vocab", [(70, 33), (4104, 5)])
def test_embedding(dtype, hidden, vocab):
    torch.manual_seed(0)
    table = torch.randn(vocab, hidden).to(dtype)
    ids = torch.randint(0, vocab, (13,), dtype=torch.int32)
    out = F().embedding(dev(ids), dev(table), 1.0)
    assert out.dtype == torch.float32
    torch.testing.assert_close(out.cpu(), table[ids.long()].float(), atol=0, rtol=0)
    out = F().embedding(dev(ids), dev(table), 12.0)
    torch.testing.assert_close(out.cpu(), table[ids.long()].float() * 12.0, atol=0, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [1, 100, 4102, 4104, 13000, 40000])
def test_add_rmsnorm(dtype, hidden):
    torch.manual_seed(1)
    n, eps = 7, 3e-5
    resid, delta = torch.randn(n, hidden) * 3, torch.randn(n, hidden)
    weight = 1 + 0.1 * torch.randn(hidden)
    r = dev(resid)
    out = F().add_rmsnorm(r, dev(delta), dev(weight), eps, dtype)
    total = (resid + delta)
    torch.testing.assert_close(r.cpu(), total, atol=0, rtol=0)          # residual updated in place
    want = plain.rms_norm(total.double(), weight.double(), eps)
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype))
    # without delta the residual is left alone; with rows it gathers
    r2 = dev(resid)
    out2 = F().add_rmsnorm(r2, None, dev(weight), eps, dtype)
    torch.testing.assert_close(r2.cpu(), resid, atol=0, rtol=0)
    torch.testing.assert_close(out2.cpu().double(), plain.rms_norm(resid.double(), weight.double(), eps), **tol(dtype))
    rows = torch.tensor([5, 0, 5], dtype=torch.int32)
    out3 = F().add_rmsnorm(r2, dev(delta), dev(weight), eps, dtype, rows=dev(rows))
    torch.testing.assert_close(r2.cpu(), resid, atol=0, rtol=0)
    torch.testing.assert_close(out3.cpu().double(), want[rows.long()], **tol(dtype))


def test_rmsnorm_eps_matters():
    x = torch.full((1, 64), 1e-3)
    w = torch.ones(64)
    a = F().add_rmsnorm(dev(x), None, dev(w), 1e-6, torch.float32).cpu()
    b = F().add_rmsnorm(dev(x), None, dev(w), 1e-5, torch.float32).cpu()
    torch.testing.assert_close(a.double(), plain.rms_norm(x.double(), w.double(), 1e-6), atol=1e-6, rtol=1e-6)
    assert float((a - b).abs().max()) > 1e-2


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [11, 272, 1000])
def test_silu_mul(dtype, inter):
    torch.manual_seed(2)
    gu = (torch.randn(5, 2 * inter) * 3).to(dtype)
    out = F().silu_mul(dev(gu))
    g, u = gu[:, :inter].double(), gu[:, inter:].double()
    torch.testing.assert_close(out.cpu().double(), g / (1 + torch.exp(-g)) * u, **tol(dtype))


@pytest.mark.parametrize("m,n,k", [(1, 101, 53), (37, 64, 16), (65, 130, 257), (3, 503, 96)])
def test_gemm_f32_is_exact_and_batch_invariant(m, n, k):
    torch.manual_seed(3)
    x, w, b = torch.randn(m, k), torch.randn(n, k), torch.randn(n)
    out = F().linear_f32(dev(x), dev(w), dev(b)).cpu()
    want = x.double() @ w.double().T + b.double()
    torch.testing.assert_close(out.double(), want, atol=1e-5 * math.sqrt(k), rtol=1e-6)
    # true 32-bit: the error is far below what a 10-bit mantissa (TF32) would leave
    assert float((out.double() - want).abs().max()) < 2e-6 * k
    alone = F().linear_f32(dev(x[m // 2 : m // 2 + 1]), dev(w), dev(b)).cpu()
    assert torch.equal(alone[0], out[m // 2])


def _scatter_to_pages(k, v, page_size, nkv, d, dtype, seed=0, extra_pages=3):
    """Put contiguous k, v [T, nkv, d] into shuffled pages; return pools + table row."""

    T = k.shape[0]
    pages = -(-T // page_size)
    g = torch.Generator().manual_seed(seed)
    ids = torch.randperm(pages + extra_pages, generator=g)[:pages]
    k_pool = torch.full((pages + extra_pages, nkv, page_size, d), 1e4, dtype=dtype)  # poison
    v_pool = torch.full_like(k_pool, -1e4)
    for t in range(T):
        k_pool[ids[t // page_size], :, t % page_size] = k[t].to(dtype)
        v_pool[ids[t // page_size], :, t % page_size] = v[t].to(dtype)
    return k_pool, v_pool, ids.to(torch.int32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page,rot", [(4, 2, 16, 4, 16), (6, 1, 32, 8, 32), (5, 5, 48, 16, 48), (8, 2, 128, 16, 64),
                                               (8, 2, 128, 16, 128), (5, 3, 64, 16, 64), (3, 1, 256, 32, 256), (32, 8, 128, 16, 128)])
def test_qk_norm_rope_write(dtype, nq, nkv, d, page, rot):
    torch.manual_seed(4)
    eps, theta = 1e-5, 1e6
    # two requests: a portion at positions 37..45 and a single token far out
    positions = torch.tensor(list(range(37, 46)) + [3001], dtype=torch.int32)
    entry = torch.tensor([0] * 9 + [1], dtype=torch.int32)
    n = positions.shape[0]
    qkv = torch.randn(n, (nq + 2 * nkv) * d).to(dtype)
    qw, kw = 1 + 0.1 * torch.randn(d), 1 + 0.1 * torch.randn(d)
    pages_per_req = -(-3002 // page)
    table = torch.stack([torch.randperm(2 * pages_per_req)[:pages_per_req],
                         torch.randperm(2 * pages_per_req)[:pages_per_req] + 2 * pages_per_req]).to(torch.int32)
    pool_shape = (4 * pages_per_req, nkv, page, d)
    k_pool, v_pool = torch.zeros(pool_shape, dtype=dtype), torch.zeros(pool_shape, dtype=dtype)
    inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
    kp, vp = dev(k_pool), dev(v_pool)
    q_out = F().qk_norm_rope_write(
        dev(qkv), num_q_heads=nq, num_kv_heads=nkv, head_dim=d, q_weight=dev(qw), k_weight=dev(kw), eps=eps,
        inv_freq=dev(inv_freq), rotary_dim=rot, positions=dev(positions), token_entry=dev(entry),
        block_table=dev(table), page_size=page, k_pool=kp, v_pool=vp)
    x = qkv.double()
    q = x[:, : nq * d].view(n, nq, d)
    k = x[:, nq * d : (nq + nkv) * d].view(n, nkv, d)
    v = x[:, (nq + nkv) * d :].view(n, nkv, d)
    q, k = plain.rms_norm(q, qw.double(), eps), plain.rms_norm(k, kw.double(), eps)
    cos, sin = plain.rotary_tables(positions, rot, theta, torch.float64)
    q = torch.cat((plain.rotate(q[..., :rot], cos, sin), q[..., rot:]), dim=-1)
    k = torch.cat((plain.rotate(k[..., :rot], cos, sin), k[..., rot:]), dim=-1)
    torch.testing.assert_close(q_out.cpu().double(), q, **tol(dtype))
    kp, vp = kp.cpu().double(), vp.cpu().double()
    written = torch.zeros(pool_shape[0], page, dtype=torch.bool)
    for i in range(n):
        pg, slot = int(table[entry[i], positions[i] // page]), int(positions[i]) % page
        torch.testing.assert_close(kp[pg, :, slot], k[i], **tol(dtype))
        torch.testing.assert_close(vp[pg, :, slot], v[i], atol=0, rtol=0)   # values are copied as they are
        written[pg, slot] = True
    assert float(kp.permute(0, 2, 1, 3)[~written].abs().max()) == 0.0        # nothing else was touched
    assert float(vp.permute(0, 2, 1, 3)[~written].abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d", [(8, 2, 128), (5, 3, 64), (6, 1, 32)])
def test_qk_norm_rope_write_many_tokens_same_bits_as_few(dtype, nq, nkv, d):
    """A long portion (one CTA per token) and the same tokens a few at a time (a token's heads spread
    over several CTAs) give the same bits, and both agree with the plain formulas."""

    torch.manual_seed(9)
    eps, theta, page, n = 1e-6, 1e4, 16, 300
    positions = torch.arange(n, dtype=torch.int32)
    entry = torch.zeros(n, dtype=torch.int32)
    qkv = torch.randn(n, (nq + 2 * nkv) * d).to(dtype)
    qw, kw = 1 + 0.1 * torch.randn(d), 1 + 0.1 * torch.randn(d)
    pages = -(-n // page)
    table = torch.randperm(pages).to(torch.int32).view(1, pages)
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))

    def run(lo, hi, kp, vp):
        return F().qk_norm_rope_write(
            dev(qkv[lo:hi]), num_q_heads=nq, num_kv_heads=nkv, head_dim=d, q_weight=dev(qw), k_weight=dev(kw), eps=eps,
            inv_freq=dev(inv_freq), rotary_dim=d, positions=dev(positions[lo:hi]), token_entry=dev(entry[lo:hi]),
            block_table=dev(table), page_size=page, k_pool=kp, v_pool=vp)

    kp1, vp1 = dev(torch.zeros(pages, nkv, page, d, dtype=dtype)), dev(torch.zeros(pages, nkv, page, d, dtype=dtype))
    kp2, vp2 = torch.zeros_like(kp1), torch.zeros_like(vp1)
    whole = run(0, n, kp1, vp1)
    pieces = torch.cat([run(lo, min(lo + 7, n), kp2, vp2) for lo in range(0, n, 7)])
    assert torch.equal(whole, pieces) and torch.equal(kp1, kp2) and torch.equal(vp1, vp2)
    x = qkv.double()
    q = plain.rms_norm(x[:, : nq * d].view(n, nq, d), qw.double(), eps)
    cos, sin = plain.rotary_tables(positions, d, theta, torch.float64)
    torch.testing.assert_close(whole.cpu().double(), plain.rotate(q, cos, sin), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_qk_write_without_norm_or_rotation(dtype):
    torch.manual_seed(5)
    nq, nkv, d, page = 2, 1, 16, 4
    qkv = torch.randn(3, (nq + 2 * nkv) * d).to(dtype)
    positions, entry = torch.tensor([0, 1, 2], dtype=torch.int32), torch.zeros(3, dtype=torch.int32)
    table = torch.tensor([[1, 0]], dtype=torch.int32)
    kp, vp = dev(torch.zeros(2, nkv, page, d, dtype=dtype)), dev(torch.zeros(2, nkv, page, d, dtype=dtype))
    q = F().qk_norm_rope_write(
        dev(qkv), num_q_heads=nq, num_kv_heads=nkv, head_dim=d, q_weight=None, k_weight=None, eps=1.0,
        inv_freq=None, rotary_dim=0, positions=dev(positions), token_entry=dev(entry), block_table=dev(table),
        page_size=page, k_pool=kp, v_pool=vp)
    assert torch.equal(q.cpu().view(3, -1), qkv[:, : nq * d])
    assert torch.equal(kp.cpu()[1, 0, :3].reshape(3, -1), qkv[:, nq * d : (nq + nkv) * d])


def _attention_case(dtype, nq, nkv, d, page, lens_and_chunks, window=0, seed=6, boost=None, boost_size=16.0):
    """Requests with cached length L and the last n tokens as queries."""

    torch.manual_seed(seed)
    qs, pos, ent, wants, tables, pools_k, pools_v = [], [], [], [], [], [], []
    base = 0
    for e, (L, n) in enumerate(lens_and_chunks):
        q, k, v = torch.randn(L, nq, d), torch.randn(L, nkv, d), torch.randn(L, nkv, d)
        if boost is not None:   # one far key dominates the last query's scores
            t = boost if boost >= 0 else L + boost
            k[t] = 0
            k[t, :, 0] = boost_size
            q[L - 1] = 0
            q[L - 1, :, 0] = boost_size
            v[t] = 5.0
        q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
        out = plain.causal_attention(q.double(), k.double(), v.double(), 1 / math.sqrt(d), window=window or None)
        kp, vp, ids = _scatter_to_pages(k, v, page, nkv, d, dtype, seed=seed + e)
        pools_k.append(kp)
        pools_v.append(vp)
        tables.append(ids + base)
        base += kp.shape[0]
        qs.append(q[L - n :])
        wants.append(out[L - n :])
        pos += list(range(L - n, L))
        ent += [e] * n
    width = max(t.shape[0] for t in tables)
    table = torch.full((len(tables), width), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        table[i, : t.shape[0]] = t
    return (torch.cat(qs), torch.cat(pools_k), torch.cat(pools_v), torch.tensor(pos, dtype=torch.int32),
            torch.tensor(ent, dtype=torch.int32), table, torch.cat(wants))


ATTENTION_SHAPES = [(4, 2, 16, 4), (6, 1, 32, 8), (5, 5, 48, 16), (8, 2, 128, 16), (2, 2, 256, 32)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nq,nkv,d,page", ATTENTION_SHAPES)
def test_paged_attention_simt(dtype, nq, nkv, d, page):
    q, kp, vp, pos, ent, table, want = _attention_case(
        dtype, nq, nkv, d, page, [(1, 1), (33, 33), (70, 5), (131, 1), (64, 2)])
    out = F().paged_attention_simt(dev(q), dev(kp), dev(vp), positions=dev(pos), token_entry=dev(ent),
                                   block_table=dev(table), scale=1 / math.sqrt(d))
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 7, 32, 33])
def test_paged_attention_simt_window(dtype, window):
    nq, nkv, d, page = 4, 2, 32, 8
    q, kp, vp, pos, ent, table, want = _attention_case(dtype, nq, nkv, d, page, [(100, 40), (9, 9)], window=window)
    out = F().paged_attention_simt(dev(q), dev(kp), dev(vp), positions=dev(pos), token_entry=dev(ent),
                                   block_table=dev(table), scale=1 / math.sqrt(d), window=window)
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("boost", [0, 15, 16, -2, 300])
def test_attention_finds_a_far_key(dtype, boost):
    """One key among hundreds carries nearly all the weight: a kernel that drops
    or misplaces it (a page's edge, the first key, the last but one) shows."""

    nq, nkv, d, page = 4, 1, 64, 16
    q, kp, vp, pos, ent, table, want = _attention_case(dtype, nq, nkv, d, page, [(700, 3)], boost=boost)
    out = F().paged_attention_simt(dev(q), dev(kp), dev(vp), positions=dev(pos), token_entry=dev(ent),
                                   block_table=dev(table), scale=1 / math.sqrt(d))
    assert float(want[-1].abs().mean()) > 3.0      # the boosted value dominates
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2))


def test_kernels_refuse_what_they_cannot_take():
    from llm_runtime_study_b200.errors import KernelError

    with pytest.raises(KernelError, match="CUDA tensor"):
        F().silu_mul(torch.zeros(2, 4))
    with pytest.raises(KernelError, match="multiple of 16"):
        q = torch.zeros(1, 1, 24, device="cuda")
        pool = torch.zeros(1, 1, 4, 24, device="cuda")
        z = torch.zeros(1, dtype=torch.int32, device="cuda")
        F().paged_attention_simt(q, pool, pool, positions=z, token_entry=z, block_table=z.view(1, 1), scale=1.0)
    with pytest.raises(KernelError, match="storage type"):
        F().silu_mul(torch.zeros(2, 4, device="cuda", dtype=torch.float16))


# ------------------------------------------------------ bfloat16 tensor-core attention
def _mma():
    from llm_runtime_study_b200.ops import attention_bf16

    return attention_bf16


BF16_TOL = dict(atol=2e-2, rtol=2e-2)


def _q_lens(ent):
    return torch.bincount(ent.long()).tolist()


@pytest.mark.parametrize("nq,nkv,d,page", ATTENTION_SHAPES + [(32, 1, 64, 16), (6, 6, 80, 4), (12, 2, 128, 8)])
def test_prefill_attention_mma(nq, nkv, d, page):
    q, kp, vp, pos, ent, table, want = _attention_case(
        torch.bfloat16, nq, nkv, d, page, [(1, 1), (33, 33), (70, 5), (131, 1), (64, 2), (200, 200), (129, 65)])
    out = _mma().prefill_attention(dev(q), dev(kp), dev(vp), positions=dev(pos), block_table=dev(table),
                                   q_lens=_q_lens(ent), scale=1 / math.sqrt(d))
    torch.testing.assert_close(out.cpu().double(), want, **BF16_TOL)


@pytest.mark.parametrize("window", [1, 7, 64, 65, 100])
def test_prefill_attention_mma_window(window):
    nq, nkv, d, page = 4, 2, 32, 8
    q, kp, vp, pos, ent, table, want = _attention_case(torch.bfloat16, nq, nkv, d, page, [(300, 140), (9, 9), (70, 1)], window=window)
    out = _mma().prefill_attention(dev(q), dev(kp), dev(vp), positions=dev(pos), block_table=dev(table),
                                   q_lens=_q_lens(ent), scale=1 / math.sqrt(d), window=window)
    torch.testing.assert_close(out.cpu().double(), want, **BF16_TOL)


@pytest.mark.parametrize("nq,nkv,d,page", ATTENTION_SHAPES + [(32, 1, 64, 16), (6, 6, 80, 4), (32, 8, 128, 16)])
@pytest.mark.parametrize("splits", [1, 2, 5, 16])
def test_decode_attention_mma(nq, nkv, d, page, splits):
    lens = [1, 33, 70, 131, 64, 700, 65]
    q, kp, vp, pos, ent, table, want = _attention_case(torch.bfloat16, nq, nkv, d, page, [(L, 1) for L in lens])
    out = _mma().decode_attention(dev(q), dev(kp), dev(vp), kv_len=dev(torch.tensor(lens, dtype=torch.int32)),
                                  block_table=dev(table), scale=1 / math.sqrt(d), splits=splits, backend="mma")
    torch.testing.assert_close(out.cpu().double(), want, **BF16_TOL)


@pytest.mark.parametrize("window", [1, 7, 64, 65, 500])
def test_decode_attention_mma_window(window):
    nq, nkv, d, page = 8, 2, 64, 16
    lens = [300, 9, 64, 65]
    q, kp, vp, pos, ent, table, want = _attention_case(torch.bfloat16, nq, nkv, d, page, [(L, 1) for L in lens], window=window)
    out = _mma().decode_attention(dev(q), dev(kp), dev(vp), kv_len=dev(torch.tensor(lens, dtype=torch.int32)),
                                  block_table=dev(table), scale=1 / math.sqrt(d), window=window, splits=3)
    torch.testing.assert_close(out.cpu().double(), want, **BF16_TOL)


@pytest.mark.parametrize("boost", [0, 15, 16, 63, 64, -2, 300, 511, 512])
def test_mma_attention_finds_a_far_key(boost):
    nq, nkv, d, page = 8, 2, 64, 16
    q, kp, vp, pos, ent, table, want = _attention_case(torch.bfloat16, nq, nkv, d, page, [(700, 3)], boost=boost)
    assert float(want[-1].abs().mean()) > 3.0
    out = _mma().prefill_attention(dev(q), dev(kp), dev(vp), positions=dev(pos), block_table=dev(table),
                                   q_lens=[3], scale=1 / math.sqrt(d))
    torch.testing.assert_close(out.cpu().double(), want, atol=3e-2, rtol=2e-2)
    last = _mma().decode_attention(dev(q[-1:]), dev(kp), dev(vp), kv_len=dev(torch.tensor([700], dtype=torch.int32)),
                                   block_table=dev(table), scale=1 / math.sqrt(d), splits=4, backend="mma")
    torch.testing.assert_close(last.cpu().double(), want[-1:], atol=3e-2, rtol=2e-2)


def test_masked_cache_rows_may_hold_anything():
    """Unused slots of a page hold poison (1e4 / -1e4 here, see _scatter_to_pages);
    NaN bit patterns beyond a request's length must not leak either."""

    nq, nkv, d, page = 4, 2, 32, 16
    q, kp, vp, pos, ent, table, want = _attention_case(torch.bfloat16, nq, nkv, d, page, [(37, 37)])
    kp[table[0, 2].long(), :, 37 - 32:] = float("nan")
    vp[table[0, 2].long(), :, 37 - 32:] = float("nan")
    out = _mma().prefill_attention(dev(q), dev(kp), dev(vp), positions=dev(pos), block_table=dev(table),
                                   q_lens=[37], scale=1 / math.sqrt(d))
    torch.testing.assert_close(out.cpu().double(), want, **BF16_TOL)
    last = _mma().decode_attention(dev(q[-1:]), dev(kp), dev(vp), kv_len=dev(torch.tensor([37], dtype=torch.int32)),
                                   block_table=dev(table), scale=1 / math.sqrt(d), splits=2)
    torch.testing.assert_close(last.cpu().double(), want[-1:], **BF16_TOL)


# ------------------------------------------- decode attention with pages streamed by TMA
@pytest.mark.parametrize("nq,nkv,d,page", [(8, 2, 128, 16), (32, 8, 128, 16), (5, 1, 64, 16), (24, 2, 64, 32), (3, 3, 192, 16),
                                           (2, 1, 256, 64), (7, 7, 128, 48)])
@pytest.mark.parametrize("splits", [1, 2, 5, 16, 64])
def test_decode_attention_tma(nq, nkv, d, page, splits):
    """Lengths around the edges of blocks, pages and parts; twice in a row, so that the tickets of
    the first launch must have come back to zero; and the same bits as the first time."""

    mma = _mma()
    assert mma.DECODE_BACKEND == "tma" and mma.tma_supported(d, page, 0)
    lens = [1, 15, 16, 17, 33, 64, 65, 131, 700, 1024]
    q, kp, vp, pos, ent, table, want = _attention_case(torch.bfloat16, nq, nkv, d, page, [(L, 1) for L in lens])
    args = (dev(q), dev(kp), dev(vp))
    kw = dict(kv_len=dev(torch.tensor(lens, dtype=torch.int32)), block_table=dev(table), scale=1 / math.sqrt(d), splits=splits)
    first = mma.decode_attention(*args, **kw)
    second = mma.decode_attention(*args, **kw)
    torch.testing.assert_close(first.cpu().double(), want, **BF16_TOL)
    assert torch.equal(first, second)
    mma.check_decode_tma_error(d)


def test_decode_attention_tma_ignores_stale_rows_and_padding():
    """Slots past a request's length hold NaN; a padded row has length 0 and no pages."""

    mma = _mma()
    nq, nkv, d, page = 8, 2, 128, 16
    lens = [37, 100]
    q, kp, vp, pos, ent, table, want = _attention_case(torch.bfloat16, nq, nkv, d, page, [(L, 1) for L in lens])
    kp[table[0, 2].long(), :, 37 - 32:] = float("nan")
    vp[table[0, 2].long(), :, 37 - 32:] = float("nan")
    q3 = torch.cat([q, torch.zeros(1, nq, d, dtype=q.dtype)])
    table3 = torch.cat([table, torch.full((1, table.shape[1]), -1, dtype=torch.int32)])
    out = mma.decode_attention(dev(q3), dev(kp), dev(vp), kv_len=dev(torch.tensor(lens + [0], dtype=torch.int32)),
                               block_table=dev(table3), scale=1 / math.sqrt(d), splits=3)
    torch.testing.assert_close(out[:2].cpu().double(), want, **BF16_TOL)
    assert float(out[2].abs().max()) == 0.0
    mma.check_decode_tma_error(d)


@pytest.mark.parametrize("boost", [0, 15, 16, 255, 256, -2, -1, 300])
def test_decode_attention_tma_finds_a_far_key(boost):
    mma = _mma()
    nq, nkv, d, page = 8, 2, 128, 16
    q, kp, vp, pos, ent, table, want = _attention_case(torch.bfloat16, nq, nkv, d, page, [(700, 1)], boost=boost)
    assert float(want[-1].abs().mean()) > 3.0
    out = mma.decode_attention(dev(q), dev(kp), dev(vp), kv_len=dev(torch.tensor([700], dtype=torch.int32)),
                               block_table=dev(table), scale=1 / math.sqrt(d), splits=3)
    torch.testing.assert_close(out.cpu().double(), want, atol=3e-2, rtol=2e-2)


def test_decode_attention_tma_uses_as_many_parts_as_the_batch_needs():
    """A launch whose grid is sized for long sequences (as under a CUDA graph) with the number of parts in use
    told by the host through a device int: whatever it says, the result is the plain one, the CTAs of unused
    parts leave the tickets alone, and a second launch finds them at zero."""

    mma = _mma()
    nq, nkv, d, page = 8, 2, 128, 16
    lens = [1, 17, 64, 131, 700, 1024]
    q, kp, vp, pos, ent, table, want = _attention_case(torch.bfloat16, nq, nkv, d, page, [(L, 1) for L in lens])
    args = (dev(q), dev(kp), dev(vp))
    values = torch.zeros(8, dtype=torch.int32, device="cuda")
    live = mma.LiveParts(values, 32768)
    kw = dict(kv_len=dev(torch.tensor(lens, dtype=torch.int32)), block_table=dev(table), scale=1 / math.sqrt(d), splits=16, live=live)
    out = mma.decode_attention(*args, **kw)                    # the first launch registers its geometry; told 0, it uses one part
    torch.testing.assert_close(out.cpu().double(), want, **BF16_TOL)
    assert live.fill(1) == [1] and live.fill(32768)[0] > 4      # short batches in one part, long ones in many
    for longest in (1024, 1, 200, 5000, 32768, 10**6):
        chosen = live.fill(longest)
        values[: len(chosen)] = torch.tensor(chosen, dtype=torch.int32)
        for _ in range(2):
            out = mma.decode_attention(*args, **kw)
            torch.testing.assert_close(out.cpu().double(), want, **BF16_TOL)
    values.fill_(99)                                            # more than the grid has: all of the grid's parts
    torch.testing.assert_close(mma.decode_attention(*args, **kw).cpu().double(), want, **BF16_TOL)
    mma.check_decode_tma_error(d)


@pytest.mark.parametrize("nq,nkv,d,page", [(8, 2, 128, 16), (32, 8, 128, 16), (5, 1, 64, 16), (24, 2, 64, 32), (3, 3, 192, 16),
                                           (2, 1, 256, 64)])
@pytest.mark.parametrize("splits,norm,rot", [(1, True, True), (4, True, True), (16, False, True), (3, True, False), (2, False, False)])
def test_decode_attention_tma_prepares_the_new_token_itself(nq, nkv, d, page, splits, norm, rot):
    """From the raw rows of the q/k/v projection: per-head RMS norm and rotation of q and of the new k, the new k
    and v stored at the new position, attention over everything.  The cache rows of the new position hold
    poison before the launch; afterwards they hold the plain model's new key and value."""

    mma = _mma()
    torch.manual_seed(9)
    eps, theta = 1e-5, 1e4
    lens = [1, 16, 17, 33, 64, 65, 200, 700]
    wq, wk = 1 + 0.1 * torch.randn(d), 1 + 0.1 * torch.randn(d)
    dims = torch.arange(0, d, 2, dtype=torch.float32)
    inv_freq = 1.0 / (theta ** (dims / d))
    rows, tables, pools_k, pools_v, wants, new_k, new_v, base = [], [], [], [], [], [], [], 0
    for e, L in enumerate(lens):
        k, v = torch.randn(L, nkv, d).bfloat16(), torch.randn(L, nkv, d).bfloat16()
        raw = torch.randn((nq + 2 * nkv) * d).bfloat16()
        q_raw, k_raw, v_raw = raw[: nq * d].view(1, nq, d).double(), raw[nq * d : (nq + nkv) * d].view(1, nkv, d).double(), raw[(nq + nkv) * d :].view(nkv, d)
        if norm:
            q_raw, k_raw = plain.rms_norm(q_raw, wq.double(), eps), plain.rms_norm(k_raw, wk.double(), eps)
        if rot:
            cos, sin = plain.rotary_tables(torch.tensor([L - 1]), d, theta, torch.float64)
            q_raw, k_raw = plain.rotate(q_raw, cos, sin), plain.rotate(k_raw, cos, sin)
        keys = torch.cat([k[: L - 1].double(), k_raw.bfloat16().double()])
        vals = torch.cat([v[: L - 1].double(), v_raw.double().view(1, nkv, d)])
        out = torch.empty(nq, d, dtype=torch.float64)
        for h in range(nq):
            kv = h // (nq // nkv)
            w = torch.softmax((keys[:, kv] @ q_raw[0, h]) / math.sqrt(d), dim=0)
            out[h] = w @ vals[:, kv]
        wants.append(out)
        new_k.append(k_raw[0])
        new_v.append(v_raw.double())
        k[L - 1], v[L - 1] = 3e4, -3e4                         # what the cache holds there before: poison
        kp, vp, ids = _scatter_to_pages(k, v, page, nkv, d, torch.bfloat16, seed=40 + e)
        pools_k.append(kp)
        pools_v.append(vp)
        tables.append(ids + base)
        base += kp.shape[0]
        rows.append(raw)
    table = torch.full((len(lens), max(t.shape[0] for t in tables)), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        table[i, : t.shape[0]] = t
    kp, vp = dev(torch.cat(pools_k)), dev(torch.cat(pools_v))
    kw = dict(num_q_heads=nq, q_weight=dev(wq) if norm else None, k_weight=dev(wk) if norm else None, eps=eps,
              inv_freq=dev(inv_freq) if rot else None, kv_len=dev(torch.tensor(lens, dtype=torch.int32)),
              block_table=dev(table), scale=1 / math.sqrt(d), splits=splits)
    first = mma.decode_attention_fused(dev(torch.stack(rows)), kp, vp, **kw)
    second = mma.decode_attention_fused(dev(torch.stack(rows)), kp, vp, **kw)      # the rows it stored are the rows it makes
    torch.testing.assert_close(first.cpu().double(), torch.stack(wants), **BF16_TOL)
    assert torch.equal(first, second)
    for e, L in enumerate(lens):
        page_id, slot = int(table[e, (L - 1) // page]), (L - 1) % page
        torch.testing.assert_close(kp[page_id, :, slot].cpu().double(), new_k[e], atol=2e-2, rtol=2e-2)
        assert torch.equal(vp[page_id, :, slot].cpu().double(), new_v[e])
    mma.check_decode_tma_error(d)


# ------------------------------------------------------------ bfloat16 projections
def _gemm():
    from llm_runtime_study_b200.ops import gemm_bf16

    return gemm_bf16


def _gemm_case(m, n, k, bias, seed=7):
    torch.manual_seed(seed)
    x = torch.randn(m, k).bfloat16()
    w = (torch.randn(n, k) * 0.05).bfloat16()
    b = torch.randn(n) if bias else None
    want = x.double() @ w.double().T + (b.double() if bias else 0)
    return x, w, b, want


@pytest.mark.parametrize("m,n,k,bias", [(1, 136, 4096, False), (8, 4096, 4096, True), (3, 1000, 520, True),
                                        (16, 272, 96, False), (9, 503, 12288, False), (5, 17, 8, True)])
@pytest.mark.parametrize("out", [torch.float32, torch.bfloat16])
def test_weight_streaming_projection(m, n, k, bias, out):
    x, w, b, want = _gemm_case(m, n, k, bias)
    got = _gemm().linear_skinny(dev(x), dev(w), dev(b) if bias else None, out)
    again = _gemm().linear_skinny(dev(x), dev(w), dev(b) if bias else None, out)
    assert torch.equal(got, again)                                   # fixed summation order
    scale = float(want.abs().max())
    torch.testing.assert_close(got.cpu().double(), want, atol=(1e-2 if out == torch.bfloat16 else 1e-5) * scale, rtol=0)
    alone = _gemm().linear_skinny(dev(x[:1]), dev(w), dev(b) if bias else None, out)
    assert torch.equal(alone[0], got[0])                             # a row does not depend on the batch


@pytest.mark.parametrize("m,n,k,bias", [
    (128, 256, 64, False), (130, 264, 72, True), (300, 1000, 520, True), (2048, 1024, 4096, False), (5000, 4096, 512, True),
    (129, 8, 8, True),
])
@pytest.mark.parametrize("out", [torch.float32, torch.bfloat16])
def test_tcgen05_projection(m, n, k, bias, out):
    """The one-CTA persistent kernel, and whatever the shape picks by itself."""

    x, w, b, want = _gemm_case(m, n, k, bias)
    scale = float(want.abs().max())
    for kernel, tile_n in (("persistent", 256), ("persistent", 128), (None, None)):
        got = _gemm().linear(dev(x), dev(w), dev(b) if bias else None, out, kernel=kernel, tile_n=tile_n)
        _gemm().check_error()
        torch.testing.assert_close(got.cpu().double(), want, atol=(1e-2 if out == torch.bfloat16 else 2e-5) * scale, rtol=0)


@pytest.mark.parametrize("m,n,k,bias", [
    (128, 256, 64, False), (130, 264, 72, True), (300, 1000, 520, True), (2048, 1024, 4096, False), (5000, 4096, 512, True),
    (17, 4096, 4096, False), (129, 24, 12288, True), (640, 520, 8, False), (1, 8, 8, True), (2048, 4096, 12288, False),
])
@pytest.mark.parametrize("out", [torch.float32, torch.bfloat16])
def test_tcgen05_stream_k_projection(m, n, k, bias, out):
    """Tile counts below, at and far above the number of SMs; K ranges cut inside tiles; three
    calls in a row, the last two with the flags the first one left."""

    x, w, b, want = _gemm_case(m, n, k, bias)
    args = (dev(x), dev(w), dev(b) if bias else None, out)
    got = _gemm().linear(*args, kernel="streamk")
    again = _gemm().linear(*args, kernel="streamk")
    third = _gemm().linear(*args, kernel="streamk")
    _gemm().check_error()
    scale = float(want.abs().max())
    torch.testing.assert_close(got.cpu().double(), want, atol=(1e-2 if out == torch.bfloat16 else 2e-5) * scale, rtol=0)
    assert torch.equal(got, again) and torch.equal(got, third)        # partial sums are added in a fixed order


@pytest.mark.parametrize("m,n,k,bias", [
    (17, 520, 328, True), (64, 4096, 4096, False), (100, 6144, 4096, True), (128, 4096, 12288, False), (24, 264, 72, True),
    (300, 1000, 4096, True), (1, 8, 8, True), (127, 24576, 512, False), (256, 4096, 4096, False), (40, 151936, 64, False),
])
@pytest.mark.parametrize("out", [torch.float32, torch.bfloat16])
def test_tcgen05_split_k_projection(m, n, k, bias, out):
    """Clusters of CTAs that share a tile's K range and add their parts through distributed shared
    memory: the shape the kernel chooses by itself, then every cluster size and several tile widths
    and ring depths, row counts below a full tile (short row boxes) and above one."""

    x, w, b, want = _gemm_case(m, n, k, bias)
    args = (dev(x), dev(w), dev(b) if bias else None, out)
    scale = float(want.abs().max())
    blocks = -(-k // 64)
    got = _gemm().linear(*args, kernel="splitk")
    again = _gemm().linear(*args, kernel="splitk")
    _gemm().check_error()
    torch.testing.assert_close(got.cpu().double(), want, atol=(1e-2 if out == torch.bfloat16 else 2e-5) * scale, rtol=0)
    assert torch.equal(got, again)                                     # parts are added in the order of the K ranges
    for tile_n, splits, stages in ((256, 1, 0), (128, 2, 3), (96, 3, 0), (32, 4, 0), (160, 4, 3), (64, 8, 0)):
        if splits > blocks or -(-m // 128) * -(-n // tile_n) * splits > 4096:
            continue
        other = _gemm().linear(*args, kernel="splitk", tile_n=tile_n, splits=splits, stages=stages)
        _gemm().check_error()
        torch.testing.assert_close(other.cpu().double(), want, atol=(1e-2 if out == torch.bfloat16 else 2e-5) * scale, rtol=0)


def test_tcgen05_split_k_rows_do_not_depend_on_their_company():
    """The tile shape is chosen from the widths only, so a row gives the same bits alone and among 127."""

    x, w, _, _ = _gemm_case(128, 1000, 4096, False)
    whole = _gemm().linear(dev(x), dev(w), None, torch.float32, kernel="splitk")
    for rows in (1, 17, 64, 100):
        part = _gemm().linear(dev(x[:rows].contiguous()), dev(w), None, torch.float32, kernel="splitk")
        assert torch.equal(part, whole[:rows])
    _gemm().check_error()


def test_tcgen05_split_k_refuses_what_it_cannot_take():
    from llm_runtime_study_b200.errors import KernelError

    x, w = torch.zeros(32, 128, device="cuda").bfloat16(), torch.zeros(64, 128, device="cuda").bfloat16()
    for kwargs in ({"tile_n": 48}, {"tile_n": 288}, {"splits": 9}, {"splits": 4}, {"tile_n": 256, "splits": 2, "stages": 1}):
        with pytest.raises(KernelError):                              # 48, 288: no such width; 9: no such cluster; 4: only two K blocks; one stage
            _gemm().linear(x, w, kernel="splitk", **kwargs)


@pytest.mark.parametrize("m,n,k,bias", [
    (256, 256, 64, False), (130, 264, 72, True), (300, 1000, 520, True), (2048, 1024, 4096, False), (5000, 4096, 512, True),
    (257, 24, 12288, True), (640, 520, 8, False), (1, 8, 8, True), (2048, 4096, 12288, False), (4096, 6144, 4096, False),
])
@pytest.mark.parametrize("out", [torch.float32, torch.bfloat16])
def test_tcgen05_pair_projection(m, n, k, bias, out):
    """The 2-CTA kernel: 256 x 256 tiles on pairs of SMs, ragged edges in every dimension."""

    x, w, b, want = _gemm_case(m, n, k, bias)
    args = (dev(x), dev(w), dev(b) if bias else None, out)
    got = _gemm().linear(*args, kernel="pair")
    again = _gemm().linear(*args, kernel="pair")
    _gemm().check_error()
    scale = float(want.abs().max())
    torch.testing.assert_close(got.cpu().double(), want, atol=(1e-2 if out == torch.bfloat16 else 2e-5) * scale, rtol=0)
    assert torch.equal(got, again)


@pytest.mark.parametrize("kernel", ["pair", "persistent"])
@pytest.mark.parametrize("m,n,k", [(256, 256, 64), (300, 1000, 520), (2048, 4096, 4096)])
def test_tcgen05_adds_to_the_residual(m, n, k, kernel):
    x, w, b, want = _gemm_case(m, n, k, True)
    torch.manual_seed(3)
    resid = torch.randn(m, n)
    target = dev(resid.clone())
    delta = _gemm().linear(dev(x), dev(w), dev(b), torch.float32, kernel=kernel)
    out = _gemm().linear(dev(x), dev(w), dev(b), add_to=target, kernel=kernel)
    _gemm().check_error()
    assert out.data_ptr() == target.data_ptr()
    assert torch.equal(out, dev(resid) + delta)


@pytest.mark.parametrize("kernel", ["streamk", "splitk"])
@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 1000, 520), (2048, 4096, 4096), (40, 520, 4096)])
def test_tcgen05_shared_tiles_add_to_the_residual(m, n, k, kernel):
    x, w, b, want = _gemm_case(m, n, k, True)
    torch.manual_seed(3)
    resid = torch.randn(m, n)
    target = dev(resid.clone())
    delta = _gemm().linear(dev(x), dev(w), dev(b), torch.float32, kernel=kernel)
    out = _gemm().linear(dev(x), dev(w), dev(b), add_to=target, kernel=kernel)
    _gemm().check_error()
    assert out.data_ptr() == target.data_ptr()
    assert torch.equal(out, dev(resid) + delta)                       # the same single float32 addition


def test_projections_refuse_unaligned_widths():
    from llm_runtime_study_b200.errors import KernelError

    x, w = torch.zeros(2, 12, device="cuda").bfloat16(), torch.zeros(4, 12, device="cuda").bfloat16()
    with pytest.raises(KernelError, match="multiple of 8"):
        _gemm().linear_skinny(x, w)
    with pytest.raises(KernelError, match="multiple of 8"):
        _gemm().linear(x, w)


# ------------------------------------------------------------- tcgen05 prefill attention
@pytest.mark.parametrize("nq,nkv,d,page", [(8, 2, 128, 16), (32, 8, 128, 16), (4, 4, 64, 8), (6, 1, 64, 32), (5, 1, 128, 64),
                                           (32, 1, 64, 16), (12, 2, 128, 8)])
@pytest.mark.parametrize("pair", [False, True])
def test_prefill_attention_tcgen05(nq, nkv, d, page, pair):
    """Both kernels (one and two row tiles per CTA): portions that fill no tile, one tile, one and a bit, many;
    with and without a cached prefix; a last key tile that only the second row tile sees (129 keys, 65 new)."""

    q, kp, vp, pos, ent, table, want = _attention_case(
        torch.bfloat16, nq, nkv, d, page, [(1, 1), (33, 33), (70, 5), (131, 1), (64, 2), (200, 200), (129, 65), (513, 300),
                                           (260, 9), (128, 128), (1000, 64)])
    out = _mma().prefill_attention_tcgen05(dev(q), dev(kp), dev(vp), positions=dev(pos), block_table=dev(table),
                                           q_lens=_q_lens(ent), scale=1 / math.sqrt(d), pair=pair)
    _mma().check_tcgen05_error(d)
    torch.testing.assert_close(out.cpu().double(), want, **BF16_TOL)


@pytest.mark.parametrize("boost", [0, 15, 16, 63, 64, -2, 300, 511, 512, 127, 128, 640, 200, 350])
@pytest.mark.parametrize("pair,new,size", [(False, 3, 16.0), (True, 3, 16.0), (True, 40, 16.0), (True, 40, 40.0), (False, 40, 40.0)])
def test_tcgen05_attention_finds_a_far_key(boost, pair, new, size):
    """One key outweighs all others for the last query, by 2^46 or (size 40) by 2^288, which float32 cannot hold:
    the kernels must move their reference maximum when they meet it, in whichever half of whichever tile it lies."""

    nq, nkv, d, page = 8, 2, 64, 16
    q, kp, vp, pos, ent, table, want = _attention_case(torch.bfloat16, nq, nkv, d, page, [(700, new)], boost=boost,
                                                       boost_size=size)
    out = _mma().prefill_attention_tcgen05(dev(q), dev(kp), dev(vp), positions=dev(pos), block_table=dev(table),
                                           q_lens=[new], scale=1 / math.sqrt(d), pair=pair)
    _mma().check_tcgen05_error(d)
    torch.testing.assert_close(out.cpu().double(), want, atol=3e-2, rtol=2e-2)


@pytest.mark.parametrize("pair", [False, True])
def test_tcgen05_attention_rescales_when_the_maximum_grows(pair):
    """Scores that keep growing along the sequence force the lazy rescaling of O in TMEM."""

    torch.manual_seed(11)
    nq, nkv, d, page, L = 4, 1, 64, 16, 400
    q, k, v = torch.randn(L, nq, d), torch.randn(L, nkv, d), torch.randn(L, nkv, d)
    k[:, :, 0] = torch.linspace(0, 40, L).view(L, 1)       # later keys score ever higher for positive q
    q[:, :, 0] = 4.0
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    want = plain.causal_attention(q.double(), k.double(), v.double(), 1 / math.sqrt(d))
    kp, vp, ids = _scatter_to_pages(k, v, page, nkv, d, torch.bfloat16, seed=3)
    out = _mma().prefill_attention_tcgen05(dev(q), dev(kp), dev(vp), positions=dev(torch.arange(L, dtype=torch.int32)),
                                           block_table=dev(ids.view(1, -1)), q_lens=[L], scale=1 / math.sqrt(d), pair=pair)
    _mma().check_tcgen05_error(d)
    torch.testing.assert_close(out.cpu().double(), want, **BF16_TOL)


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("nq,nkv,d,boost", [(272, 16, 64, 1.0), (32, 8, 128, 4.0), (8, 2, 64, 3.0), (56, 8, 128, 1.0), (40, 8, 128, 3.0)])
def test_tcgen05_attention_gives_the_same_bits_every_time(pair, nq, nkv, d, boost):
    """Many CTAs, started longest first as the engine starts them, with scores spread widely enough that rows
    move their reference maximum often: forty launches give the same bits, and they are the plain result.  (A
    softmax warp that ran a tile ahead of the others once let a product start on a half-written P; with groups of
    7 or 5 query heads the last rows of a tile belong to no token, and what lay in shared memory there once decided
    which way the rows beside them were computed.)"""

    mma = _mma()
    page, L = 16, 520 if nq > 64 else 1100
    scale = 1 / math.sqrt(d)
    q, k, v, kp, vp, ids = _long_sequence(L, nq, nkv, d, page, seed=77)
    q = (q.float() * boost).bfloat16()
    gs = min(nq // nkv, 16)
    tiles = mma.tile_map([L], (2 if pair else 1) * (128 // gs), torch.device("cuda"), [L])
    args = dict(positions=dev(torch.arange(L, dtype=torch.int32)), block_table=dev(ids.view(1, -1)), q_lens=[L], scale=scale,
                pair=pair, tiles=tiles)
    qd, kd, vd = dev(q), dev(kp), dev(vp)
    first = mma.prefill_attention_tcgen05(qd, kd, vd, **args)
    for _ in range(40):
        assert torch.equal(mma.prefill_attention_tcgen05(qd, kd, vd, **args), first)
    mma.check_tcgen05_error(d)
    rows = sorted(set(random.Random(d).sample(range(L), 24)) | {0, L - 1})
    torch.testing.assert_close(first.cpu().double()[rows], _plain_attention_rows(q, k, v, rows, scale), **BF16_TOL)


# ------------------------------------------------------------- long sequences
def _long_sequence(L, nq, nkv, d, page, seed, far=None):
    """One sequence of L tokens in shuffled pages (written without a loop over tokens); ``far``: a key that
    outweighs all others for the last query."""

    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(L, h, d, generator=g) for h in (nq, nkv, nkv))
    if far is not None:
        k[far] = 0
        k[far, :, 0] = 16.0
        q[L - 1] = 0
        q[L - 1, :, 0] = 16.0
        v[far] = 5.0
    q, k, v = q.bfloat16(), k.bfloat16(), v.bfloat16()
    pages = -(-L // page)
    ids = torch.randperm(pages + 3, generator=g)[:pages]
    pools = []
    for x, poison in ((k, 1e4), (v, -1e4)):
        padded = torch.full((pages * page, nkv, d), poison, dtype=torch.bfloat16)
        padded[:L] = x
        pool = torch.full((pages + 3, nkv, page, d), poison, dtype=torch.bfloat16)
        pool[ids] = padded.view(pages, page, nkv, d).permute(0, 2, 1, 3)
        pools.append(pool)
    return q, k, v, pools[0], pools[1], ids.to(torch.int32)


def _plain_attention_rows(q, k, v, rows, scale):
    """The plain formula (softmax of q.k^T * scale over keys 0..row, times v) in float64, for some query rows."""

    group = q.shape[1] // k.shape[1]
    out = torch.empty(len(rows), q.shape[1], q.shape[2], dtype=torch.float64)
    for i, r in enumerate(rows):
        for head in range(q.shape[1]):
            kv = head // group
            weights = torch.softmax((k[: r + 1, kv].double() @ q[r, head].double()) * scale, dim=0)
            out[i, head] = weights @ v[: r + 1, kv].double()
    return out


@pytest.mark.parametrize("lens", [(32768, 20000, 9001, 4097), (16385,)])
def test_decode_attention_over_long_sequences(lens):
    """Tens of thousands of keys per request, in as many parts as the engine would choose and in the most the
    kernel takes; one far key stands out in each sequence."""

    mma = _mma()
    nq, nkv, d, page = 8, 2, 128, 16
    qs, pools_k, pools_v, tables, wants, base = [], [], [], [], [], 0
    for i, L in enumerate(lens):
        q, k, v, kp, vp, ids = _long_sequence(L, nq, nkv, d, page, seed=40 + i, far=(L * (i + 1)) // 7)
        qs.append(q[L - 1 :])
        wants.append(_plain_attention_rows(q, k, v, [L - 1], 1 / math.sqrt(d)))
        pools_k.append(kp)
        pools_v.append(vp)
        tables.append(ids + base)
        base += kp.shape[0]
    table = torch.full((len(lens), max(t.numel() for t in tables)), -1, dtype=torch.int32)
    for i, t in enumerate(tables):
        table[i, : t.numel()] = t
    want = torch.cat(wants)
    chosen = mma.parts_for(len(lens), nq, nkv, d, page, 0, max(lens))
    assert chosen > 1
    for splits in (chosen, mma.TMA_MAX_SPLITS, 1):
        out = mma.decode_attention(dev(torch.cat(qs)), dev(torch.cat(pools_k)), dev(torch.cat(pools_v)),
                                   kv_len=dev(torch.tensor(lens, dtype=torch.int32)), block_table=dev(table),
                                   scale=1 / math.sqrt(d), splits=splits)
        torch.testing.assert_close(out.cpu().double(), want, **BF16_TOL)
    mma.check_decode_tma_error(d)


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("L,new", [(8192, 8192), (8192, 2048), (12000, 333)])
def test_prefill_attention_over_long_sequences(pair, L, new):
    """Thousands of new tokens behind thousands of cached ones; some rows of the result (the first and last of the
    portion, rows at the edges of key tiles, a handful in between) against the plain formula."""

    mma = _mma()
    nq, nkv, d, page = 8, 2, 128, 16
    q, k, v, kp, vp, ids = _long_sequence(L, nq, nkv, d, page, seed=50 + new % 7, far=L // 3)
    first = L - new
    rows = sorted({first, first + 1, L - 1, L - 2} | {r for r in (63, 64, 127, 128, 2047, 2048, 4095, 4096, 6143) if r >= first}
                  | set(random.Random(new).sample(range(first, L), 12)))
    want = _plain_attention_rows(q, k, v, rows, 1 / math.sqrt(d))
    out = mma.prefill_attention_tcgen05(dev(q[first:]), dev(kp), dev(vp), positions=dev(torch.arange(first, L, dtype=torch.int32)),
                                        block_table=dev(ids.view(1, -1)), q_lens=[new], scale=1 / math.sqrt(d), pair=pair)
    mma.check_tcgen05_error(d)
    got = out.cpu().double()[[r - first for r in rows]]
    torch.testing.assert_close(got, want, **BF16_TOL)


# ----------------------------------------------------------- fused SwiGLU epilogues
def _interleave(gate, up):
    blocks = gate.shape[0] // 8
    return torch.stack((gate.view(blocks, 8, -1), up.view(blocks, 8, -1)), dim=1).reshape(2 * gate.shape[0], -1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter", [8, 272, 1000])
def test_silu_mul_interleaved(dtype, inter):
    torch.manual_seed(12)
    g, u = (torch.randn(5, inter) * 3).to(dtype), (torch.randn(5, inter) * 3).to(dtype)
    packed = _interleave(g.T.contiguous(), u.T.contiguous()).T.contiguous()      # columns in blocks of eight
    out = F().silu_mul_interleaved(dev(packed))
    want = g.double() / (1 + torch.exp(-g.double())) * u.double()
    torch.testing.assert_close(out.cpu().double(), want, **tol(dtype))


@pytest.mark.parametrize("m,inter,k", [(1, 16, 64), (8, 272, 96), (16, 1000, 520), (130, 272, 96), (2048, 1536, 1024), (300, 8, 4096)])
def test_projection_with_swiglu_epilogue(m, inter, k):
    torch.manual_seed(13)
    x = torch.randn(m, k).bfloat16()
    gate, up = (torch.randn(inter, k) * 0.08).bfloat16(), (torch.randn(inter, k) * 0.08).bfloat16()
    g, u = x.double() @ gate.double().T, x.double() @ up.double().T
    want = g / (1 + torch.exp(-g)) * u
    w = dev(_interleave(gate, up))
    if m <= 16:
        got = _gemm().linear_skinny(dev(x), w, None, torch.bfloat16, swiglu=True)
    else:
        got = _gemm().linear(dev(x), w, None, torch.bfloat16, swiglu=True, kernel="persistent")
        _gemm().check_error()
        for kernel in ("streamk", "pair", "splitk"):
            other = _gemm().linear(dev(x), w, None, torch.bfloat16, swiglu=True, kernel=kernel)
            _gemm().check_error()
            torch.testing.assert_close(other.cpu().double(), want, atol=2e-2 * float(want.abs().max()), rtol=0)
    assert got.shape == (m, inter)
    torch.testing.assert_close(got.cpu().double(), want, atol=2e-2 * float(want.abs().max()), rtol=0)


# ------------------------------------------------ RMS norms carried by the weight-streaming projections
@pytest.mark.parametrize("m,n,k,bias", [(1, 4096, 4096, False), (8, 4096, 12288, False), (3, 1000, 520, True),
                                        (16, 264, 96, True), (9, 100, 72, False), (2, 12288, 64, False)])
def test_projection_adds_into_the_residual_and_prepares_the_next_norm(m, n, k, bias):
    """resid += x W^T (+ b); on the way out the rows times the next norm's weight in bfloat16, and every row's
    factor rsqrt(mean of squares + eps), added up over the kernel's CTAs in their order by a small kernel behind it."""

    x, w, b, product = _gemm_case(m, n, k, bias)
    torch.manual_seed(n)
    resid = torch.randn(m, n)
    next_weight = 1 + 0.05 * torch.randn(n)
    eps = 1e-5
    want = resid.double() + product
    resid_dev = dev(resid)
    args = (dev(x), dev(w), dev(b) if bias else None)
    weighted, scale = _gemm().linear_skinny_residual(*args, resid_dev, dev(next_weight), eps)
    size = float(want.abs().max())
    torch.testing.assert_close(resid_dev.cpu().double(), want, atol=1e-5 * size, rtol=0)
    torch.testing.assert_close(weighted.cpu().double(), want * next_weight.double(), atol=1e-2 * size, rtol=0)
    torch.testing.assert_close(scale[:m].cpu().double(), torch.rsqrt((want * want).mean(dim=1) + eps), rtol=1e-5, atol=0)
    # again on fresh rows: the sums are added in a fixed order
    resid_again = dev(resid)
    weighted_again, scale_again = _gemm().linear_skinny_residual(*args, resid_again, dev(next_weight), eps)
    assert torch.equal(resid_again, resid_dev) and torch.equal(weighted_again, weighted) and torch.equal(scale_again[:m], scale[:m])
    # and the same bits whatever the other rows are
    resid_one = dev(resid[:1])
    weighted_one, scale_one = _gemm().linear_skinny_residual(dev(x[:1]), dev(w), dev(b) if bias else None, resid_one, dev(next_weight), eps)
    assert torch.equal(resid_one[0], resid_dev[0]) and torch.equal(weighted_one[0], weighted[0]) and torch.equal(scale_one[0], scale[0])


@pytest.mark.parametrize("m,n,k,bias", [(1, 6144, 4096, False), (8, 136, 4096, True), (3, 1000, 520, True),
                                        (16, 272, 96, False), (12, 503, 72, False), (5, 17, 8, True)])
@pytest.mark.parametrize("out", [torch.float32, torch.bfloat16])
def test_projection_finishes_a_norm_that_was_left_half_done(m, n, k, bias, out):
    """Rows that lack a factor each: the kernel applies the factors to its results, before the bias."""

    x, w, b, product = _gemm_case(m, n, k, bias)
    torch.manual_seed(k)
    factor = torch.zeros(16)
    factor[:m] = 0.2 + torch.rand(m)
    want = (product - (b.double() if bias else 0)) * factor[:m, None].double() + (b.double() if bias else 0)
    got = _gemm().linear_skinny(dev(x), dev(w), dev(b) if bias else None, out, row_scale=dev(factor))
    size = float(want.abs().max())
    torch.testing.assert_close(got.cpu().double(), want, atol=(1e-2 if out == torch.bfloat16 else 2e-5) * size, rtol=0)


def test_swiglu_projection_finishes_a_norm():
    torch.manual_seed(21)
    m, inter, k = 7, 272, 96
    x = torch.randn(m, k).bfloat16()
    gate, up = (torch.randn(inter, k) * 0.08).bfloat16(), (torch.randn(inter, k) * 0.08).bfloat16()
    factor = torch.zeros(16)
    factor[:m] = 0.5 + torch.rand(m)
    g, u = (x.double() @ gate.double().T) * factor[:m, None].double(), (x.double() @ up.double().T) * factor[:m, None].double()
    want = g / (1 + torch.exp(-g)) * u
    got = _gemm().linear_skinny(dev(x), dev(_interleave(gate, up)), None, torch.bfloat16, swiglu=True, row_scale=dev(factor))
    torch.testing.assert_close(got.cpu().double(), want, atol=2e-2 * float(want.abs().max()), rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,hidden,vocab", [(1, 4096, 1000), (16, 104, 37), (5, 264, 503), (3, 8192, 50)])
def test_embedding_prepares_the_first_norm(dtype, n, hidden, vocab):
    torch.manual_seed(2)
    table = torch.randn(vocab, hidden).to(dtype)
    ids = torch.randint(0, vocab, (n,), dtype=torch.int32)
    norm_weight = 1 + 0.05 * torch.randn(hidden)
    rows, weighted, scale = F().embedding_weighted(dev(ids), dev(table), 1.5, dev(norm_weight), 1e-5)
    want = table[ids.long()].double() * 1.5
    torch.testing.assert_close(rows.cpu().double(), want, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(weighted.cpu().double(), want * norm_weight.double(), atol=1e-2 * float(want.abs().max()), rtol=1e-2)
    torch.testing.assert_close(scale[:n].cpu().double(), torch.rsqrt((want * want).mean(dim=1) + 1e-5), rtol=1e-5, atol=0)


def test_weighted_rows_through_projections_equal_the_norm_kernel():
    """The two halves together against the norm kernel followed by the plain product, on one layer's worth of
    shapes: rows prepared by a projection into the residual, finished by the projection after it."""

    from llm_runtime_study_b200.parts import Projection, Runtime
    from llm_runtime_study_b200.parts.norm import RMSNorm

    torch.manual_seed(5)
    runtime = Runtime(torch.device("cuda:0"), torch.bfloat16)
    hidden, inner, m = 264, 520, 6
    down = Projection([(torch.randn(hidden, inner) * 0.05).bfloat16()], None, runtime)
    up = Projection([(torch.randn(inner, hidden) * 0.05).bfloat16()], [torch.randn(inner)], runtime)
    norm = RMSNorm(hidden, 1e-5)
    norm.load({"weight": 1 + 0.05 * torch.randn(hidden)}, runtime)
    x = dev(torch.randn(m, inner).bfloat16())
    resid = dev(torch.randn(m, hidden))
    # the fused way
    resid_a = resid.clone()
    rows = down(x, torch.float32, add_to=resid_a, next_norm=norm)
    assert type(rows).__name__ == "WeightedRows"
    got = up(rows, torch.float32)
    # the plain way: product, add, norm kernel, product
    resid_b = resid.clone()
    delta = down(x, torch.float32)
    normed = norm.add_norm(resid_b, delta)
    want = up(normed, torch.float32)
    torch.testing.assert_close(resid_a, resid_b, atol=1e-5, rtol=1e-5)
    torch.testing.assert_close(got, want, atol=2e-2 * float(want.abs().max()), rtol=0)
    torch.testing.assert_close(rows.normalised().float(), normed.float(), atol=2e-2 * float(normed.float().abs().max()), rtol=0)
