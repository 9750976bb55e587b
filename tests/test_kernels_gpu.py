"""Each kernel alone against a plain torch reference, at other sizes than the engine's."""

import math

import pytest
import torch

import plain_qwen2 as P
from kernel_refs import attention_reference, pack_queries, paged_layout

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-6, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embedding(dtype):
    from turboserve_b200.ops import kernels

    table = torch.randn(300, 72).to(dtype).to(DEV)
    ids = torch.tensor([0, 299, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.embedding(ids, table, out, status)
    assert torch.equal(out, table.float()[ids.long()]) and status.item() == 0
    bad = torch.tensor([3, 300, -1], dtype=torch.int32, device=DEV)
    kernels.embedding(bad, table, out, status)
    assert status.item() == 1 and torch.equal(out[1], torch.zeros(72, device=DEV)) and torch.equal(out[0], table[3].float())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [72, 1000, 5120])
def test_add_rmsnorm(dtype, hidden):
    from turboserve_b200.ops import kernels

    rows, eps = 7, 3e-5
    residual = torch.randn(rows, hidden, device=DEV) * 3
    delta = (torch.randn(rows, hidden, device=DEV)).to(dtype)
    gain = 1 + 0.1 * torch.randn(hidden, device=DEV)
    before = residual.clone()
    out = torch.empty(rows, hidden, dtype=dtype, device=DEV)
    kernels.add_rmsnorm(residual, delta, gain, eps, out)
    summed = before + delta.float()
    assert torch.equal(residual, summed)  # the residual sum is exact fp32
    ref = P.rms_norm(summed.double(), gain.double(), eps)
    assert torch.allclose(out.double(), ref, **tol(dtype))
    # without a delta the residual is left alone
    kernels.add_rmsnorm(residual, None, gain, eps, out)
    assert torch.equal(residual, summed) and torch.allclose(out.double(), ref, **tol(dtype))
    # selected rows: output row r comes from source row rows[r], nothing is written back
    pick = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out3 = torch.empty(3, hidden, dtype=dtype, device=DEV)
    kernels.add_rmsnorm(residual, delta, gain, eps, out3, pick)
    ref3 = P.rms_norm((summed + delta.float())[pick.long()].double(), gain.double(), eps)
    assert torch.equal(residual, summed) and torch.allclose(out3.double(), ref3, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("act", ["silu", "gelu", "gelu_pytorch_tanh"])
def test_act_mul(dtype, act):
    from turboserve_b200.ops import kernels

    gate_up = (torch.randn(5, 2 * 136, device=DEV) * 2).to(dtype)
    out = torch.empty(5, 136, dtype=dtype, device=DEV)
    kernels.act_mul(gate_up, out, act)
    x = gate_up.double().cpu()
    ref = P.activation(x[:, :136], act) * x[:, 136:]
    assert torch.allclose(out.double().cpu(), ref, **tol(dtype))
    # many rows (bfloat16: the kernel with 16-byte accesses), plain and in runs of 64: the same bits as row by row
    for block in (0, 64):
        many = (torch.randn(70, 2 * 192, device=DEV) * 2).to(dtype)
        whole = torch.empty(70, 192, dtype=dtype, device=DEV)
        kernels.act_mul(many, whole, act, block=block)
        rows = torch.empty_like(whole)
        for lo in range(0, 70, 7):
            kernels.act_mul(many[lo:lo + 7], rows[lo:lo + 7], act, block=block)
        assert torch.equal(whole, rows)
        x = many.double().cpu()
        gate, up = (x[:, :192], x[:, 192:]) if block == 0 else (x.view(70, 3, 2, 64)[:, :, 0].reshape(70, 192), x.view(70, 3, 2, 64)[:, :, 1].reshape(70, 192))
        assert torch.allclose(whole.double().cpu(), P.activation(gate, act) * up, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d, rotary_dim, factor", [
    (48, 48, 1.0), (48, 32, 4.0), (48, 0, 1.0), (128, 128, 1.0),  # four elements per access: the per-token kernel
    (50, 20, 2.0), (50, 50, 1.0), (36, 36, 1.0),                  # widths that are not: the per-head kernel
])
def test_rope_and_cache_write(dtype, d, rotary_dim, factor):
    from turboserve_b200.ops import kernels

    nh, nkv, page = 5, 1, 8
    contexts, q_lens = [19, 1, 40], [19, 1, 30]  # 50 tokens: enough for the per-token kernel where the shape allows it
    _, _, k_pages, v_pages, table = paged_layout(contexts, page, nkv, d, dtype, DEV)
    k_before, v_before = k_pages.clone(), v_pages.clone()
    total = sum(q_lens)
    positions, seq_of = [], []
    for s, (c, n) in enumerate(zip(contexts, q_lens)):
        positions += list(range(c - n, c)); seq_of += [s] * n
    width = (nh + 2 * nkv) * d
    qkv = torch.randn(total, width).to(dtype)
    bias = torch.randn(width) * 0.5
    theta = 5000.0
    inv_freq = (1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))) if rotary_dim else None
    dev_qkv = qkv.to(DEV).clone()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.rope_cache_write(dev_qkv, bias.to(DEV), torch.tensor(positions, dtype=torch.int32, device=DEV),
                             torch.tensor(seq_of, dtype=torch.int32, device=DEV), table, k_pages, v_pages, total, nh, nkv, d,
                             inv_freq.to(DEV) if rotary_dim else None, rotary_dim, factor, True, status)
    assert status.item() == 0
    x = (qkv.double() + bias.double()).view(total, nh + 2 * nkv, d)
    ref = x.clone()
    if rotary_dim:
        cos, sin = P.rope_cos_sin(torch.tensor(positions), rotary_dim, theta, factor, torch.float64)
        ref[:, : nh + nkv, :rotary_dim] = P.apply_rope(x[:, : nh + nkv, :rotary_dim], cos, sin)
    got_q = dev_qkv.view(total, nh + 2 * nkv, d)[:, :nh].double().cpu()
    assert torch.allclose(got_q, ref[:, :nh], **tol(dtype))
    touched = torch.zeros(k_pages.shape[0], page, dtype=torch.bool)
    for t, (pos, s) in enumerate(zip(positions, seq_of)):
        pg, off = int(table[s, pos // page]), pos % page
        touched[pg, off] = True
        assert torch.allclose(k_pages[pg, off].double().cpu(), ref[t, nh: nh + nkv], **tol(dtype)), (t, pos)
        assert torch.allclose(v_pages[pg, off].double().cpu(), ref[t, nh + nkv:], **tol(dtype))
    # nothing else in the pool was written
    assert torch.equal(k_pages.cpu()[~touched], k_before.cpu()[~touched])
    assert torch.equal(v_pages.cpu()[~touched], v_before.cpu()[~touched])


@pytest.mark.parametrize("dtype", DTYPES)
def test_rope_gives_the_same_bits_for_few_and_for_many_tokens(dtype):
    """A step of many tokens runs a block per token, a step of few a warp per head: the same values either way."""
    from turboserve_b200.ops import kernels

    nh, nkv, d, page, n = 3, 2, 64, 16, 80
    _, _, k_pages, v_pages, table = paged_layout([n], page, nkv, d, dtype, DEV)
    width = (nh + 2 * nkv) * d
    qkv = torch.randn(n, width).to(dtype).to(DEV)
    bias = (torch.randn(width) * 0.5).to(DEV)
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))).to(DEV)
    positions = torch.arange(n, dtype=torch.int32, device=DEV)
    seq_of = torch.zeros(n, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    whole, k_whole, v_whole = qkv.clone(), k_pages.clone(), v_pages.clone()
    kernels.rope_cache_write(whole, bias, positions, seq_of, table, k_whole, v_whole, n, nh, nkv, d, inv_freq, d, 1.0, True, status)
    cut, k_cut, v_cut = qkv.clone(), k_pages.clone(), v_pages.clone()
    for lo in range(0, n, 8):
        kernels.rope_cache_write(cut[lo:lo + 8], bias, positions[lo:lo + 8], seq_of[lo:lo + 8], table, k_cut, v_cut, 8, nh, nkv, d,
                                 inv_freq, d, 1.0, True, status)
    assert status.item() == 0
    assert torch.equal(whole, cut) and torch.equal(k_whole, k_cut) and torch.equal(v_whole, v_cut)


def run_generic(q, k_pages, v_pages, table, seq_of, positions, nh, nkv, d, window, scale):
    from turboserve_b200.ops import kernels

    n = q.shape[0]
    out = torch.empty(n, nh * d, dtype=q.dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.paged_attention_generic(q.view(n, nh * d), out, k_pages, v_pages, table, seq_of, positions, n, nh, nkv, d,
                                    window, scale, status)
    assert status.item() == 0
    return out.view(n, nh, d)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh, nkv, d, page, window", [(6, 2, 48, 8, None), (3, 1, 80, 16, 20), (8, 8, 256, 4, None), (7, 1, 16, 32, 33)])
def test_generic_attention_over_scrambled_pages(dtype, nh, nkv, d, page, window):
    contexts, q_lens = [1, 37, 130, 64], [1, 5, 130, 1]
    k_dense, v_dense, k_pages, v_pages, table = paged_layout(contexts, page, nkv, d, dtype, DEV)
    q, positions, seq_of = pack_queries(contexts, q_lens, nh, d, dtype, DEV)
    scale = 0.37 / math.sqrt(d)
    out = run_generic(q.to(DEV), k_pages, v_pages, table, seq_of, positions, nh, nkv, d, window, scale).double().cpu()
    start = 0
    for s, n in enumerate(q_lens):
        ref = attention_reference(q[start:start + n].float(), k_dense[s], v_dense[s], positions[start:start + n].cpu(), window, scale)
        assert torch.allclose(out[start:start + n], ref, **tol(dtype)), f"sequence {s}"
        start += n


@pytest.mark.parametrize("dtype", DTYPES)
def test_generic_attention_finds_one_far_key_and_respects_the_window_edge(dtype):
    """Random scores would hide a skipped key: make one key's score stand out."""
    nh, nkv, d, page = 2, 1, 32, 8
    ctx = 301
    gen = torch.Generator().manual_seed(7)
    for far, window, expect_hit in [(3, None, True), (ctx - 41, 40, False), (ctx - 40, 40, True), (ctx - 1, 40, True)]:
        k = torch.randn(ctx, nkv, d, generator=gen) * 0.01
        v = torch.randn(ctx, nkv, d, generator=gen)
        direction = torch.randn(d, generator=gen); direction /= direction.norm()
        k[far, 0] = direction * 30
        v[far, 0] = 7.0
        q = (direction * 30).repeat(1, nh, 1)
        pages = -(-ctx // page)
        order = torch.randperm(pages + 2).tolist()
        k_pages = torch.zeros(pages + 2, page, nkv, d); v_pages = torch.zeros(pages + 2, page, nkv, d)
        table = torch.tensor([order[:pages]], dtype=torch.int32)
        for p in range(pages):
            lo, hi = p * page, min((p + 1) * page, ctx)
            k_pages[order[p], : hi - lo] = k[lo:hi]; v_pages[order[p], : hi - lo] = v[lo:hi]
        out = run_generic(q.to(dtype).to(DEV), k_pages.to(dtype).to(DEV), v_pages.to(dtype).to(DEV), table.to(DEV),
                          torch.zeros(1, dtype=torch.int32, device=DEV), torch.tensor([ctx - 1], dtype=torch.int32, device=DEV),
                          nh, nkv, d, window, 1.0)
        if expect_hit:
            assert (out.float() - 7.0).abs().max() < 0.05, (far, window)
        else:  # the key just behind the window is not seen: what is left is close to the mean of the window's values
            assert out.float().abs().max() < 1.5, (far, window)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m, n, k", [(1, 24, 8), (37, 101, 77), (64, 130, 1000), (200, 65, 64)])
def test_gemm_simt(dtype, m, n, k):
    from turboserve_b200.ops import kernels

    a = torch.randn(m, k).to(dtype); w = torch.randn(n, k).to(dtype); bias = torch.randn(n)
    out = torch.empty(m, n, dtype=dtype, device=DEV)
    kernels.gemm_simt(a.to(DEV), w.to(DEV), out, bias.to(DEV))
    ref = a.double() @ w.double().T + bias.double()
    t = dict(atol=1e-4, rtol=1e-5) if dtype == torch.float32 else dict(atol=0.15, rtol=2e-2)
    assert torch.allclose(out.double().cpu(), ref, **t)
    out32 = torch.empty(m, n, dtype=torch.float32, device=DEV)
    kernels.gemm_simt(a.to(DEV), w.to(DEV), out32)
    assert torch.allclose(out32.double().cpu(), ref - bias.double(), atol=1e-4 * math.sqrt(k), rtol=1e-5)
    # a row's result does not depend on how many rows there are
    one = torch.empty(1, n, dtype=torch.float32, device=DEV)
    kernels.gemm_simt(a[m - 1:].to(DEV), w.to(DEV), one)
    assert torch.equal(one[0], out32[m - 1])


@pytest.mark.parametrize("m", [1, 3, 8, 9, 16, 33, 64])
@pytest.mark.parametrize("n, k", [(24, 8), (100, 40), (257, 104), (96, 1000), (3584, 512), (50, 4096)])
def test_gemm_skinny(m, n, k):
    from turboserve_b200.ops.skinny import gemm_skinny

    a = torch.randn(m, k).to(torch.bfloat16); w = torch.randn(n, k).to(torch.bfloat16); bias = torch.randn(n)
    ref = a.double() @ w.double().T
    for ksplit in (0, 1, 2, 4, 8):
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
        gemm_skinny(a.to(DEV), w.to(DEV), out, None, ksplit=ksplit)
        assert torch.allclose(out.double().cpu(), ref, atol=2e-4 * math.sqrt(k), rtol=1e-5), ksplit
    out16 = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    gemm_skinny(a.to(DEV), w.to(DEV), out16, bias.to(DEV))
    assert torch.allclose(out16.double().cpu(), ref + bias.double(), atol=0.02 * math.sqrt(k), rtol=1e-2)


def test_gemm_skinny_refuses_what_it_cannot_do():
    from turboserve_b200.ops.kernels import KernelError
    from turboserve_b200.ops.skinny import gemm_skinny

    w = torch.zeros(16, 12, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError):
        gemm_skinny(torch.zeros(2, 12, dtype=torch.bfloat16, device=DEV), w, torch.zeros(2, 16, device=DEV))  # K % 8
    w = torch.zeros(16, 16, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError):
        gemm_skinny(torch.zeros(65, 16, dtype=torch.bfloat16, device=DEV), w, torch.zeros(65, 16, device=DEV))  # M > 64


def test_argmax_and_ties():
    from turboserve_b200.ops import kernels

    logits = torch.randn(5, 5003, device=DEV)
    logits[1, 77] = logits[1, 4000] = 50.0  # a tie: the lowest id wins
    logits[2, 5002] = 60.0
    tokens = torch.empty(5, dtype=torch.int32, device=DEV)
    kernels.argmax(logits, tokens)
    expect = logits.argmax(-1).tolist(); expect[1] = 77
    assert tokens.tolist() == expect


@pytest.mark.parametrize("vocab", [1000, 5003])
def test_sampling_stages_against_the_plain_sampler(vocab):
    from turboserve_b200.ops import kernels

    g = torch.Generator().manual_seed(vocab)
    rows = [
        dict(temperature=0.0), dict(temperature=1.0), dict(temperature=0.7, top_k=5), dict(temperature=1.3, top_p=0.6),
        dict(temperature=0.9, top_k=50, top_p=0.8), dict(temperature=0.0, repetition_penalty=1.7),
        dict(temperature=1.1, repetition_penalty=0.6, top_p=0.95), dict(temperature=2.0, top_k=1),
    ]
    n = len(rows)
    logits = torch.randn(n, vocab, generator=g) * 3
    histories = [torch.randint(0, vocab, (30,), generator=g).tolist() + [int(logits[i].argmax())] for i in range(n)]
    for counter in range(6):
        seeds = [1000 + 17 * i for i in range(n)]
        starts, flat = [0], []
        for i, r in enumerate(rows):
            if r.get("repetition_penalty", 1.0) != 1.0:
                flat += histories[i]
            starts.append(len(flat))
        tokens = torch.empty(n, dtype=torch.int32, device=DEV)
        logprobs = torch.empty(n, device=DEV)
        kernels.sample(
            logits.to(DEV), torch.empty(n * vocab, device=DEV), tokens,
            temperature=torch.tensor([r["temperature"] for r in rows], device=DEV),
            top_k=torch.tensor([r.get("top_k", 0) for r in rows], dtype=torch.int32, device=DEV),
            top_p=torch.tensor([r.get("top_p", 1.0) for r in rows], device=DEV),
            penalty=torch.tensor([r.get("repetition_penalty", 1.0) for r in rows], device=DEV),
            seed=torch.tensor(seeds, dtype=torch.int64, device=DEV),
            counter=torch.tensor([counter] * n, dtype=torch.int32, device=DEV),
            history=torch.tensor(flat, dtype=torch.int32, device=DEV),
            history_start=torch.tensor(starts, dtype=torch.int32, device=DEV), logprobs=logprobs,
        )
        for i, r in enumerate(rows):
            tok, lp = P.sample_token(logits[i], history=histories[i], seed=seeds[i], counter=counter, **r)
            assert tokens[i].item() == tok, (counter, i, r)
            assert abs(logprobs[i].item() - lp) < 1e-4


def test_sampling_follows_the_distribution_and_ignores_neighbours():
    from turboserve_b200.ops import kernels

    vocab, draws = 50, 4000
    row = torch.randn(vocab) * 2
    logits = row.repeat(draws, 1).to(DEV)
    tokens = torch.empty(draws, dtype=torch.int32, device=DEV)
    kernels.sample(logits, torch.empty(draws * vocab, device=DEV), tokens,
                   temperature=torch.ones(draws, device=DEV), seed=torch.full((draws,), 7, dtype=torch.int64, device=DEV),
                   counter=torch.arange(draws, dtype=torch.int32, device=DEV))
    freq = torch.bincount(tokens.long().cpu(), minlength=vocab).double() / draws
    assert (freq - torch.softmax(row.double(), 0)).abs().max() < 0.03
    # the same (seed, counter) draws the same token whatever else is in the batch
    alone = torch.empty(1, dtype=torch.int32, device=DEV)
    kernels.sample(logits[:1], torch.empty(vocab, device=DEV), alone, temperature=torch.ones(1, device=DEV),
                   seed=torch.full((1,), 7, dtype=torch.int64, device=DEV), counter=torch.tensor([123], dtype=torch.int32, device=DEV))
    assert alone.item() == tokens[123].item()


# -- tensor-core attention (bfloat16, head sizes 64 and 128) ------------------------------------------


def flash_case(nh, nkv, d, page, window, contexts, q_lens, seed=0):
    from turboserve_b200.ops import attention_bf16 as fa

    dtype = torch.bfloat16
    k_dense, v_dense, k_pages, v_pages, table = paged_layout(contexts, page, nkv, d, dtype, DEV, seed=seed)
    q, positions, seq_of = pack_queries(contexts, q_lens, nh, d, dtype, DEV, seed=seed + 1)
    scale = 0.9 / math.sqrt(d)
    refs, start = [], 0
    for s, n in enumerate(q_lens):
        refs.append(attention_reference(q[start:start + n].float(), k_dense[s], v_dense[s], positions[start:start + n].cpu(), window, scale))
        start += n
    total = sum(q_lens)
    qd = q.to(DEV).view(total, nh * d)
    return fa, qd, k_pages, v_pages, table, positions, seq_of, torch.cat(refs), scale


@pytest.mark.parametrize("nh, nkv, d, page, window", [
    (28, 4, 128, 16, None), (6, 2, 64, 8, None), (3, 1, 64, 32, 40), (14, 2, 128, 16, 100), (4, 4, 128, 64, None),
    (8, 1, 64, 128, 70), (40, 1, 64, 16, None),
])
def test_flash_prefill_mixed_query_lengths(nh, nkv, d, page, window):
    contexts, q_lens = [1, 37, 300, 64, 129, 200], [1, 5, 300, 1, 2, 67]
    fa, q, k_pages, v_pages, table, positions, seq_of, ref, scale = flash_case(nh, nkv, d, page, window, contexts, q_lens)
    total = sum(q_lens)
    qsl = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    ctx_lens = torch.tensor(contexts, dtype=torch.int32, device=DEV)
    out = torch.full((total, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    fa.flash_prefill(q, out, k_pages, v_pages, table, qsl, ctx_lens, len(contexts), total, nh, nkv, d, window, scale)
    got = out.view(total, nh, d).double().cpu()
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max().item() < 2e-2, (got - ref).abs().max().item()


@pytest.mark.parametrize("nh, nkv, d, page, window", [
    (28, 4, 128, 16, None), (6, 2, 64, 8, None), (3, 1, 64, 32, 40), (16, 1, 128, 16, 100), (4, 4, 128, 64, None),
    (14, 2, 128, 8, None), (8, 2, 128, 4, 50), (7, 1, 128, 128, None),
])
@pytest.mark.parametrize("splits", [1, 2, 7, 8, 9, 32])  # 2..8: joined inside a cluster; more: through scratch
@pytest.mark.parametrize("tma", [False, True])
def test_flash_decode_with_splits(nh, nkv, d, page, window, splits, tma):
    contexts = [1, 37, 300, 64, 129, 1000, 65]
    q_lens = [1] * len(contexts)
    fa, q, k_pages, v_pages, table, positions, seq_of, ref, scale = flash_case(nh, nkv, d, page, window, contexts, q_lens, seed=3)
    n = len(contexts) + 2  # two padding tokens that belong to no request
    pad = lambda t, fill: torch.cat([t, torch.full((2,), fill, dtype=t.dtype, device=DEV)])
    qp = torch.cat([q, torch.zeros(2, nh * d, dtype=torch.bfloat16, device=DEV)])
    out = torch.full((n, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    scratch = torch.full((max(4, fa.decode_scratch_floats(n, nh, splits, d)),), float("nan"), device=DEV)
    if tma:
        assert fa.tma_decode_supports(d, page, nh // nkv)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        fa.flash_decode_tma(qp, out, k_pages, v_pages, table, pad(seq_of, -1), pad(positions, 0), n, nh, nkv, d, window, scale,
                            splits, scratch, status)
        assert status.item() == 0
    else:
        fa.flash_decode(qp, out, k_pages, v_pages, table, pad(seq_of, -1), pad(positions, 0), n, nh, nkv, d, window, scale, splits, scratch)
    got = out[: len(contexts)].view(len(contexts), nh, d).double().cpu()
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max().item() < 2e-2, (got - ref).abs().max().item()


@pytest.mark.parametrize("decode", [False, True, "tma"])
def test_flash_kernels_find_one_far_key_and_respect_the_window_edge(decode):
    from turboserve_b200.ops import attention_bf16 as fa

    nh, nkv, d, page = 7, 1, 128, 16
    ctx = 1301
    gen = torch.Generator().manual_seed(11)
    for far, window, expect_hit in [(3, None, True), (700, None, True), (ctx - 41, 40, False), (ctx - 40, 40, True), (ctx - 1, 40, True)]:
        k = torch.randn(ctx, nkv, d, generator=gen) * 0.01
        v = torch.randn(ctx, nkv, d, generator=gen)
        direction = torch.randn(d, generator=gen); direction /= direction.norm()
        k[far, 0] = direction * 30
        v[far, 0] = 7.0
        pages = -(-ctx // page)
        order = torch.randperm(pages + 2).tolist()
        k_pages = torch.zeros(pages + 2, page, nkv, d); v_pages = torch.zeros(pages + 2, page, nkv, d)
        table = torch.tensor([order[:pages]], dtype=torch.int32)
        for p in range(pages):
            lo, hi = p * page, min((p + 1) * page, ctx)
            k_pages[order[p], : hi - lo] = k[lo:hi]; v_pages[order[p], : hi - lo] = v[lo:hi]
        if window:  # pages wholly behind the window are gone, as the cache manager would have it
            table[0, : (ctx - window) // page] = -1
        q = (direction * 30).repeat(1, nh).to(torch.bfloat16).to(DEV)
        out = torch.empty(1, nh * d, dtype=torch.bfloat16, device=DEV)
        args = (k_pages.to(torch.bfloat16).to(DEV), v_pages.to(torch.bfloat16).to(DEV), table.to(DEV))
        if decode:
            scratch = torch.empty(fa.decode_scratch_floats(1, nh, 5, d), device=DEV)
            run = fa.flash_decode_tma if decode == "tma" else fa.flash_decode
            run(q, out, *args, torch.zeros(1, dtype=torch.int32, device=DEV),
                torch.tensor([ctx - 1], dtype=torch.int32, device=DEV), 1, nh, nkv, d, window, 1.0, 5, scratch)
        else:
            fa.flash_prefill(q, out, *args, torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                             torch.tensor([ctx], dtype=torch.int32, device=DEV), 1, 1, nh, nkv, d, window, 1.0)
        if expect_hit:
            assert (out.float() - 7.0).abs().max() < 0.05, (far, window)
        else:  # what is left is close to the mean of the 40 values in the window
            assert out.float().abs().max() < 1.5, (far, window)


@pytest.mark.parametrize("nh, nkv, d, page, window, contexts", [
    (28, 4, 128, 16, None, [3000] + [40, 17, 64, 100, 9, 33, 1]),        # one context far above the others
    (6, 2, 64, 8, None, [1500, 20, 31, 8]),                              # the register-fed kernel
    (10, 2, 128, 16, 200, [2500, 130, 60, 1, 90, 77]),                   # with a window
    (28, 4, 128, 16, None, [300, 280, 310, 290]),                        # an even batch: as before
    (28, 4, 128, 16, None, [300] * 40 + [5000]),                         # many requests: 1 part each when even, 8 here
])
def test_a_lopsided_decode_batch_is_cut_by_each_requests_own_length(nh, nkv, d, page, window, contexts):
    from turboserve_b200.engine.batch import RequestSlice, StepContext, Workspace, build_step_batch, skew_class
    from turboserve_b200.ops import kernels
    from turboserve_b200.ops.skinny import num_sms

    q_lens = [1] * len(contexts)
    fa, q, k_pages, v_pages, table, positions, seq_of, ref, scale = flash_case(nh, nkv, d, page, window, contexts, q_lens, seed=41)
    rows = table.cpu().tolist()
    slices = [RequestSlice([0], c - 1, [[p for p in rows[i] if p >= 0]], i, [0]) for i, c in enumerate(contexts)]
    batch = build_step_batch(slices, 1, DEV)
    assert batch.is_decode_only and batch.decode_skew == skew_class(contexts)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ctx = StepContext(batch=batch, workspace=Workspace(DEV), dtype=torch.bfloat16, device=torch.device(DEV), status=status)
    out = torch.full((len(contexts), nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    before = kernels.launch_count()
    assert fa.paged_attention_bf16(q, out, k_pages, v_pages, batch.block_tables[0], batch, nh, nkv, d, window, scale, ctx)
    launched = kernels.launch_count() - before
    sms, n = num_sms(torch.device(DEV)), len(contexts)
    even = fa.decode_splits(n, nkv, sms)
    if batch.decode_skew >= fa.WORK_LIST_FROM and fa.tma_decode_supports(d, page, nh // nkv):
        # the kernel that walks a work list: every request cut by its own length, joined by the second kernel
        assert launched == 2
        items = batch.decode_items[int(window or 0)]
        parts_of = items.parts_of[:n].tolist()
        visible = [min(c, window) if window else c for c in contexts]
        assert parts_of[visible.index(max(visible))] == max(parts_of)
        if max(visible) > 1024:
            assert max(parts_of) > min(parts_of)
        assert items.num_items == sum(parts_of) <= n + fa.decode_item_target(nkv, sms)
    else:
        parts = min(even * batch.decode_skew, fa.MAX_SPLITS, (n + fa.SKEW_SPLIT_ROOM * ((2 * sms) // nkv)) // n)
        if batch.decode_skew > 1:
            assert parts > even or even == fa.MAX_SPLITS
        assert launched == (2 if parts > fa.CLUSTER_MAX_SPLITS else 1)  # more parts than a cluster holds: the join kernel follows
    assert status.item() == 0
    got = out.view(len(contexts), nh, d).double().cpu()
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max().item() < 2e-2, (got - ref).abs().max().item()


# -- tcgen05 attention for steps with prompts (bfloat16, head size 128) -------------------------------


def run_flash_tc(q, k_pages, v_pages, table, contexts, q_lens, nh, nkv, d, window, scale, max_context=None):
    from turboserve_b200.ops import attention_tc as atc

    total = sum(q_lens)
    qsl = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=DEV)
    ctx_lens = torch.tensor(contexts, dtype=torch.int32, device=DEV)
    out = torch.full((total, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert atc.supports(q, out, d, k_pages.shape[1], nh // nkv, scale)
    atc.flash_prefill_tc(q, out, k_pages, v_pages, table, qsl, ctx_lens, len(contexts), total, nh, nkv, d, window, scale, status,
                         max_context=max_context if max_context is not None else max(contexts))
    assert status.item() == 0
    return out


@pytest.mark.parametrize("nh, nkv, page, window, contexts, q_lens", [
    (28, 4, 16, None, [1, 37, 300, 64, 129, 200], [1, 5, 300, 1, 2, 67]),
    (14, 2, 16, 100, [1, 37, 300, 64, 129, 200], [1, 5, 300, 1, 2, 67]),
    (4, 4, 64, None, [500, 20], [500, 3]),
    (8, 1, 128, 70, [300, 700], [300, 2]),
    (2, 2, 8, None, [260], [130]),
    (6, 2, 4, 33, [90, 200], [90, 40]),
    (5, 1, 32, None, [1500], [2]),
    (40, 1, 16, 300, [900, 128], [513, 128]),
    # few row tiles with many keys each
    (28, 4, 16, None, [1500, 800], [1500, 800]),
    (8, 2, 64, 1000, [2000, 5], [600, 5]),
    (3, 3, 16, None, [1100, 790, 769], [40, 3, 769]),
])
def test_flash_prefill_tc_mixed_query_lengths(nh, nkv, page, window, contexts, q_lens):
    d = 128
    _, q, k_pages, v_pages, table, positions, seq_of, ref, scale = flash_case(nh, nkv, d, page, window, contexts, q_lens, seed=5)
    out = run_flash_tc(q, k_pages, v_pages, table, contexts, q_lens, nh, nkv, d, window, scale)
    got = out.view(sum(q_lens), nh, d).double().cpu()
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max().item() < 2e-2, (got - ref).abs().max().item()
    again = run_flash_tc(q, k_pages, v_pages, table, contexts, q_lens, nh, nkv, d, window, scale)
    assert torch.equal(again, out)


@pytest.mark.parametrize("nh, nkv, page, window, contexts, q_lens, parts", [
    (28, 4, 16, None, [3000], [300], True),             # a portion late in a long context
    (8, 2, 64, 1000, [2000, 5], [600, 5], True),        # a window: the last parts of a tile are empty
    (3, 3, 16, None, [1100, 790, 769], [40, 3, 769], True),
    (28, 4, 16, None, [1500, 800], [1500, 800], False),  # more row tiles than multiprocessors: whole
    (4, 4, 32, None, [300], [20], False),               # too few keys to be worth it
])
def test_flash_prefill_tc_cuts_the_keys_of_few_row_tiles_into_parts(nh, nkv, page, window, contexts, q_lens, parts):
    from turboserve_b200.ops import kernels

    d = 128
    _, q, k_pages, v_pages, table, positions, seq_of, ref, scale = flash_case(nh, nkv, d, page, window, contexts, q_lens, seed=31)
    whole = run_flash_tc(q, k_pages, v_pages, table, contexts, q_lens, nh, nkv, d, window, scale, max_context=0)
    before = kernels.launch_count()
    cut = run_flash_tc(q, k_pages, v_pages, table, contexts, q_lens, nh, nkv, d, window, scale)
    assert kernels.launch_count() - before == (2 if parts else 1)
    got = cut.view(sum(q_lens), nh, d).double().cpu()
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max().item() < 2e-2
    # the same sums in another order: a few units in the last place of bfloat16
    assert (cut.float() - whole.float()).abs().max().item() <= 2.0 ** -6 * max(1.0, ref.abs().max().item())
    if not parts:
        assert torch.equal(cut, whole)


@pytest.mark.parametrize("nh, nkv, d, page, window, contexts, q_lens", [
    (10, 2, 128, 16, None, [700, 33, 1500, 300, 64, 90], [1, 1, 1, 37, 1, 5]),   # three lead; the fourth single is in the middle
    (10, 2, 128, 16, None, [300, 90, 1500, 700, 64, 33], [37, 5, 1, 1, 1, 1]),   # the scheduler's order: prompts, then decodes
    (6, 2, 64, 8, 50, [200, 120, 77], [1, 1, 60]),                               # head size 64: decode + mma.sync kernels
    (6, 2, 64, 8, 50, [120, 77, 200, 31], [1, 60, 1, 1]),                        # both ends
    (4, 4, 128, 32, None, [40, 900], [1, 2]),
    (4, 4, 128, 32, None, [40, 900, 17], [2, 3, 2]),                             # nobody brings one token: one kernel as before
])
def test_mixed_steps_send_single_tokens_at_either_end_to_the_decode_kernel(nh, nkv, d, page, window, contexts, q_lens):
    from turboserve_b200.engine.batch import RequestSlice, StepContext, Workspace, build_step_batch
    from turboserve_b200.ops import kernels

    fa, q, k_pages, v_pages, table, positions, seq_of, ref, scale = flash_case(nh, nkv, d, page, window, contexts, q_lens, seed=21)
    rows = table.cpu().tolist()
    slices = [RequestSlice([0] * n, c - n, [[p for p in rows[i] if p >= 0]], i, []) for i, (c, n) in enumerate(zip(contexts, q_lens))]
    batch = build_step_batch(slices, 1, DEV)
    assert batch.num_leading_decode == next((i for i, n in enumerate(q_lens) if n != 1), len(q_lens))
    assert batch.num_trailing_decode == next((i for i, n in enumerate(reversed(q_lens)) if n != 1), len(q_lens))
    ends = (1 if batch.num_leading_decode else 0) + (1 if batch.num_trailing_decode else 0)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ctx = StepContext(batch=batch, workspace=Workspace(DEV), dtype=torch.bfloat16, device=torch.device(DEV), status=status)
    out = torch.full((sum(q_lens), nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    before = kernels.launch_count()
    assert fa.paged_attention_bf16(q, out, k_pages, v_pages, batch.block_tables[0], batch, nh, nkv, d, window, scale, ctx)
    launched = kernels.launch_count() - before  # the decode kernel may bring a join kernel along
    assert 1 + ends <= launched <= 2 + 2 * ends  # the tiled kernel too, when it cuts the keys of its tiles into parts
    assert status.item() == 0
    got = out.view(sum(q_lens), nh, d).double().cpu()
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max().item() < 2e-2, (got - ref).abs().max().item()


def test_flash_prefill_tc_finds_one_far_key_and_respects_the_window_edge():
    nh, nkv, d, page = 7, 1, 128, 16
    ctx = 1301
    gen = torch.Generator().manual_seed(12)
    for far, window, expect_hit in [(3, None, True), (700, None, True), (ctx - 41, 40, False), (ctx - 40, 40, True), (ctx - 1, 40, True)]:
        k = torch.randn(ctx, nkv, d, generator=gen) * 0.01
        v = torch.randn(ctx, nkv, d, generator=gen)
        direction = torch.randn(d, generator=gen); direction /= direction.norm()
        k[far, 0] = direction * 30
        v[far, 0] = 7.0
        pages = -(-ctx // page)
        order = torch.randperm(pages + 2, generator=gen).tolist()
        k_pages = torch.zeros(pages + 2, page, nkv, d); v_pages = torch.zeros(pages + 2, page, nkv, d)
        table = torch.tensor([order[:pages]], dtype=torch.int32)
        for p in range(pages):
            lo, hi = p * page, min((p + 1) * page, ctx)
            k_pages[order[p], : hi - lo] = k[lo:hi]; v_pages[order[p], : hi - lo] = v[lo:hi]
        if window:  # pages wholly behind the window are gone, as the cache manager would have it
            table[0, : (ctx - window) // page] = -1
        # two query tokens: the last of the context and the one before it (only the last is checked)
        q = (direction * 30).repeat(2, nh).to(torch.bfloat16).to(DEV)
        out = run_flash_tc(q, k_pages.to(torch.bfloat16).to(DEV), v_pages.to(torch.bfloat16).to(DEV), table.to(DEV),
                           [ctx], [2], nh, nkv, d, window, 1.0)[1:]
        if expect_hit:
            assert (out.float() - 7.0).abs().max() < 0.05, (far, window)
        else:
            assert out.float().abs().max() < 1.5, (far, window)


def test_flash_prefill_tc_flags_a_missing_page_in_reach():
    nh, nkv, d, page = 4, 2, 128, 16
    contexts, q_lens = [100], [100]
    _, q, k_pages, v_pages, table, positions, seq_of, ref, scale = flash_case(nh, nkv, d, page, None, contexts, q_lens, seed=9)
    from turboserve_b200.ops import attention_tc as atc

    table = table.clone()
    table[0, 2] = -1
    out = torch.empty(100, nh * d, dtype=torch.bfloat16, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    atc.flash_prefill_tc(q, out, k_pages, v_pages, table, torch.tensor([0, 100], dtype=torch.int32, device=DEV),
                         torch.tensor([100], dtype=torch.int32, device=DEV), 1, 100, nh, nkv, d, None, scale, status)
    assert status.item() & 4


def test_flash_prefill_tc_refuses_what_it_cannot_do():
    from turboserve_b200.ops import attention_tc as atc

    q = torch.zeros(4, 256, dtype=torch.bfloat16, device=DEV)
    assert not atc.supports(q, q, 64, 16, 2, 0.1)          # head size
    assert not atc.supports(q, q, 128, 2, 2, 0.1)          # page smaller than 4
    assert not atc.supports(q, q, 128, 24, 2, 0.1)         # page no power of two
    assert not atc.supports(q.float(), q, 128, 16, 2, 0.1) # dtype
    assert not atc.supports(q, q, 128, 16, 2, 0.0)         # scale
    assert atc.supports(q, q, 128, 16, 2, 0.1)


@pytest.mark.parametrize("m", [1, 8, 16, 17, 33, 64, 100, 128])
@pytest.mark.parametrize("n, k", [(24, 8), (100, 72), (257, 1000), (128, 64), (3584, 512), (777, 2304)])
def test_gemm_tc(m, n, k):
    """The TMA + tcgen05 product: ragged N and K (zero-filled by the tensor map), K slices, both outputs."""
    from turboserve_b200.ops.tc import gemm_tc

    a = torch.randn(m, k).to(torch.bfloat16); w = torch.randn(n, k).to(torch.bfloat16); bias = torch.randn(n)
    ref = a.double() @ w.double().T
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for slices in (1, 2, 3):
        if slices > 1 and k < 512:
            continue
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
        gemm_tc(a.to(DEV), w.to(DEV), out, bias.to(DEV), slices=slices, status=status)
        assert torch.allclose(out.double().cpu(), ref + bias.double(), atol=2e-4 * math.sqrt(k), rtol=1e-5), slices
    out16 = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    gemm_tc(a.to(DEV), w.to(DEV), out16, None, slices=1, status=status)
    assert torch.allclose(out16.double().cpu(), ref, atol=0.02 * math.sqrt(k), rtol=1e-2)
    assert status.item() == 0


@pytest.mark.parametrize("act", ["silu", "gelu_pytorch_tanh"])
@pytest.mark.parametrize("m", [1, 8, 17, 64, 128])
@pytest.mark.parametrize("inter, k", [(64, 64), (576, 264), (1920, 1000)])
def test_gemm_tc_with_the_activation_in_its_epilogue(act, m, inter, k):
    from turboserve_b200.ops import kernels, tc
    from turboserve_b200.ops.linear import GATE_BLOCK, interleave_gate_up

    g = torch.Generator().manual_seed(m + inter)
    gate = (torch.randn(inter, k, generator=g) * 0.2).to(torch.bfloat16).to(DEV)
    up = (torch.randn(inter, k, generator=g) * 0.2).to(torch.bfloat16).to(DEV)
    bias_g, bias_u = torch.randn(inter, generator=g).to(DEV), torch.randn(inter, generator=g).to(DEV)
    x = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    weight, block = interleave_gate_up(gate, up)
    bias, _ = interleave_gate_up(bias_g, bias_u)
    assert block == GATE_BLOCK and weight.shape == (2 * inter, k)
    assert torch.equal(weight[:64], gate[:64]) and torch.equal(weight[64:128], up[:64])
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    fused = torch.full((m, inter), float("nan"), dtype=torch.bfloat16, device=DEV)
    tc.gemm_tc_gated(x, weight, fused, bias, act, m, status=status)
    # the same through the plain product and the activation kernel: equal bit for bit
    both = torch.empty(m, 2 * inter, dtype=torch.bfloat16, device=DEV)
    tc.gemm_tc(x, weight, both, bias, m, slices=1, status=status)
    apart = torch.empty(m, inter, dtype=torch.bfloat16, device=DEV)
    kernels.act_mul(both, apart, act, m, block=block)
    assert status.item() == 0
    assert torch.equal(fused, apart)
    xd = x.double().cpu()
    gd = xd @ gate.double().cpu().T + bias_g.double().cpu()
    ud = xd @ up.double().cpu().T + bias_u.double().cpu()
    ref = (torch.nn.functional.silu(gd) if act == "silu" else torch.nn.functional.gelu(gd, approximate="tanh")) * ud
    err = (fused.double().cpu() - ref).abs().max().item()
    assert err < 0.03 * max(1.0, ref.abs().max().item()), err


def test_act_mul_reads_interleaved_runs():
    from turboserve_b200.ops import kernels

    inter = 192
    g = torch.Generator().manual_seed(3)
    for dtype in DTYPES:
        gate = torch.randn(5, inter, generator=g).to(dtype).to(DEV)
        up = torch.randn(5, inter, generator=g).to(dtype).to(DEV)
        plain = torch.cat([gate, up], dim=1).contiguous()
        runs = torch.stack([gate.view(5, 3, 64), up.view(5, 3, 64)], dim=2).reshape(5, 2 * inter).contiguous()
        a, b = torch.empty(5, inter, dtype=dtype, device=DEV), torch.empty(5, inter, dtype=dtype, device=DEV)
        kernels.act_mul(plain, a, "silu")
        kernels.act_mul(runs, b, "silu", block=64)
        assert torch.equal(a, b)
    with pytest.raises(kernels.KernelError):
        kernels.act_mul(plain, a, "silu", block=40)  # the runs must divide the width


def test_linear_rule_picks_a_kernel_for_every_shape():
    """Every branch of ops/linear.py against a float64 product."""
    from turboserve_b200.ops.linear import linear

    for m, n, k in [(3, 20000, 64), (40, 16400, 128), (5, 96, 200), (30, 96, 200), (100, 17000, 64), (7, 50, 100), (6, 5120, 72)]:
        a = torch.randn(m, k).to(torch.bfloat16); w = (torch.randn(n, k) / math.sqrt(k)).to(torch.bfloat16); bias = torch.randn(n)
        ref = a.double() @ w.double().T + bias.double()
        for dtype in (torch.bfloat16, torch.float32):
            out = torch.empty(m, n, dtype=dtype, device=DEV)
            linear(a.to(DEV), w.to(DEV), out, bias.to(DEV))
            assert (out.double().cpu() - ref).abs().max().item() < 0.06, (m, n, k, dtype)


def test_a_row_of_float32_logits_does_not_depend_on_how_many_rows_are_asked_for():
    """Up to 64 rows the head runs the tcgen05 product, beyond that the library: both hand back
    float32 accumulators (not a rounded bfloat16 result), so the same row of activations gives
    logits that differ by rounding of the sum only, far below a bfloat16 step, whether it is one
    of 3 rows or of 65. A bfloat16 detour would tie hundreds of a wide vocabulary's logits."""
    from turboserve_b200.ops.linear import linear

    torch.manual_seed(5)
    k, n = 256, 20000
    w = (torch.randn(n, k) / math.sqrt(k)).to(torch.bfloat16).to(DEV)
    x = torch.randn(65, k).to(torch.bfloat16).to(DEV)
    few = torch.empty(3, n, dtype=torch.float32, device=DEV)
    many = torch.empty(65, n, dtype=torch.float32, device=DEV)
    linear(x[:3].contiguous(), w, few)
    linear(x, w, many)
    ref = (x[:3].double() @ w.double().T)
    assert (few.double() - ref).abs().max().item() < 1e-5 and (many[:3].double() - ref).abs().max().item() < 1e-5
    # not values on the bfloat16 grid
    assert (many[:3] != many[:3].to(torch.bfloat16).float()).float().mean().item() > 0.9
    biased = torch.empty(65, n, dtype=torch.bfloat16, device=DEV)
    bias = torch.randn(n, device=DEV)
    linear(x, w, biased, bias)
    assert torch.equal(biased[:3], (ref + bias.double()).to(torch.bfloat16)) or \
        ((biased[:3].double() - (ref + bias.double())).abs() <= (ref + bias.double()).abs() * 2 ** -8).all()


@pytest.mark.parametrize("nh, nkv, page, window, rotary_dim, with_bias", [
    (28, 4, 16, None, 128, True), (7, 1, 16, None, 128, False), (10, 2, 8, 70, 64, True), (16, 1, 64, None, 0, True),
    (3, 3, 4, 33, 128, True),
])
@pytest.mark.parametrize("splits", [1, 3, 8, 9])
def test_decode_attention_that_encodes_and_appends_itself_equals_the_two_kernel_path(nh, nkv, page, window, rotary_dim, with_bias, splits):
    """``flash_decode_tma_fused`` takes the raw q/k/v product: bias, rotation and the append to the cache
    happen inside it. Same output (to a bfloat16 step of the softmax's different order) and the
    very same bytes in the cache as the rotation kernel followed by the TMA-fed decode kernel;
    nothing but each token's own slot of the pages is written, the product itself is not touched."""
    from turboserve_b200.ops import attention_bf16 as fa
    from turboserve_b200.ops import kernels

    d = 128
    contexts = [1, 37, 300, 64, 129, 1000, 65, 128]  # position 0, page edges, a token whose own tile holds no cached key (pos 64, 128)
    k_dense, v_dense, k_pages, v_pages, table = paged_layout(contexts, page, nkv, d, torch.bfloat16, DEV, seed=41)
    n = len(contexts) + 1  # one padding token
    gen = torch.Generator().manual_seed(42)
    width = (nh + 2 * nkv) * d
    qkv = torch.randn(n, width + 8, generator=gen).to(torch.bfloat16).to(DEV)  # a row stride wider than the heads
    bias = torch.randn(width, generator=gen).to(DEV) if with_bias else None
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / max(rotary_dim, 1)))).to(DEV) if rotary_dim else None
    positions = torch.tensor([c - 1 for c in contexts] + [0], dtype=torch.int32, device=DEV)
    seq_of = torch.tensor(list(range(len(contexts))) + [-1], dtype=torch.int32, device=DEV)
    scale = 1.0 / math.sqrt(d)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    scratch = torch.full((max(4, fa.decode_scratch_floats(n, nh, splits, d)),), float("nan"), device=DEV)

    # the two-kernel path on copies
    qkv_a, k_a, v_a = qkv.clone(), k_pages.clone(), v_pages.clone()
    kernels.rope_cache_write(qkv_a, bias, positions, seq_of, table, k_a, v_a, n, nh, nkv, d, inv_freq, rotary_dim, 2.0, True, status)
    out_a = torch.full((n, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    fa.flash_decode_tma(qkv_a, out_a, k_a, v_a, table, seq_of, positions, n, nh, nkv, d, window, scale, splits, scratch, status)
    # the fused kernel on the originals
    qkv_b, k_b, v_b = qkv.clone(), k_pages.clone(), v_pages.clone()
    out_b = torch.full((n, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    fusion = fa.DecodeFusion(bias, inv_freq, rotary_dim, 2.0, True)
    fa.flash_decode_tma_fused(qkv_b, fusion, out_b, k_b, v_b, table, seq_of, positions, n, nh, nkv, d, window, scale, splits, scratch, status)
    torch.cuda.synchronize()
    assert status.item() == 0
    assert torch.equal(qkv_b, qkv)                                   # the product is read only
    assert torch.equal(k_b, k_a) and torch.equal(v_b, v_a)           # the same bytes appended, nothing else touched
    assert not torch.equal(k_b, k_pages)
    live = len(contexts)
    assert torch.isfinite(out_b[:live].float()).all() and torch.isnan(out_b[live:].float()).all()
    assert (out_b[:live].float() - out_a[:live].float()).abs().max().item() <= 2.0 ** -6 * max(1.0, out_a[:live].float().abs().max().item())
    # and against float64 from the appended cache: the dense keys with the token's own (rotated) key and value at the end
    for s, ctx in enumerate(contexts):
        rows = table[s].cpu().tolist()
        k_all = torch.cat([k_a[rows[p // page], p % page][None] for p in range(ctx)]).float().cpu()
        v_all = torch.cat([v_a[rows[p // page], p % page][None] for p in range(ctx)]).float().cpu()
        q_rot = qkv_a[s, : nh * d].view(1, nh, d).float().cpu()
        ref = attention_reference(q_rot, k_all, v_all, torch.tensor([ctx - 1]), window, scale)
        assert (out_b[s].view(1, nh, d).double().cpu() - ref).abs().max().item() < 2e-2, s
    # without the append (a run that only reads): the cache is left alone and the token still sees itself
    k_c, v_c = k_pages.clone(), v_pages.clone()
    out_c = torch.empty_like(out_b)
    fa.flash_decode_tma_fused(qkv_b, fa.DecodeFusion(bias, inv_freq, rotary_dim, 2.0, False), out_c, k_c, v_c, table, seq_of,
                              positions, n, nh, nkv, d, window, scale, splits, scratch, status)
    assert torch.equal(k_c, k_pages) and torch.equal(v_c, v_pages) and torch.equal(out_c[:live], out_b[:live])


@pytest.mark.parametrize("kind", ["registers", "registers64", "tma", "tma64", "fused"])
def test_decode_kernels_mask_and_flag_a_page_that_is_missing_inside_the_visible_keys(kind):
    """A table entry of -1 inside a request's visible keys (a page given back too early) is never
    read as if it held zeros: its keys get no weight, and bit 4 of the status word says so.
    A page that is missing where no key is visible (behind a window) raises nothing."""
    from turboserve_b200.ops import attention_bf16 as fa

    nh, nkv, page = 4, 2, 16
    d = 64 if kind.endswith("64") else 128
    ctx, lost = 200, 5  # page 5 holds keys 80 .. 95
    k_dense, v_dense, k_pages, v_pages, table = paged_layout([ctx], page, nkv, d, torch.bfloat16, DEV, seed=51)
    q, positions, seq_of = pack_queries([ctx], [1], nh, d, torch.bfloat16, DEV, seed=52)
    q = q.to(DEV).view(1, nh * d)
    scale = 1.0 / math.sqrt(d)
    keep = torch.ones(ctx, dtype=torch.bool)
    keep[lost * page:(lost + 1) * page] = False
    # what the softmax over the other keys gives: positions are what matters to the mask, so drop the rows and keep causality trivial
    ref = attention_reference(q.view(1, nh, d).float().cpu(), k_dense[0][keep], v_dense[0][keep], torch.tensor([int(keep.sum()) - 1]), None, scale)

    def run(tab, window):
        out = torch.full((1, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        scratch = torch.empty(max(4, fa.decode_scratch_floats(1, nh, 3, d)), device=DEV)
        if kind.startswith("registers"):
            fa.flash_decode(q, out, k_pages, v_pages, tab, seq_of, positions, 1, nh, nkv, d, window, scale, 3, scratch, status)
        elif kind.startswith("tma"):
            fa.flash_decode_tma(q, out, k_pages, v_pages, tab, seq_of, positions, 1, nh, nkv, d, window, scale, 3, scratch, status)
        else:
            # the fused kernel takes the product: no bias, no rotation, and the token's own key and value in place
            qkv = torch.cat([q, k_dense[0][ctx - 1].reshape(1, -1).to(torch.bfloat16).to(DEV), v_dense[0][ctx - 1].reshape(1, -1).to(torch.bfloat16).to(DEV)], dim=1).contiguous()
            fa.flash_decode_tma_fused(qkv, fa.DecodeFusion(None, None, 0, 1.0, True), out, k_pages, v_pages, tab, seq_of, positions,
                                      1, nh, nkv, d, window, scale, 3, scratch, status)
        return out, status.item()

    whole, flags = run(table, None)
    assert flags == 0
    holed = table.clone()
    holed[0, lost] = -1
    out, flags = run(holed, None)
    assert flags == 4
    assert (out.view(1, nh, d).double().cpu() - ref).abs().max().item() < 2e-2
    assert (out.float() - whole.float()).abs().max().item() > 1e-3  # 16 of 200 keys are gone: the result moved
    behind, flags = run(holed, 60)  # a window of 60: keys 140 .. 199, page 5 is out of reach
    assert flags == 0 and torch.isfinite(behind.float()).all()


@pytest.mark.parametrize("vocab, chunks", [(777, 1), (777, 8), (152064, 8), (1000, 3)])
def test_sampling_with_options_by_state_slot_equals_sampling_with_options_by_row(vocab, chunks):
    """``sample_slots`` finds a row's options through its state slot, derives the index of the token
    being generated from the request's length, skips padding rows, and cuts rows that need one
    pass into several blocks: the ids equal those of ``sample`` given the same options row by row."""
    from turboserve_b200.ops import kernels

    gen = torch.Generator().manual_seed(vocab)
    num_slots, rows = 12, 9
    logits = (torch.randn(rows, vocab, generator=gen) * 3).to(DEV)
    logits[2, 5] = logits[2, 700] = logits[2].max() + 1.0  # a tie for the greedy row: the lower id wins in every cut
    # per slot: temperature, top_k, top_p, seed, prompt length
    slot_opts = {3: (0.0, 0, 1.0, 1, 4), 7: (0.8, 0, 1.0, 22, 9), 0: (1.3, 40, 1.0, 5, 1), 11: (0.6, 0, 0.9, 8, 30),
                 5: (1.0, 25, 0.7, 13, 2), 9: (0.0, 10, 0.5, 3, 7), 2: (2.0, 0, 1.0, 77, 100), 6: (0.9, 0, 1.0, 1 << 40, 3)}
    row_slot = [3, 7, 9, 0, 11, 5, 2, 6, 4]
    row_seq = [0, 1, 2, 3, 4, 5, 6, 7, -1]  # the last row is padding
    row_context = [10, 9, 50, 17, 33, 2, 164, 5, 0]
    temperature = torch.zeros(num_slots); top_p = torch.ones(num_slots)
    top_k = torch.zeros(num_slots, dtype=torch.int32); prompt_len = torch.zeros(num_slots, dtype=torch.int32)
    seed = torch.zeros(num_slots, dtype=torch.int64)
    for slot, (t, k, p, s, plen) in slot_opts.items():
        temperature[slot], top_k[slot], top_p[slot], seed[slot], prompt_len[slot] = t, k, p, s, plen
    work = torch.empty(rows * vocab, device=DEV)
    partial = torch.zeros(rows * (4 * chunks + 1), dtype=torch.int32, device=DEV)
    dev = lambda t: t.to(DEV)
    for _ in range(2):  # twice: the counters in `partial` are left at zero
        tokens = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
        kernels.sample_slots(logits, work, tokens, rows, temperature=dev(temperature), top_k=dev(top_k), top_p=dev(top_p),
                             seed=dev(seed), prompt_len=dev(prompt_len), seq_slot=dev(torch.tensor(row_slot, dtype=torch.int32)),
                             seq_of_token=dev(torch.tensor(row_seq, dtype=torch.int32)), seq_context=dev(torch.tensor(row_context, dtype=torch.int32)),
                             partial=partial, chunks=chunks)
        live = rows - 1
        by_row = torch.empty(live, dtype=torch.int32, device=DEV)
        opts = [slot_opts[s] for s in row_slot[:live]]
        kernels.sample(logits[:live], work, by_row, temperature=dev(torch.tensor([o[0] for o in opts])),
                       top_k=dev(torch.tensor([o[1] for o in opts], dtype=torch.int32)), top_p=dev(torch.tensor([o[2] for o in opts])),
                       seed=dev(torch.tensor([o[3] for o in opts], dtype=torch.int64)),
                       counter=dev(torch.tensor([c - o[4] for c, o in zip(row_context, opts)], dtype=torch.int32)))
        assert tokens[:live].tolist() == by_row.tolist()
        assert tokens[live].item() == -7 and tokens[2].item() == 5
        assert int(partial.view(rows, -1)[:, 0].abs().sum()) == 0
    # and against the plain sampler
    for r in (0, 1, 4, 7):
        t, k, p, s, plen = slot_opts[row_slot[r]]
        expect, _ = P.sample_token(logits[r].cpu(), temperature=t, top_k=k, top_p=p, seed=s, counter=row_context[r] - plen)
        assert tokens[r].item() == expect


@pytest.mark.parametrize("vocab, chunks", [(777, 8), (152064, 8), (1000, 1)])
def test_sampling_by_slot_with_a_penalty_from_the_bitmap_and_log_probabilities(vocab, chunks):
    """By slot the history of a request is a bitmap over the vocabulary: ``mark_seen`` sets the bits of
    a step's tokens for the slots that have a penalty (and for no other), the sampling kernel adds
    the token whose logits a row holds, and the ids and log-probabilities equal those of
    ``sample`` given the same histories as lists. The tokens are chosen so that the penalty
    decides: the largest logits of every row are in its history. A row finds its request as in a
    step with prompts in it: row -> token of the step -> request -> slot, none of them the identity."""
    from turboserve_b200.ops import kernels

    gen = torch.Generator().manual_seed(vocab + 1)
    num_slots, rows = 10, 7
    logits = (torch.randn(rows, vocab, generator=gen) * 3).to(DEV)
    # per slot: temperature, top_k, top_p, penalty, wants a log-probability, seed, prompt length
    slot_opts = {4: (0.0, 0, 1.0, 1.5, 1, 1, 3), 1: (0.9, 0, 1.0, 1.3, 0, 7, 2), 8: (1.1, 30, 0.9, 2.0, 0, 9, 5),
                 2: (0.7, 0, 0.8, 1.2, 1, 4, 1), 6: (0.0, 0, 1.0, 1.0, 1, 2, 6), 0: (1.0, 50, 1.0, 1.0, 0, 3, 2),
                 9: (0.0, 0, 1.0, 0.7, 0, 5, 4)}
    row_slot = [4, 1, 8, 2, 6, 0, 9]
    row_context = [9, 12, 30, 8, 20, 5, 11]
    words = (vocab + 31) // 32
    temperature = torch.zeros(num_slots); top_p = torch.ones(num_slots); penalty = torch.ones(num_slots)
    top_k = torch.zeros(num_slots, dtype=torch.int32); prompt_len = torch.zeros(num_slots, dtype=torch.int32)
    want = torch.zeros(num_slots, dtype=torch.int32); seed = torch.zeros(num_slots, dtype=torch.int64)
    for slot, (t, k, p, pen, lp, s, plen) in slot_opts.items():
        temperature[slot], top_k[slot], top_p[slot], penalty[slot], want[slot], seed[slot], prompt_len[slot] = t, k, p, pen, lp, s, plen
    dev = lambda t: t.to(DEV)
    penalty_dev = dev(penalty)
    # histories: the top logits of the row (so the penalty moves the choice), some random ids, the edges of the vocabulary
    histories = []
    for r in range(rows):
        top = logits[r].topk(6).indices.tolist()
        histories.append(top[:4] + torch.randint(0, vocab, (20,), generator=gen).tolist() + [0, vocab - 1, 31, 32])
    step_tokens = [h[0] for h in histories]  # the row's best token is the one its request ran in this step
    seen = torch.zeros(num_slots, words, dtype=torch.int32, device=DEV)
    seen[3].fill_(-1)  # a slot nobody uses: must stay as it is
    # One step's worth of tokens. The requests of the step come in the reverse order of the rows
    # (request q's logits are row rows - 1 - q), each brings its history but for the token at its
    # end, whose logits the row holds; mark_seen sees that last token as padding, so that only the
    # sampling kernel can have added it.
    token_ids, seq_of_token, last_token = [], [], {}
    for q in range(rows):
        r = rows - 1 - q
        token_ids += histories[r][1:] + [histories[r][0]]
        seq_of_token += [q] * len(histories[r])
        last_token[r] = len(token_ids) - 1
    seq_slot = dev(torch.tensor([row_slot[rows - 1 - q] for q in range(rows)], dtype=torch.int32))
    seq_context = dev(torch.tensor([row_context[rows - 1 - q] for q in range(rows)], dtype=torch.int32))
    without_last = list(seq_of_token)
    for r in range(rows):
        without_last[last_token[r]] = -1
    kernels.mark_seen(dev(torch.tensor(token_ids, dtype=torch.int32)), dev(torch.tensor(without_last, dtype=torch.int32)),
                      seq_slot, penalty_dev, seen, len(token_ids), vocab)
    marked = seen.cpu()
    assert marked[6].abs().sum() == 0 and marked[0].abs().sum() == 0  # slots without a penalty are not marked
    assert (marked[3] == -1).all() and marked[5].abs().sum() == 0
    bit = lambda slot, t: (int(marked[slot, t >> 5]) >> (t & 31)) & 1
    assert all(bit(4, t) for t in histories[0][1:]) and not bit(4, histories[0][0])
    assert sum(bin(int(w) & 0xFFFFFFFF).count("1") for w in marked[4]) == len(set(histories[0][1:]))

    work = torch.empty(rows * vocab, device=DEV)
    partial = torch.zeros(rows * (4 * chunks + 1), dtype=torch.int32, device=DEV)
    tokens = torch.full((rows,), -7, dtype=torch.int32, device=DEV)
    logprobs = torch.full((rows,), 123.0, device=DEV)
    kernels.sample_slots(logits, work, tokens, rows, temperature=dev(temperature), top_k=dev(top_k), top_p=dev(top_p),
                         seed=dev(seed), prompt_len=dev(prompt_len), seq_slot=seq_slot, seq_context=seq_context, partial=partial,
                         chunks=chunks, row_token=dev(torch.tensor([last_token[r] for r in range(rows)], dtype=torch.int32)),
                         seq_of_token=dev(torch.tensor(seq_of_token, dtype=torch.int32)),
                         step_tokens=dev(torch.tensor(token_ids, dtype=torch.int32)), penalty=penalty_dev, seen=seen,
                         want_logprob=dev(want), logprobs=logprobs)
    after = seen.cpu()
    assert (int(after[4, step_tokens[0] >> 5]) >> (step_tokens[0] & 31)) & 1  # the step's token joined the history
    assert after[6].abs().sum() == 0 and (after[3] == -1).all()
    opts = [slot_opts[s] for s in row_slot]
    by_row = torch.empty(rows, dtype=torch.int32, device=DEV)
    by_row_logprobs = torch.empty(rows, device=DEV)
    starts = [0]
    for h in histories:
        starts.append(starts[-1] + len(h))
    kernels.sample(logits, work, by_row, temperature=dev(torch.tensor([o[0] for o in opts])),
                   top_k=dev(torch.tensor([o[1] for o in opts], dtype=torch.int32)), top_p=dev(torch.tensor([o[2] for o in opts])),
                   penalty=dev(torch.tensor([o[3] for o in opts])), seed=dev(torch.tensor([o[5] for o in opts], dtype=torch.int64)),
                   counter=dev(torch.tensor([c - o[6] for c, o in zip(row_context, opts)], dtype=torch.int32)),
                   history_start=dev(torch.tensor(starts, dtype=torch.int32)),
                   history=dev(torch.tensor([t for h in histories for t in h], dtype=torch.int32)), logprobs=by_row_logprobs)
    assert tokens.tolist() == by_row.tolist()
    assert int(partial.view(rows, -1)[:, 0].abs().sum()) == 0
    for r, o in enumerate(opts):
        expect, logprob = P.sample_token(logits[r].cpu(), temperature=o[0], top_k=o[1], top_p=o[2], repetition_penalty=o[3],
                                         history=histories[r], seed=o[5], counter=row_context[r] - o[6])
        assert tokens[r].item() == expect, r
        if o[4]:
            assert abs(logprobs[r].item() - logprob) < 1e-4
            assert abs(logprobs[r].item() - by_row_logprobs[r].item()) <= 1e-5  # the row's sum is added up in another order
        else:
            assert logprobs[r].item() == 123.0  # nobody asked: not written
    assert tokens[0].item() != logits[0].argmax().item()  # the penalty decided the greedy row


@pytest.mark.parametrize("nh, nkv, d, page, window", [(28, 4, 128, 16, None), (5, 1, 128, 8, 300), (16, 2, 128, 64, None),
                                                      (14, 2, 64, 16, None), (6, 2, 64, 4, 200)])
def test_decode_attention_over_a_work_list(nh, nkv, d, page, window):
    """Every request cut into parts by its own length: more parts than a short request has 64-key tiles
    (some are empty), one part (the output is written at once, the join kernel skips it), unused
    items and a padding token at the end of the list."""
    from turboserve_b200.engine.batch import DecodeItems, plan_decode_items
    from turboserve_b200.ops import attention_bf16 as fa

    contexts = [5000, 1, 70, 640, 129, 64]
    q_lens = [1] * len(contexts)
    _, q, k_pages, v_pages, table, positions, seq_of, ref, scale = flash_case(nh, nkv, d, page, window, contexts, q_lens, seed=61)
    live, n = len(contexts), len(contexts) + 1
    visible = [min(c, window) if window else c for c in contexts]
    item_token, item_part, parts_of, first_item = plan_decode_items(visible, target_items=40, min_keys=64)
    parts_of[2], first_item = 3, None  # a 70-key request in three parts: its third part has no tile
    first_item = [sum(parts_of[:i]) for i in range(live)]
    pairs = [(i, p) for i in sorted(range(live), key=lambda r: -visible[r]) for p in range(parts_of[i])]
    item_token, item_part = [t for t, _ in pairs] + [-1, -1], [p for _, p in pairs] + [0, 0]
    dev = lambda values: torch.tensor(values, dtype=torch.int32, device=DEV)
    items = DecodeItems(dev(item_token), dev(item_part), dev(parts_of + [1]), dev(first_item + [0]), len(item_token))
    assert max(parts_of) > 3 and min(parts_of) == 1
    qp = torch.cat([q, torch.zeros(1, nh * d, dtype=torch.bfloat16, device=DEV)])
    pad = lambda t, fill: torch.cat([t, torch.full((1,), fill, dtype=t.dtype, device=DEV)])
    out = torch.full((n, nh * d), float("nan"), dtype=torch.bfloat16, device=DEV)
    scratch = torch.full((items.num_items * nh * (d + 2),), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    fa.flash_decode_tma_items(qp, out, k_pages, v_pages, table, pad(seq_of, -1), pad(positions, 0), n, nh, nkv, d, window, scale,
                              items, scratch, status)
    assert status.item() == 0
    got = out[:live].view(live, nh, d).double().cpu()
    assert torch.isfinite(got).all() and torch.isnan(out[live:].float()).all()
    assert (got - ref).abs().max().item() < 2e-2, (got - ref).abs().max().item()


def test_the_forms_of_the_float32_product_give_the_same_bits():
    """Rows 0..63 of a product of 200 rows (the 128x128 tiling) equal the product of those 64 rows alone
    (the 64x64 tiling) bit for bit, and so do 1 to 16 of them through the weight-streaming form, at
    sizes that are no multiple of any tile (k = 77 leaves a chunk of one float, n = 130 two features
    in the last warp) and with unaligned rows."""
    from turboserve_b200.ops import kernels

    torch.manual_seed(9)
    for k, n, pad in [(200, 150, 0), (1030, 257, 0), (77, 130, 3), (77, 130, 0), (3584, 520, 0), (18944, 64, 0)]:
        a = torch.randn(200, k + pad, device=DEV)[:, :k]   # pad: a row stride that is no multiple of four
        w = torch.randn(n, k + pad, device=DEV)[:, :k] / math.sqrt(k)
        bias = torch.randn(n, device=DEV)
        big = torch.empty(200, n, device=DEV)
        small = torch.empty(64, n, device=DEV)
        kernels.gemm_simt(a, w, big, bias)
        kernels.gemm_simt(a[:64], w, small, bias, 64)
        assert torch.equal(big[:64], small), (k, n, pad)
        ref = a.double() @ w.double().T + bias.double()
        assert (big.double() - ref).abs().max().item() < 1e-4 * max(1.0, ref.abs().max().item())
        # and the weight-streaming form that up to 16 rows take when their stride is a multiple of four floats (else the 64x64 tiling again)
        for rows in (1, 3, 8, 9, 16):
            few = torch.full((rows, n), float("nan"), device=DEV)
            kernels.gemm_simt(a[5:5 + rows], w, few, bias, rows)
            assert torch.equal(few, big[5:5 + rows]), (k, n, pad, rows)
            plain = torch.full((rows, n), float("nan"), device=DEV)
            kernels.gemm_simt(a[5:5 + rows], w, plain, None, rows)
            assert torch.isfinite(plain).all() and (plain.double() - (ref[5:5 + rows] - bias.double())).abs().max().item() < 1e-4 * max(1.0, ref.abs().max().item())
