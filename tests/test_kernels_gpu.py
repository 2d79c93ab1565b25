"""Each CUDA kernel alone against a plain torch reference of the same operation, at sizes
other than the tiny models': widths and vocabularies that are no power of two, head sizes
16..256, any number of heads and groups, ragged batches."""

import math

import pytest
import torch

import plain_qwen3 as plain
from ondeviceinfer_b200.kernels import ops

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def close(actual, expected, dtype, scale=1.0):
    actual, expected = actual.float().cpu(), expected.float().cpu()
    if dtype == "float32":
        assert torch.allclose(actual, expected, atol=2e-5 * scale, rtol=2e-5), float((actual - expected).abs().max())
    else:
        limit = 2e-2 * max(1.0, float(expected.abs().max()))
        assert float((actual - expected).abs().max()) <= limit, float((actual - expected).abs().max())


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("V,H,n", [(389, 80, 7), (1000, 4096, 3)])
def test_embed(dtype, V, H, n):
    torch.manual_seed(0)
    table = torch.randn(V, H).to(DT[dtype]).to(DEV)
    ids = torch.randint(0, V, (n,), dtype=torch.int32, device=DEV)
    ids[0], ids[-1] = V - 1, 0
    out = torch.empty(n, H, dtype=torch.float32, device=DEV)
    ops.embed(table, ids, out)
    assert torch.equal(out.cpu(), table.float().cpu()[ids.cpu().long()])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("H,eps", [(80, 1e-5), (1000, 1e-6), (4096, 3e-6), (5120, 1e-6)])
def test_rmsnorm_and_row_gather(dtype, H, eps):
    torch.manual_seed(1)
    x = (torch.randn(9, H) * 3).to(DEV)
    w = (1 + 0.1 * torch.randn(H)).to(DEV)
    out = torch.empty(9, H, dtype=DT[dtype], device=DEV)
    ops.rmsnorm(x, w, eps, out)
    expected = plain.rms_norm(x.cpu().to(DT[dtype]), w.cpu().to(DT[dtype]), eps)
    close(out, expected, dtype)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    picked = torch.empty(3, H, dtype=DT[dtype], device=DEV)
    ops.rmsnorm(x, w, eps, picked, rows)
    assert torch.equal(picked, out[rows.long()])


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("H", [80, 4096, 5120])
def test_rmsnorm_with_a_pending_residual_add(dtype, H):
    """x += add in place and the norm of the sum in one pass: the same bits as the add followed by the norm."""
    torch.manual_seed(12)
    x = torch.randn(5, H)
    add = torch.randn(5, H).to(DT[dtype])
    w = (1 + 0.1 * torch.randn(H)).to(DEV)
    two_x, one_x = x.clone().to(DEV), x.clone().to(DEV)
    two, one = torch.empty(5, H, dtype=DT[dtype], device=DEV), torch.empty(5, H, dtype=DT[dtype], device=DEV)
    ops.residual_add(two_x, add.to(DEV))
    ops.rmsnorm(two_x, w, 1e-6, two)
    assert ops.rmsnorm_adds(one_x, w, one, add.to(DEV))
    ops.rmsnorm(one_x, w, 1e-6, one, add=add.to(DEV))
    assert torch.equal(one_x, two_x) and torch.equal(one, two)
    assert torch.equal(one_x.cpu(), x + add.float())
    assert not ops.rmsnorm_adds(one_x, w, one, add.to(DEV).float() if dtype == "bfloat16" else add.to(DEV).bfloat16())
    with pytest.raises(ops.KernelError):
        ops.rmsnorm(one_x, w, 1e-6, one, rows=torch.arange(5, dtype=torch.int32, device=DEV), add=add.to(DEV))


def test_rope_table_matches_host_angles():
    theta, dim = 1e6, 128
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    pos = torch.tensor([0, 1, 63, 64, 4095, 40959], dtype=torch.int32)
    cos = torch.empty(len(pos), dim // 2, dtype=torch.float32, device=DEV)
    sin = torch.empty_like(cos)
    ops.rope_table(inv_freq.to(DEV), pos.to(DEV), cos, sin)
    ec, es = plain.rope_tables(pos, dim, theta, torch.float32)
    assert torch.allclose(cos.cpu(), ec[:, :dim // 2], atol=2e-7, rtol=0)
    assert torch.allclose(sin.cpu(), es[:, :dim // 2], atol=2e-7, rtol=0)


def paged_setup(lengths, past, nkv, d, dtype, ring_pages=0, page=64, seed=0):
    """Random keys/values for sequences with `past` cached and `lengths` new positions, laid
    into shuffled pages.  Returns pools, index tensors and the dense per-sequence K/V."""
    g = torch.Generator().manual_seed(seed)
    n_seqs = len(lengths)
    total = [p + t for p, t in zip(past, lengths)]
    per_seq = [min(-(-n // page), ring_pages) if ring_pages else -(-n // page) for n in total]
    n_pages = sum(per_seq) + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    k_pool = torch.zeros(n_pages, nkv, page, d)
    v_pool = torch.zeros(n_pages, nkv, page, d)
    page_lists, dense = [], []
    for s in range(n_seqs):
        pages = [order.pop() for _ in range(per_seq[s])]
        page_lists.append(pages)
        k = torch.randn(nkv, total[s], d, generator=g)
        v = torch.randn(nkv, total[s], d, generator=g)
        dense.append((k, v))
        for pos in range(total[s]):
            slot = (pos // page) % ring_pages if ring_pages else pos // page
            k_pool[pages[slot], :, pos % page] = k[:, pos]
            v_pool[pages[slot], :, pos % page] = v[:, pos]
    start = [0]
    for pages in page_lists:
        start.append(start[-1] + len(pages))
    cu = [0]
    for t in lengths:
        cu.append(cu[-1] + t)
    to = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return dict(k_pool=k_pool.to(DT[dtype]).to(DEV), v_pool=v_pool.to(DT[dtype]).to(DEV), dense=dense,
                page_start=to(start), page_ids=to([p for l in page_lists for p in l]), cu_q=to(cu), past=to(past),
                tok_seq=to([s for s, t in enumerate(lengths) for _ in range(t)]),
                tok_pos=to([past[s] + i for s, t in enumerate(lengths) for i in range(t)]))


def plain_attention(q, dense, lengths, past, nq, nkv, d, window, scale, dtype):
    """softmax(q k^T * scale + mask) v per sequence; q [tokens, nq, d]."""
    outs, offset, g = [], 0, nq // nkv
    for s, t in enumerate(lengths):
        k, v = dense[s]
        k, v = k.to(DT[dtype]).float(), v.to(DT[dtype]).float()
        qs = q[offset:offset + t].to(DT[dtype]).float().transpose(0, 1)          # [nq, t, d]
        scores = qs @ k.repeat_interleave(g, 0).transpose(-1, -2) * scale
        qpos = torch.arange(past[s], past[s] + t).unsqueeze(1)
        kpos = torch.arange(past[s] + t).unsqueeze(0)
        visible = kpos <= qpos
        if window:
            visible &= kpos > qpos - window
        scores = scores.masked_fill(~visible, float("-inf"))
        outs.append((torch.softmax(scores, -1) @ v.repeat_interleave(g, 0)).transpose(0, 1))
        offset += t
    return torch.cat(outs).reshape(-1, nq * d)


ATTN_CASES = [
    # d, nq, nkv, lengths, past, window, splits
    (16, 4, 2, [5, 11, 17], [0, 0, 0], 0, 1),
    (48, 6, 2, [1, 70, 33], [0, 0, 0], 0, 1),
    (128, 5, 1, [1, 1, 1, 1], [300, 64, 63, 0], 0, 1),          # decode, ragged pasts
    (128, 5, 1, [1, 1, 1, 1], [300, 64, 63, 0], 0, 4),          # the same with split keys
    (128, 32, 1, [9], [120], 0, 1),                              # 32 query heads on one kv head
    (64, 8, 8, [40, 3], [100, 200], 0, 1),                       # chunks on a cache, no grouping
    (256, 2, 1, [20, 1], [0, 77], 0, 1),
    (32, 3, 3, [130, 2], [0, 190], 50, 1),                       # window
    (32, 6, 2, [1, 1], [400, 70], 50, 3),                        # window, decode, splits
]


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("d,nq,nkv,lengths,past,window,splits", ATTN_CASES)
def test_attention_simt(dtype, d, nq, nkv, lengths, past, window, splits):
    torch.manual_seed(2)
    setup = paged_setup(lengths, past, nkv, d, dtype)
    n = sum(lengths)
    q = torch.randn(n, nq, d)
    scale = 1.0 / math.sqrt(d)
    out = torch.empty(n, nq * d, dtype=DT[dtype], device=DEV)
    partial = torch.empty(n * nq * splits * (d + 2), dtype=torch.float32, device=DEV) if splits > 1 else None
    ops.attention_simt(q.to(DT[dtype]).to(DEV), setup["k_pool"], setup["v_pool"], out, setup["cu_q"],
                       setup["past"], setup["page_start"], setup["page_ids"], n_seqs=len(lengths),
                       max_q_len=max(lengths), nq=nq, nkv=nkv, d=d, page_size=64, ring_pages=0, window=window,
                       scale=scale, splits=splits, partial=partial)
    expected = plain_attention(q, setup["dense"], lengths, past, nq, nkv, d, window, scale, dtype)
    close(out, expected, dtype, scale=4.0)


@pytest.mark.parametrize("dtype", DT)
def test_attention_finds_one_far_key_among_hundreds(dtype):
    """Random data would hide a key that is skipped: make one far key the only one that
    matters (its score stands out by a large margin) and ask for its value back."""
    d, nq, nkv = 128, 4, 2
    lengths, past = [1, 1, 300], [700, 64, 0]
    setup = paged_setup(lengths, past, nkv, d, dtype, seed=3)
    n = sum(lengths)
    q = torch.randn(n, nq, d) * 0.1
    targets = {0: 5, 1: 63, 2 + 299: 1}            # packed token -> the key position to find
    for tok, key in targets.items():
        seq = 0 if tok == 0 else (1 if tok == 1 else 2)
        k, v = setup["dense"][seq]
        direction = torch.nn.functional.normalize(k[:, key], dim=-1)       # [nkv, d]
        q[tok] = direction.repeat_interleave(nq // nkv, 0) * 40.0
    scale = 1.0 / math.sqrt(d)
    out = torch.empty(n, nq * d, dtype=DT[dtype], device=DEV)
    # the pools hold the rounded keys; keep the crafted queries as they are
    for splits in (1, 5):
        partial = torch.empty(n * nq * splits * (d + 2), dtype=torch.float32, device=DEV) if splits > 1 else None
        ops.attention_simt(q.to(DT[dtype]).to(DEV), setup["k_pool"], setup["v_pool"], out, setup["cu_q"],
                           setup["past"], setup["page_start"], setup["page_ids"], n_seqs=3, max_q_len=300,
                           nq=nq, nkv=nkv, d=d, page_size=64, ring_pages=0, window=0, scale=scale,
                           splits=splits if max(lengths) == 1 else 1, partial=partial)
        expected = plain_attention(q, setup["dense"], lengths, past, nq, nkv, d, 0, scale, dtype)
        close(out, expected, dtype, scale=4.0)
        for tok, key in targets.items():
            seq = 0 if tok == 0 else (1 if tok == 1 else 2)
            value = setup["dense"][seq][1][:, key].to(DT[dtype]).float().repeat_interleave(nq // nkv, 0).reshape(-1)
            assert float((out[tok].float().cpu() - value).abs().max()) < 0.05, (tok, key)


@pytest.mark.parametrize("dtype", DT)
def test_attention_window_edge(dtype):
    """The key just outside the window would dominate if it were seen; the key just inside
    must be seen.  Window 50, query at position 199: keys 150..199 are visible."""
    d, nq, nkv, window = 32, 2, 1, 50
    for inside in (False, True):
        setup = paged_setup([1], [199], nkv, d, dtype, seed=11)
        k, v = setup["dense"][0]
        key = 150 if inside else 149
        q = torch.nn.functional.normalize(k[:, key], dim=-1).repeat_interleave(nq, 0)[None] * 60.0
        out = torch.empty(1, nq * d, dtype=DT[dtype], device=DEV)
        ops.attention_simt(q.to(DT[dtype]).to(DEV), setup["k_pool"], setup["v_pool"], out, setup["cu_q"],
                           setup["past"], setup["page_start"], setup["page_ids"], n_seqs=1, max_q_len=1, nq=nq,
                           nkv=nkv, d=d, page_size=64, ring_pages=0, window=window, scale=1 / math.sqrt(d))
        expected = plain_attention(q[0][None].reshape(1, nq, d), setup["dense"], [1], [199], nq, nkv, d, window,
                                   1 / math.sqrt(d), dtype)
        close(out, expected, dtype, scale=4.0)
        value = v[:, key].to(DT[dtype]).float().repeat_interleave(nq, 0).reshape(-1)
        gap = float((out[0].float().cpu() - value).abs().max())
        assert (gap < 0.05) == inside, (inside, gap)


@pytest.mark.parametrize("dtype", DT)
@pytest.mark.parametrize("d,rot,nq,nkv,norm,ring", [(16, 16, 4, 2, True, 0), (128, 128, 8, 2, True, 0),
                                                    (48, 32, 3, 1, False, 0), (256, 64, 2, 2, True, 0),
                                                    (32, 32, 2, 1, True, 3), (64, 0, 2, 2, True, 0),
                                                    (128, 128, 6, 2, True, -1)])
def test_head_prep(dtype, d, rot, nq, nkv, norm, ring):
    """Per-head norm (or none), rotation of the first `rot` lanes (or none), cache write
    into shuffled pages (or a ring of pages), against plain torch."""
    torch.manual_seed(4)
    lengths, past = [3, 1, 70], [0, 200, 10]
    if ring == -1:          # many tokens: the form in which a warp takes several heads of a token
        lengths, past, ring = [200, 90], [0, 30], 0
    elif ring:
        lengths, past = [3, 1, 20], [0, 200, 100]
    setup = paged_setup(lengths, past, nkv, d, dtype, ring_pages=ring, seed=5)
    n = sum(lengths)
    tdt = DT[dtype]
    qkv = torch.randn(n, (nq + 2 * nkv) * d).to(tdt)
    qw, kw = (1 + 0.1 * torch.randn(d)), (1 + 0.1 * torch.randn(d))
    eps, theta = 1e-5, 10000.0
    k_pool, v_pool = torch.zeros_like(setup["k_pool"]), torch.zeros_like(setup["v_pool"])
    cos = sin = None
    if rot:
        inv_freq = 1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))
        cos = torch.empty(n, rot // 2, dtype=torch.float32, device=DEV)
        sin = torch.empty_like(cos)
        ops.rope_table(inv_freq.to(DEV), setup["tok_pos"], cos, sin)
    q_out = torch.empty(n, nq * d, dtype=tdt, device=DEV)
    ops.head_prep(qkv.to(DEV), q_out, k_pool, v_pool, qw.to(DEV) if norm else None, kw.to(DEV) if norm else None,
                  cos, sin, setup["tok_seq"], setup["tok_pos"], setup["page_start"], setup["page_ids"],
                  nq=nq, nkv=nkv, d=d, rot_dim=rot, page_size=64, ring_pages=ring, write_kv=True, eps=eps)
    # plain: norm in the model dtype's rounding, rotation on the first `rot` lanes
    pos = setup["tok_pos"].cpu()
    x = qkv.view(n, nq + 2 * nkv, d)
    q, k, v = x[:, :nq], x[:, nq:nq + nkv], x[:, nq + nkv:]
    if norm:
        q, k = plain.rms_norm(q, qw.to(tdt), eps), plain.rms_norm(k, kw.to(tdt), eps)
    if rot:
        c, s = plain.rope_tables(pos, rot, theta, torch.float32)

        def rotate(t):
            t = t.float()
            head = plain.apply_rope(t[..., :rot].transpose(0, 1), c, s).transpose(0, 1)
            return torch.cat((head, t[..., rot:]), -1)

        q, k = rotate(q), rotate(k)
    close(q_out.view(n, nq, d), q, dtype)
    page_start, page_ids = setup["page_start"].cpu(), setup["page_ids"].cpu()
    seqs = setup["tok_seq"].cpu()
    for t in range(n):
        slot = int(pos[t]) // 64
        slot = slot % ring if ring else slot
        page = int(page_ids[int(page_start[int(seqs[t])]) + slot])
        close(k_pool[page, :, int(pos[t]) % 64], k[t], dtype)
        assert torch.equal(v_pool[page, :, int(pos[t]) % 64].cpu(), v[t])
    written = (k_pool.float().abs().sum(-1) > 0).sum().item()
    assert written == n * nkv, "keys were written to rows that no token owns"
    # write_kv off: queries only, the cache is not touched
    k2, v2 = torch.zeros_like(k_pool), torch.zeros_like(v_pool)
    q2 = torch.empty_like(q_out)
    ops.head_prep(qkv.to(DEV), q2, k2, v2, qw.to(DEV) if norm else None, kw.to(DEV) if norm else None,
                  cos, sin, setup["tok_seq"], setup["tok_pos"], setup["page_start"], setup["page_ids"],
                  nq=nq, nkv=nkv, d=d, rot_dim=rot, page_size=64, ring_pages=ring, write_kv=False, eps=eps)
    assert torch.equal(q2, q_out) and float(k2.float().abs().sum()) == 0.0


@pytest.mark.parametrize("dtype", DT)
def test_silu_mul_and_residual_add(dtype):
    torch.manual_seed(6)
    n, I = 5, 208
    gu = (torch.randn(n, 2 * I) * 3).to(DT[dtype])
    out = torch.empty(n, I, dtype=DT[dtype], device=DEV)
    ops.silu_mul(gu.to(DEV), out)
    g, u = gu[:, :I].float(), gu[:, I:].float()
    close(out, torch.nn.functional.silu(g) * u, dtype)
    hidden = torch.randn(n, I)
    y = torch.randn(n, I).to(DT[dtype])
    h = hidden.clone().to(DEV)
    ops.residual_add(h, y.to(DEV))
    assert torch.equal(h.cpu(), hidden + y.float())


@pytest.mark.parametrize("M,N,K", [(1, 389, 96), (7, 64, 6), (130, 257, 97), (64, 192, 160), (33, 5, 4096)])
def test_gemm_f32_is_true_fp32_and_row_independent(M, N, K):
    torch.manual_seed(7)
    a, w = torch.randn(M, K), torch.randn(N, K)
    out = torch.empty(M, N, device=DEV)
    ops.gemm_f32(a.to(DEV), w.to(DEV), out)
    expected = (a.double() @ w.double().t()).float()
    assert torch.allclose(out.cpu(), expected, atol=1e-6 * K, rtol=1e-5)
    # a TF32 product would be off by ~1e-3 relative; make sure we are far below that
    assert float((out.cpu() - expected).abs().max()) < 2e-5 * math.sqrt(K)
    # a row's result does not depend on the other rows of the batch
    single = torch.empty(1, N, device=DEV)
    ops.gemm_f32(a[M // 2:M // 2 + 1].to(DEV), w.to(DEV), single)
    assert torch.equal(single[0], out[M // 2])
    # residual, in place
    res = torch.randn(M, N)
    r = res.clone().to(DEV)
    ops.gemm_f32(a.to(DEV), w.to(DEV), r, r)
    assert torch.allclose(r.cpu(), res + out.cpu(), atol=1e-6, rtol=1e-6)
    # a bias joins the product before the residual
    bias = torch.randn(N)
    r = res.clone().to(DEV)
    ops.gemm_f32(a.to(DEV), w.to(DEV), r, r, bias=bias.to(DEV))
    assert torch.equal(r.cpu(), (out.cpu() + bias) + res)


def test_sample_greedy_ties_and_temperature_against_plain():
    torch.manual_seed(8)
    V = 1237
    logits = torch.randn(6, V) * 2
    logits[0, 100] = logits[0, 900] = 50.0          # tie: the lower index wins
    logits[1, V - 1] = 60.0
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    ops.sample(logits.to(DEV), out, 0.0)
    assert out.tolist() == [int(torch.argmax(l)) for l in logits] and out[0] == 100 and out[1] == V - 1
    streams = torch.arange(6, dtype=torch.int32, device=DEV)
    for temperature in (0.8, 0.1, 2.5):
        for step in range(20):
            steps = torch.full((6,), step, dtype=torch.int32, device=DEV)
            ops.sample(logits.to(DEV), out, temperature, 11, streams, steps)
            for r in range(6):
                u = plain.uniform_draw(11, r, step)
                expected = plain.sample(logits[r], temperature, u)
                if out[r].item() != expected:
                    # only a draw within rounding of a CDF step may land on the neighbour
                    p = torch.softmax(logits[r].double() / temperature, 0).cumsum(0)
                    assert abs(out[r].item() - expected) == 1 and float((p - u).abs().min()) < 1e-5


def test_sample_wide_vocabulary_over_many_chunks():
    """A row cut into many chunks: ties across chunks, the maximum in the last (partial) chunk, and
    draws that land in early, middle and late chunks; twice, so that the tickets are seen to return to zero."""
    torch.manual_seed(9)
    V = 150001                                       # odd: rows start at unaligned addresses
    logits = torch.randn(5, V) * 3
    logits[0, 4097] = logits[0, 140000] = 40.0       # tie across chunks: the lower index wins
    logits[1, V - 1] = 45.0
    logits[2, 2048] = 45.0                           # first element of the second chunk
    logits[3] = -2.0                                 # flat but for a few heavy tokens spread over the row
    for i, idx in enumerate((5, 70000, 149990)):
        logits[3, idx] = 9.0 + i
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    dev = logits.to(DEV)
    streams = torch.arange(5, dtype=torch.int32, device=DEV)
    for _ in range(2):
        ops.sample(dev, out, 0.0)
        assert out.tolist() == [int(torch.argmax(l)) for l in logits] and out[0] == 4097
        seen = set()
        for temperature in (1.0, 0.3):
            cdfs = [torch.softmax(l.double() / temperature, 0).cumsum(0) for l in logits]
            for step in range(12):
                steps = torch.full((5,), step, dtype=torch.int32, device=DEV)
                ops.sample(dev, out, temperature, 5, streams, steps)
                for r in range(5):
                    u = plain.uniform_draw(5, r, step)
                    expected = plain.sample(logits[r], temperature, u)
                    seen.add((r, expected * 3 // V))
                    if out[r].item() != expected:
                        assert abs(out[r].item() - expected) == 1 and float((cdfs[r] - u).abs().min()) < 1e-5
        assert {(4, 0), (4, 1), (4, 2)} <= seen      # early, middle and late chunks were all drawn from


def test_kernels_refuse_what_they_cannot_take():
    x = torch.zeros(2, 8, device=DEV)
    with pytest.raises(ops.KernelError):
        ops.rmsnorm(x.cpu(), torch.ones(8), 1e-6, x.cpu())                       # no CPU path
    with pytest.raises(ops.KernelError):
        ops.rmsnorm(x, torch.ones(9, device=DEV), 1e-6, torch.empty_like(x))     # sizes disagree
    with pytest.raises(ops.KernelError):
        ops.gemm_f32(x, torch.zeros(4, 7, device=DEV), torch.empty(2, 4, device=DEV))
    with pytest.raises(ops.KernelError):
        ops.attention_simt(x, x, x, x, None, None, None, None, n_seqs=1, max_q_len=1, nq=1, nkv=1, d=24,
                           page_size=64, ring_pages=0, window=0, scale=1.0)       # head size not a multiple of 16
    with pytest.raises(ops.KernelError):
        ops.embed(x.half(), torch.zeros(2, dtype=torch.int32, device=DEV), torch.empty(2, 8, device=DEV))


GEMM_SHAPES = [
    # tokens, features, K, tile, splits (None: the plan's choice)
    (1, 389, 96, None, None), (8, 4096, 4096, None, None), (16, 128, 64, 16, 1),
    (33, 1000, 1000, None, None), (64, 1536, 2048, None, None), (40, 512, 4096, 64, 4),
    (130, 4096, 1024, 128, 2), (100, 389, 96, None, None), (300, 520, 200, 256, 1),
    (8, 520, 2048, 16, 8), (50, 389, 1024, 64, 3), (20, 256, 4096, 32, 12),
    (333, 208, 80, 128, 1), (1030, 1024, 512, None, None),
]


@pytest.mark.parametrize("biased", [False, True])
@pytest.mark.parametrize("epi", ["store_bf16", "store_f32", "residual", "swiglu"])
@pytest.mark.parametrize("tokens,N,K,tile,splits", GEMM_SHAPES)
def test_gemm_tcgen05(tokens, N, K, tile, splits, epi, biased):
    """The tensor-core product and its four epilogues against fp32 torch on the same bf16
    inputs: every tile width, K splits, several token tiles, ragged edges in all three sizes;
    with and without a bias per weight row."""
    code = {"store_bf16": ops.EPI_STORE_BF16, "store_f32": ops.EPI_STORE_F32, "residual": ops.EPI_RESIDUAL,
            "swiglu": ops.EPI_SWIGLU}[epi]
    if epi == "swiglu" and tile == 256:
        pytest.skip("the gated epilogue keeps two accumulators: tiles up to 128")
    torch.manual_seed(9)
    x = torch.randn(tokens, K).bfloat16().to(DEV)
    rows = 2 * N if epi == "swiglu" else N
    w = (torch.randn(rows, K) / math.sqrt(K)).bfloat16().to(DEV)
    bias = torch.randn(rows).to(DEV) if biased else None
    ref = (x.float() @ w.float().t()).cpu()
    if biased:
        ref = ref + bias.cpu()
    if epi == "store_bf16":
        out, expected = torch.empty(tokens, N, dtype=torch.bfloat16, device=DEV), ref
    elif epi == "store_f32":
        out, expected = torch.empty(tokens, N, dtype=torch.float32, device=DEV), ref
    elif epi == "residual":
        res = torch.randn(tokens, N)
        out, expected = res.clone().to(DEV), res + ref
    else:
        out = torch.empty(tokens, N, dtype=torch.bfloat16, device=DEV)
        expected = torch.nn.functional.silu(ref[:, :N]) * ref[:, N:]
    ops.gemm_bf16(x, w, out, code, bn=tile, splits=splits, bias=bias)
    torch.cuda.synchronize()
    ops.raise_on_kernel_fault()
    if epi == "store_f32":
        # K splits through a cluster and through global scratch add in the same order: same bits
        other = torch.empty_like(out)
        ops.gemm_bf16(x, w, other, code, bn=tile, splits=splits, cluster=False, bias=bias)
        assert torch.equal(other, out)
    if out.dtype == torch.bfloat16:
        close(out, expected, "bfloat16")
    else:
        assert torch.allclose(out.cpu(), expected, atol=1e-4, rtol=1e-4), float((out.cpu() - expected).abs().max())
    # launched again, the split tickets must have been left at zero
    if epi == "store_f32":
        again = torch.empty_like(out)
        ops.gemm_bf16(x, w, again, code, bn=tile, splits=splits, bias=bias)
        assert torch.equal(again, out)


NORM_GEMM_SHAPES = [
    # tokens, hidden (the normed rows' width), features of the product that consumes them, tile, splits
    (8, 4096, 6144, None, None), (1, 200, 389, None, None), (16, 1000, 520, 16, 1), (5, 136, 256, 16, 2),
    (32, 4096, 1024, None, None), (20, 520, 640, 32, 3), (3, 64, 128, 16, 1),
    (1, 8, 8, None, None), (32, 72, 136, None, None), (17, 4104, 200, None, None),      # one k-block; widths off every tile edge
]


@pytest.mark.parametrize("gated", [False, True])
@pytest.mark.parametrize("tokens,H,N,tile,splits", NORM_GEMM_SHAPES)
def test_gemm_tcgen05_norm_prologue_and_sums_of_squares(tokens, H, N, tile, splits, gated):
    """A residual product that leaves the sums of squares of its rows, then a product that takes those
    rows through the fused RMSNorm: against the stand-alone norm kernel followed by the plain product
    (same roundings, so nearly the same bits) and against fp32 torch."""
    torch.manual_seed(21)
    K0 = 192
    a = torch.randn(tokens, K0).bfloat16().to(DEV)
    w0 = (torch.randn(H, K0) / math.sqrt(K0)).bfloat16().to(DEV)
    rows = (torch.randn(tokens, H) * 3).to(DEV)
    start = rows.clone()
    parts = torch.full((ops.gemm_bf16_sumsq_parts(H), tokens), float("nan"), device=DEV)
    assert ops.gemm_bf16_gives_sumsq(tokens, H, K0)
    ops.gemm_bf16(a, w0, rows, ops.EPI_RESIDUAL, sumsq_out=parts)
    torch.cuda.synchronize()
    expected_rows = start.cpu() + a.float().cpu() @ w0.float().cpu().t()
    assert torch.allclose(rows.cpu(), expected_rows, atol=1e-4, rtol=1e-4)
    padded = torch.zeros(tokens, parts.shape[0] * 128)
    padded[:, :H] = rows.cpu()
    expected_parts = (padded.view(tokens, -1, 128) ** 2).sum(-1).t()
    assert torch.allclose(parts.cpu(), expected_parts, rtol=1e-5, atol=1e-6), float((parts.cpu() - expected_parts).abs().max())

    g = (1.0 + 0.2 * torch.randn(H)).to(DEV)
    eps = 1e-5
    w_rows = 2 * N if gated else N
    w = (torch.randn(w_rows, H) / math.sqrt(H)).bfloat16().to(DEV)
    epi = ops.EPI_SWIGLU if gated else ops.EPI_STORE_BF16
    fused = torch.empty(tokens, N, dtype=torch.bfloat16, device=DEV)
    ops.gemm_bf16(None, w, fused, epi, bn=tile, splits=splits, norm=(rows, g, parts, eps))
    normed = torch.empty(tokens, H, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(rows, g, eps, normed)
    plain_way = torch.empty_like(fused)
    ops.gemm_bf16(normed, w, plain_way, epi, bn=tile, splits=splits)
    torch.cuda.synchronize()
    ops.raise_on_kernel_fault()
    # the two ways differ only where 1/rms, summed in another order, moves a value across a rounding step
    differ = (fused.float() - plain_way.float()).abs()
    scale = plain_way.float().abs().max().item()
    assert float(differ.max()) <= 0.02 * scale and float((differ > 0).float().mean()) < 0.05, (float(differ.max()), scale)
    r = rows.cpu()
    y = (r * torch.rsqrt((r * r).mean(-1, keepdim=True) + eps)).bfloat16().float() * g.cpu()
    ref = y.bfloat16().float() @ w.float().cpu().t()
    expected = torch.nn.functional.silu(ref[:, :N]) * ref[:, N:] if gated else ref
    close(fused, expected, "bfloat16")


@pytest.mark.parametrize("lengths,past,K,nq,nkv,norm,rot,lazy,ring,biased", [
    ([1] * 8, [300, 64, 63, 1000, 0, 5, 127, 128], 4096, 32, 8, True, True, True, 0, False),     # a decode step, a cluster per head
    ([1] * 8, [300, 64, 63, 1000, 0, 5, 127, 128], 4096, 32, 8, True, True, False, 0, True),
    ([3, 1, 16], [0, 200, 10], 256, 4, 2, True, True, False, 0, False),                          # a short K: one split, 32 columns
    ([3, 1, 16], [0, 200, 10], 256, 4, 2, False, False, True, 0, True),                          # neither norm nor rotation
    ([1, 1, 1], [70, 2, 900], 1024, 6, 3, True, False, True, 0, True),
    ([5, 6], [0, 64], 2048, 2, 1, False, True, False, 0, False),
    ([1, 1, 2], [500, 130, 62], 512, 4, 2, True, True, True, 2, False),                          # a ring of two pages per sequence
])
def test_gemm_tcgen05_prepares_heads_in_its_epilogue(lengths, past, K, nq, nkv, norm, rot, lazy, ring, biased):
    """The q/k/v product with the head preparation in its epilogue against the product followed by the
    head-preparation kernel: the same bits in the queries and in the cache, nothing written elsewhere."""
    torch.manual_seed(23)
    d = 128
    setup = paged_setup(lengths, past, nkv, d, "bfloat16", ring_pages=ring, seed=24)
    n = sum(lengths)
    w = (torch.randn((nq + 2 * nkv) * d, K) / math.sqrt(K)).bfloat16().to(DEV)
    qw = (1 + 0.1 * torch.randn(d)).to(DEV) if norm else None
    kw = (1 + 0.1 * torch.randn(d)).to(DEV) if norm else None
    cos = sin = None
    if rot:
        inv_freq = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        cos = torch.empty(n, d // 2, dtype=torch.float32, device=DEV)
        sin = torch.empty_like(cos)
        ops.rope_table(inv_freq.to(DEV), setup["tok_pos"], cos, sin)
    rows = (torch.randn(n, K) * 2).to(DEV)
    g = (1 + 0.1 * torch.randn(K)).to(DEV)
    x = torch.empty(n, K, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(rows, g, 1e-6, x)
    parts = torch.zeros(ops.gemm_bf16_sumsq_parts(K), n, device=DEV)
    padded = torch.zeros(n, parts.shape[0] * 128, device=DEV)
    padded[:, :K] = rows
    parts.copy_((padded.view(n, -1, 128) ** 2).sum(-1).t())
    common = dict(nq=nq, nkv=nkv, d=d, rot_dim=d if rot else 0, page_size=64, ring_pages=ring, write_kv=True, eps=1e-5)
    tail = (qw, kw, cos, sin, setup["tok_seq"], setup["tok_pos"], setup["page_start"], setup["page_ids"])

    bias = torch.randn(w.shape[0]).to(DEV) if biased else None
    qkv = torch.empty(n, w.shape[0], dtype=torch.bfloat16, device=DEV)
    if lazy:
        ops.gemm_bf16(None, w, qkv, ops.EPI_STORE_BF16, norm=(rows, g, parts, 1e-6), bias=bias)
    else:
        ops.gemm_bf16(x, w, qkv, ops.EPI_STORE_BF16, bias=bias)
    if biased:      # the bias is in the projections that the two forms share
        plain_qkv = x.float() @ w.float().t() + bias
        assert float((qkv.float() - plain_qkv).abs().max()) <= 0.02 * float(plain_qkv.abs().max())
    q_two = torch.zeros(n, nq * d, dtype=torch.bfloat16, device=DEV)
    k_two, v_two = torch.zeros_like(setup["k_pool"]), torch.zeros_like(setup["v_pool"])
    ops.head_prep(qkv, q_two, k_two, v_two, *tail, **common)

    assert ops.gemm_bf16_fuses_head_prep(n, w.shape[0], K, d=d, rot_dim=d if rot else 0, rotated=rot, write_kv=True)
    q_one = torch.zeros_like(q_two)
    k_one, v_one = torch.zeros_like(k_two), torch.zeros_like(v_two)
    block = ops.head_prep(None, q_one, k_one, v_one, *tail, **common)
    ops.gemm_bf16(None if lazy else x, w, None, ops.EPI_HEAD_PREP, head_prep=block,
                  norm=(rows, g, parts, 1e-6) if lazy else None, bias=bias)
    torch.cuda.synchronize()
    ops.raise_on_kernel_fault()
    assert float(q_two.float().abs().sum()) > 0 and float(k_two.float().abs().sum()) > 0
    assert torch.equal(q_one, q_two) and torch.equal(k_one, k_two) and torch.equal(v_one, v_two)


def test_gemm_tcgen05_refuses_unaligned_k():
    x = torch.zeros(4, 12, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 12, dtype=torch.bfloat16, device=DEV)
    assert not ops.gemm_bf16_supported(x, w)
    with pytest.raises(ops.KernelError):
        ops.gemm_bf16(x, w, torch.empty(4, 8, dtype=torch.bfloat16, device=DEV), ops.EPI_STORE_BF16)


MMA_CASES = [
    # d, nq, nkv, lengths, past, splits
    (16, 4, 2, [5, 11, 17], [0, 0, 0], 1),
    (48, 6, 2, [1, 70, 33], [0, 0, 0], 1),
    (128, 32, 8, [200, 64, 65, 1], [0, 0, 0, 0], 1),           # whole prompts, page edges
    (128, 4, 1, [40, 3, 130], [100, 200, 7], 1),                # chunks on a cache
    (64, 8, 8, [1, 1, 1], [0, 63, 64], 1),                      # decode, the first positions and a page edge
    (128, 32, 8, [1, 1, 1, 1], [300, 64, 63, 1000], 1),         # decode, ragged
    (128, 32, 8, [1, 1, 1, 1], [300, 64, 63, 1000], 4),         # the same with split keys
    (128, 40, 2, [1, 1], [500, 2], 3),                          # 20 query heads per kv head: two row chunks
    (256, 2, 1, [20, 1], [0, 77], 1),
    (80, 3, 1, [1], [129], 2),
    (128, 16, 2, [1, 1, 1], [900, 3, 450], 8),                  # eight splits, some of them empty for short sequences
    (128, 32, 8, [1, 1], [1500, 64], 12),                       # more than a cluster holds: global partials
    (128, 8, 2, [1, 1], [5000, 4095], 32),                      # long contexts, the most splits the engine uses
]


@pytest.mark.parametrize("d,nq,nkv,lengths,past,splits", MMA_CASES)
def test_attention_mma(d, nq, nkv, lengths, past, splits):
    torch.manual_seed(12)
    setup = paged_setup(lengths, past, nkv, d, "bfloat16", seed=13)
    n = sum(lengths)
    q = torch.randn(n, nq, d)
    scale = 1.0 / math.sqrt(d)
    out = torch.empty(n, nq * d, dtype=torch.bfloat16, device=DEV)
    decode = max(lengths) == 1
    splits = splits if decode else 1
    partial = torch.empty(n * nq * splits * (d + 2), dtype=torch.float32, device=DEV) if splits > 1 else None
    ops.attention_mma(q.bfloat16().to(DEV), setup["k_pool"], setup["v_pool"], out, setup["cu_q"], setup["past"],
                      setup["page_start"], setup["page_ids"], n_seqs=len(lengths), max_q_len=max(lengths), nq=nq,
                      nkv=nkv, d=d, page_size=64, scale=scale, splits=splits, partial=partial)
    expected = plain_attention(q, setup["dense"], lengths, past, nq, nkv, d, 0, scale, "bfloat16")
    close(out, expected, "bfloat16")
    if splits > 1:
        # merged by a second kernel instead of by the block that comes last: the same bits, and launched
        # again the tickets must have been left at zero
        for merge_in_kernel in (False, True):
            other = torch.zeros_like(out)
            ops.attention_mma(q.bfloat16().to(DEV), setup["k_pool"], setup["v_pool"], other, setup["cu_q"], setup["past"],
                              setup["page_start"], setup["page_ids"], n_seqs=len(lengths), max_q_len=1, nq=nq, nkv=nkv,
                              d=d, page_size=64, scale=scale, splits=splits, partial=partial,
                              merge_in_kernel=merge_in_kernel)
            assert torch.equal(other, out)
    if 1 < splits <= 8:
        # the same splits merged inside a thread-block cluster instead of through global partials
        other = torch.empty_like(out)
        ops.attention_mma(q.bfloat16().to(DEV), setup["k_pool"], setup["v_pool"], other, setup["cu_q"], setup["past"],
                          setup["page_start"], setup["page_ids"], n_seqs=len(lengths), max_q_len=1, nq=nq, nkv=nkv,
                          d=d, page_size=64, scale=scale, splits=splits, cluster=True)
        close(other, expected, "bfloat16")
        assert float((other.float() - out.float()).abs().max()) <= 2e-2


def test_attention_mma_finds_one_far_key():
    """One key among a thousand carries the answer (decode form with and without splits,
    prefill form at the last row of a long prompt)."""
    d, nq, nkv = 128, 8, 2
    lengths, past = [1, 1], [1000, 190]
    setup = paged_setup(lengths, past, nkv, d, "bfloat16", seed=14)
    q = torch.randn(2, nq, d) * 0.1
    targets = {0: 3, 1: 127}
    for tok, key in targets.items():
        k = setup["dense"][tok][0]
        q[tok] = torch.nn.functional.normalize(k[:, key], dim=-1).repeat_interleave(nq // nkv, 0) * 40.0
    scale = 1.0 / math.sqrt(d)
    for splits in (1, 6):
        out = torch.empty(2, nq * d, dtype=torch.bfloat16, device=DEV)
        partial = torch.empty(2 * nq * splits * (d + 2), dtype=torch.float32, device=DEV) if splits > 1 else None
        ops.attention_mma(q.bfloat16().to(DEV), setup["k_pool"], setup["v_pool"], out, setup["cu_q"], setup["past"],
                          setup["page_start"], setup["page_ids"], n_seqs=2, max_q_len=1, nq=nq, nkv=nkv, d=d,
                          page_size=64, scale=scale, splits=splits, partial=partial)
        for tok, key in targets.items():
            value = setup["dense"][tok][1][:, key].bfloat16().float().repeat_interleave(nq // nkv, 0).reshape(-1)
            assert float((out[tok].float().cpu() - value).abs().max()) < 0.05, (splits, tok)
    # prefill form: 700 tokens, the last query must find key 5
    setup = paged_setup([700], [0], nkv, d, "bfloat16", seed=15)
    q = torch.randn(700, nq, d) * 0.1
    k, v = setup["dense"][0]
    q[699] = torch.nn.functional.normalize(k[:, 5], dim=-1).repeat_interleave(nq // nkv, 0) * 40.0
    out = torch.empty(700, nq * d, dtype=torch.bfloat16, device=DEV)
    ops.attention_mma(q.bfloat16().to(DEV), setup["k_pool"], setup["v_pool"], out, setup["cu_q"], setup["past"],
                      setup["page_start"], setup["page_ids"], n_seqs=1, max_q_len=700, nq=nq, nkv=nkv, d=d,
                      page_size=64, scale=scale)
    value = v[:, 5].bfloat16().float().repeat_interleave(nq // nkv, 0).reshape(-1)
    assert float((out[699].float().cpu() - value).abs().max()) < 0.05
    expected = plain_attention(q, setup["dense"], [700], [0], nq, nkv, d, 0, scale, "bfloat16")
    close(out, expected, "bfloat16")


@pytest.mark.parametrize("wanted", [None, 1, 2, 5, 1000])
def test_attention_mma_blocks_of_equal_size(wanted):
    """Decode over unequal sequences with every block taking the same number of 64-key tiles: a long
    sequence uses more of its splits than a short one.  One far key carries each answer, so a block that
    was left out shows.  The number on the device may be anything (too small for the bound on the splits,
    or larger than every sequence): the sequences are covered all the same."""
    d, nq, nkv = 128, 8, 2
    lengths, past = [1, 1, 1, 1], [1300, 10, 64, 700]
    keys = {0: 1290, 1: 2, 2: 64, 3: 5}
    setup = paged_setup(lengths, past, nkv, d, "bfloat16", seed=24)
    q = torch.randn(4, nq, d) * 0.1
    for tok, key in keys.items():
        q[tok] = torch.nn.functional.normalize(setup["dense"][tok][0][:, key], dim=-1).repeat_interleave(nq // nkv, 0) * 40.0
    scale = 1.0 / math.sqrt(d)
    per, splits = ops.plan_key_splits([p + 1 for p in past], nkv, blocks=16, max_splits=8)
    assert per * splits >= 21 and splits > 1
    number = per if wanted is None else wanted
    out = torch.empty(4, nq * d, dtype=torch.bfloat16, device=DEV)
    partial = torch.full((4 * nq * splits * (d + 2),), float("nan"), dtype=torch.float32, device=DEV)
    ops.attention_mma(q.bfloat16().to(DEV), setup["k_pool"], setup["v_pool"], out, setup["cu_q"], setup["past"],
                      setup["page_start"], setup["page_ids"], n_seqs=4, max_q_len=1, nq=nq, nkv=nkv, d=d,
                      page_size=64, scale=scale, splits=splits, partial=partial,
                      tiles_per_split=torch.tensor([number], dtype=torch.int32, device=DEV))
    for tok, key in keys.items():
        value = setup["dense"][tok][1][:, key].bfloat16().float().repeat_interleave(nq // nkv, 0).reshape(-1)
        assert float((out[tok].float().cpu() - value).abs().max()) < 0.05, tok
    expected = plain_attention(q, setup["dense"], lengths, past, nq, nkv, d, 0, scale, "bfloat16")
    close(out, expected, "bfloat16")
    with pytest.raises(ops.KernelError):
        ops.attention_mma(q.bfloat16().to(DEV), setup["k_pool"], setup["v_pool"], out, setup["cu_q"], setup["past"],
                          setup["page_start"], setup["page_ids"], n_seqs=4, max_q_len=1, nq=nq, nkv=nkv, d=d,
                          page_size=64, scale=scale, splits=4, cluster=True,
                          tiles_per_split=torch.tensor([2], dtype=torch.int32, device=DEV))


@pytest.mark.parametrize("d", [128, 64, 48])
def test_attention_mma_with_the_hosts_list_of_blocks(d):
    """The same decode with the host's list of (sequence, split) blocks instead of one block per sequence and
    split: the same bits, whatever the order of the list and however much longer than the list the grid is; and
    a list made for shorter sequences than the device holds is reported, not computed with."""
    nq, nkv = 8, 2
    lengths, past = [1, 1, 1, 1, 1], [1300, 10, 64, 700, 2100]
    kv_lens = [p + 1 for p in past]
    setup = paged_setup(lengths, past, nkv, d, "bfloat16", seed=25)
    q = (torch.randn(5, nq, d) * 0.3).bfloat16().to(DEV)
    scale = 1.0 / math.sqrt(d)
    per, splits = ops.plan_key_splits(kv_lens, nkv, blocks=24, max_splits=8)
    assert splits > 2

    def run(plan):
        out = torch.empty(5, nq * d, dtype=torch.bfloat16, device=DEV)
        partial = torch.full((5 * nq * splits * (d + 2),), float("nan"), dtype=torch.float32, device=DEV)
        ops.attention_mma(q, setup["k_pool"], setup["v_pool"], out, setup["cu_q"], setup["past"], setup["page_start"],
                          setup["page_ids"], n_seqs=5, max_q_len=1, nq=nq, nkv=nkv, d=d, page_size=64, scale=scale,
                          splits=splits, partial=partial, tiles_per_split=torch.tensor(plan, dtype=torch.int32, device=DEV))
        return out

    one_number = run([per])
    blocks = ops.key_split_list(kv_lens, per, 40)
    count = blocks[1]
    assert count == sum(-(-(-(-n // 64)) // per) for n in kv_lens) and len(blocks) == 42
    assert blocks[2] >> 8 in (0, 4) and blocks[2] & 128 == 0        # a full block of a long sequence comes first
    assert torch.equal(run(blocks), one_number)
    assert torch.equal(run(blocks[:2 + count]), one_number)                          # a grid exactly as long as the list
    assert torch.equal(run(blocks[:2] + blocks[2:2 + count][::-1] + [0] * 7), one_number)    # any order
    expected = plain_attention(q.float().cpu(), setup["dense"], lengths, past, nq, nkv, d, 0, scale, "bfloat16")
    close(one_number, expected, "bfloat16")
    torch.cuda.synchronize()
    ops.raise_on_kernel_fault()
    stale = ops.key_split_list([n - 64 * per if n > 64 * per else n for n in kv_lens], per, 40)
    assert stale[1] < count
    run(stale)
    with pytest.raises(ops.KernelError, match="list of key blocks"):
        ops.raise_on_kernel_fault()
    ops.raise_on_kernel_fault()                                                      # the word is clear again
    with pytest.raises(ops.KernelError):
        ops.key_split_list(kv_lens, per, count - 1)
    with pytest.raises(ops.KernelError):
        run([per, 0])


MERGE_CASES = [
    # tokens, heads, head size, splits, output features, with a plan, bias
    (8, 32, 128, 4, 4096, True, False),        # the output projection of a decode step: clusters of 8 K splits
    (1, 32, 128, 16, 4096, True, False),       # one sequence, many splits
    (5, 6, 64, 3, 384, False, True),           # heads of 64, one K split, every token uses all splits, a bias
    (20, 8, 128, 2, 1024, True, False),        # a token tile of 32
    (16, 40, 128, 8, 5120, True, True),        # a width that is no power of two: 40 heads
    (3, 4, 192, 32, 768, True, False),         # heads of 192 (three k-blocks each), the most splits
]


@pytest.mark.parametrize("tokens,heads,d,splits,n_out,planned,biased", MERGE_CASES)
def test_gemm_bf16_merges_attention_splits_like_the_combine_kernel(tokens, heads, d, splits, n_out, planned, biased):
    """The output projection fed with the unmerged splits of a decode attention against the combine kernel
    followed by the same product: the same bits (the prologue rounds what the combine kernel would have
    rounded), with splits that have no keys (maximum -inf, garbage values) and, with a plan, tokens that use
    fewer splits than the bound; the sums of squares it leaves are the same too."""
    gen = torch.Generator().manual_seed(tokens * 131 + splits)
    K = heads * d
    assert ops.gemm_bf16_fuses_merge(tokens, n_out, K, splits=splits, nq=heads, d=d)
    partial = torch.randn(tokens, heads, splits, d + 2, generator=gen)
    partial[..., d] = torch.randn(tokens, heads, splits, generator=gen) * 3.0           # maxima
    partial[..., d + 1] = torch.rand(tokens, heads, splits, generator=gen) * 50 + 0.5   # sums
    empty = torch.rand(tokens, heads, splits, generator=gen) < 0.15
    empty[..., 0] = False
    partial[..., d][empty] = float("-inf")
    partial[..., :d][empty] = float("nan")                  # whatever an empty split holds must not matter
    plan, past = None, torch.randint(0, 64 * splits * 3, (tokens,), generator=gen, dtype=torch.int32)
    if planned:
        plan = torch.tensor([3, 0, 0], dtype=torch.int32, device=DEV)          # 3 tiles a split (a list's first number)
        past[0] = 64 * 3 * splits - 1                                          # one token uses every split
        if tokens > 1:
            past[1] = 5                                                        # and one a single split
    partial, past = partial.to(DEV), past.to(DEV)
    w = (torch.randn(n_out, K, generator=gen) / math.sqrt(K)).bfloat16().to(DEV)
    bias = torch.randn(n_out, generator=gen).to(DEV) if biased else None
    residual = torch.randn(tokens, n_out, generator=gen).to(DEV)

    merged = torch.empty(tokens, K, dtype=torch.bfloat16, device=DEV)
    ops.attention_mma_combine(partial, merged, past, nq=heads, d=d, splits=splits, tiles_per_split=plan)
    assert bool(torch.isfinite(merged.float()).all())
    expected, sums_expected = residual.clone(), torch.empty(ops.gemm_bf16_sumsq_parts(n_out), tokens, device=DEV)
    ops.gemm_bf16(merged, w, expected, ops.EPI_RESIDUAL, bias=bias, sumsq_out=sums_expected)
    got, sums = residual.clone(), torch.empty_like(sums_expected)
    ops.gemm_bf16(None, w, got, ops.EPI_RESIDUAL, bias=bias, sumsq_out=sums,
                  merge=(partial, past, plan, splits, heads, d))
    torch.cuda.synchronize()
    ops.raise_on_kernel_fault()
    assert torch.equal(got, expected)
    assert torch.equal(sums, sums_expected)
    # and against plain arithmetic: softmax-weighted sum of the used splits, then the product
    used = [splits if plan is None else -(-(int(p) // 64 + 1) // max(3, -(-(int(p) // 64 + 1) // splits))) for p in past.tolist()]
    ref = torch.zeros(tokens, K, dtype=torch.float64)
    host = partial.double().cpu()
    for t in range(tokens):
        m, l, acc = host[t, :, :used[t], d], host[t, :, :used[t], d + 1], host[t, :, :used[t], :d]
        wgt = torch.exp(m - m.max(-1, keepdim=True).values)
        acc = torch.where(torch.isfinite(m)[..., None], acc, torch.zeros_like(acc))
        ref[t] = ((wgt[..., None] * acc).sum(1) / (wgt * l).sum(-1, keepdim=True)).reshape(-1)
    product = ref.bfloat16().double() @ w.double().cpu().t() + (bias.double().cpu() if biased else 0.0)
    close(got, (residual.double().cpu() + product).float(), "bfloat16")


TC_ATTN_CASES = [
    # d, nq, nkv, lengths, past
    (128, 4, 2, [128], [0]),                      # exactly one tile of queries, two pages of keys
    (128, 8, 2, [200, 64, 65, 1], [0, 0, 0, 0]),  # whole prompts, page and tile edges
    (128, 4, 1, [40, 3, 130], [100, 200, 7]),     # chunks on a cache
    (64, 6, 3, [300, 17], [0, 50]),
    (128, 32, 8, [700], [0]),                     # many pages: every buffer and stage wraps several times
    (128, 4, 1, [900, 1], [2100, 3000]),          # a long chunk and a single token on long caches
    (128, 3, 1, [150, 70], [0, 10]),              # an odd group size: one head per CTA
    (64, 2, 2, [130], [5]),                       # no grouping
]


@pytest.mark.parametrize("d,nq,nkv,lengths,past", TC_ATTN_CASES)
def test_attention_tcgen05(d, nq, nkv, lengths, past):
    torch.manual_seed(16)
    setup = paged_setup(lengths, past, nkv, d, "bfloat16", seed=17)
    n = sum(lengths)
    q = torch.randn(n, nq, d)
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros(n, nq * d, dtype=torch.bfloat16, device=DEV)
    expected = plain_attention(q, setup["dense"], lengths, past, nq, nkv, d, 0, scale, "bfloat16")
    for heads_per_cta in (1, 2) if (nq // nkv) % 2 == 0 else (1,):
        out.zero_()
        ops.attention_tcgen05(q.bfloat16().to(DEV), setup["k_pool"], setup["v_pool"], out, setup["cu_q"],
                              setup["past"], setup["page_start"], setup["page_ids"], n_seqs=len(lengths),
                              max_q_len=max(lengths), nq=nq, nkv=nkv, d=d, page_size=64, scale=scale,
                              heads_per_cta=heads_per_cta)
        torch.cuda.synchronize()
        ops.raise_on_kernel_fault()
        close(out, expected, "bfloat16")


@pytest.mark.parametrize("heads_per_cta", (1, 2))
def test_attention_tcgen05_repeats_bit_for_bit(heads_per_cta):
    """More CTAs than SMs, so that CTAs share an SM and their warps drift apart: a wait that took
    one phase of a barrier for another showed as a few rows that changed from run to run."""
    d, nq, nkv, lengths, past = 128, 32, 8, [700], [0]
    torch.manual_seed(19)
    setup = paged_setup(lengths, past, nkv, d, "bfloat16", seed=20)
    q = torch.randn(700, nq, d).bfloat16().to(DEV)
    first = None
    for _ in range(60):
        out = torch.zeros(700, nq * d, dtype=torch.bfloat16, device=DEV)
        ops.attention_tcgen05(q, setup["k_pool"], setup["v_pool"], out, setup["cu_q"], setup["past"],
                              setup["page_start"], setup["page_ids"], n_seqs=1, max_q_len=700, nq=nq, nkv=nkv, d=d,
                              page_size=64, scale=1.0 / math.sqrt(d), heads_per_cta=heads_per_cta)
        torch.cuda.synchronize()
        if first is None:
            first = out
        assert torch.equal(out, first)
    ops.raise_on_kernel_fault()
    expected = plain_attention(q.float().cpu(), setup["dense"], lengths, past, nq, nkv, d, 0, 1.0 / math.sqrt(d), "bfloat16")
    close(first, expected, "bfloat16")


def test_attention_tcgen05_finds_one_far_key():
    d, nq, nkv = 128, 8, 2
    setup = paged_setup([700], [0], nkv, d, "bfloat16", seed=18)
    q = torch.randn(700, nq, d) * 0.1
    k, v = setup["dense"][0]
    q[699] = torch.nn.functional.normalize(k[:, 5], dim=-1).repeat_interleave(nq // nkv, 0) * 40.0
    q[130] = torch.nn.functional.normalize(k[:, 129], dim=-1).repeat_interleave(nq // nkv, 0) * 40.0
    scale = 1.0 / math.sqrt(d)
    out = torch.zeros(700, nq * d, dtype=torch.bfloat16, device=DEV)
    ops.attention_tcgen05(q.bfloat16().to(DEV), setup["k_pool"], setup["v_pool"], out, setup["cu_q"], setup["past"],
                          setup["page_start"], setup["page_ids"], n_seqs=1, max_q_len=700, nq=nq, nkv=nkv, d=d,
                          page_size=64, scale=scale)
    torch.cuda.synchronize()
    ops.raise_on_kernel_fault()
    for tok, key in ((699, 5), (130, 129)):
        value = v[:, key].bfloat16().float().repeat_interleave(nq // nkv, 0).reshape(-1)
        assert float((out[tok].float().cpu() - value).abs().max()) < 0.05, (tok, key)
    expected = plain_attention(q, setup["dense"], [700], [0], nq, nkv, d, 0, scale, "bfloat16")
    close(out, expected, "bfloat16")


PREFILL_GEMM_SHAPES = [
    # tokens, features, K: whole tiles, ragged edges in all three sizes, fewer tiles than clusters, many tiles per
    # cluster, more than one group of token tiles, an output width that the TMA store refuses
    (128, 256, 64), (2048, 4096, 4096), (300, 520, 200), (33, 1000, 1000), (1030, 1024, 512), (130, 6144, 72),
    (5000, 389, 96), (4500, 776, 136),
]
# the shapes of a 2,048-token prefill at Qwen3-8B and Qwen3-14B layer sizes: the down projection's long K with
# the reduce-add epilogue, the gate/up product's 2 x 12,288 features, a ragged token count at the long K
PREFILL_GEMM_MODEL_SHAPES = [
    (2048, 4096, 12288, "residual", False), (2048, 4096, 12288, "store_bf16", True),
    (2048, 12288, 4096, "swiglu", False), (2048, 5120, 17408, "residual", True),
    (1900, 4096, 12288, "residual", False), (2100, 6144, 4096, "store_bf16", True),
]


@pytest.mark.parametrize("tokens,N,K,epi,biased", PREFILL_GEMM_MODEL_SHAPES)
def test_gemm_prefill_tcgen05_at_model_sizes(tokens, N, K, epi, biased):
    test_gemm_prefill_tcgen05(tokens, N, K, epi, biased)


@pytest.mark.parametrize("biased", [False, True])
@pytest.mark.parametrize("epi", ["store_bf16", "store_f32", "residual", "swiglu"])
@pytest.mark.parametrize("tokens,N,K", PREFILL_GEMM_SHAPES)
def test_gemm_prefill_tcgen05(tokens, N, K, epi, biased):
    """The persistent product for many tokens and its four epilogues against fp32 torch on the same
    bf16 inputs; twice, so that a second launch finds the same result; with and without a bias."""
    code = {"store_bf16": ops.EPI_STORE_BF16, "store_f32": ops.EPI_STORE_F32, "residual": ops.EPI_RESIDUAL,
            "swiglu": ops.EPI_SWIGLU}[epi]
    torch.manual_seed(31)
    x = torch.randn(tokens, K).bfloat16().to(DEV)
    rows = 2 * N if epi == "swiglu" else N
    w = (torch.randn(rows, K) / math.sqrt(K)).bfloat16().to(DEV)
    bias = torch.randn(rows).to(DEV) if biased else None
    ref = (x.float() @ w.float().t()).cpu()
    if biased:
        ref = ref + bias.cpu()
    res = torch.randn(tokens, N)
    for _ in range(2):
        if epi == "store_bf16":
            out, expected = torch.zeros(tokens, N, dtype=torch.bfloat16, device=DEV), ref
        elif epi == "store_f32":
            out, expected = torch.zeros(tokens, N, dtype=torch.float32, device=DEV), ref
        elif epi == "residual":
            out, expected = res.clone().to(DEV), res + ref
        else:
            out = torch.zeros(tokens, N, dtype=torch.bfloat16, device=DEV)
            expected = torch.nn.functional.silu(ref[:, :N]) * ref[:, N:]
        if not ops.gemm_prefill_supported(x, w, N, out.dtype):
            with pytest.raises(ops.KernelError):        # rows of the output that do not start on 16 bytes are refused
                ops.gemm_prefill_bf16(x, w, out, code, bias=bias)
            return
        ops.gemm_prefill_bf16(x, w, out, code, bias=bias)
        torch.cuda.synchronize()
        ops.raise_on_kernel_fault()
        if out.dtype == torch.bfloat16:
            close(out, expected, "bfloat16")
        else:
            assert torch.allclose(out.cpu(), expected, atol=1e-4, rtol=1e-4), float((out.cpu() - expected).abs().max())


@pytest.mark.parametrize("lengths,past,K,nq,nkv,norm,rot,ring,biased", [
    ([300, 17, 2000], [0, 50, 0], 512, 4, 2, True, True, 0, False),          # unequal prompts, ragged token tiles
    ([300, 17, 2000], [0, 50, 0], 512, 4, 2, True, True, 0, True),
    ([700], [100], 1024, 6, 3, False, True, 0, True),                        # no norm
    ([256, 256], [0, 0], 256, 2, 1, True, False, 0, False),                  # no rotation, whole tiles
    ([130, 100], [400, 60], 768, 3, 1, True, True, 3, False),                # an odd number of heads, rings of three pages (no step wraps its ring)
])
def test_gemm_prefill_tcgen05_prepares_heads_in_its_epilogue(lengths, past, K, nq, nkv, norm, rot, ring, biased):
    """The q/k/v product of many tokens with the head preparation in its epilogue against the product followed
    by the head-preparation kernel: close (the two add the squares of a head in different orders), and nothing
    written elsewhere in the cache."""
    torch.manual_seed(41)
    d = 128
    setup = paged_setup(lengths, past, nkv, d, "bfloat16", ring_pages=ring, seed=42)
    n = sum(lengths)
    w = (torch.randn((nq + 2 * nkv) * d, K) / math.sqrt(K)).bfloat16().to(DEV)
    x = torch.randn(n, K).bfloat16().to(DEV)
    qw = (1 + 0.1 * torch.randn(d)).to(DEV) if norm else None
    kw = (1 + 0.1 * torch.randn(d)).to(DEV) if norm else None
    cos = sin = None
    if rot:
        inv_freq = 1.0 / (10000.0 ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
        cos = torch.empty(n, d // 2, dtype=torch.float32, device=DEV)
        sin = torch.empty_like(cos)
        ops.rope_table(inv_freq.to(DEV), setup["tok_pos"], cos, sin)
    common = dict(nq=nq, nkv=nkv, d=d, rot_dim=d if rot else 0, page_size=64, ring_pages=ring, write_kv=True, eps=1e-5)
    tail = (qw, kw, cos, sin, setup["tok_seq"], setup["tok_pos"], setup["page_start"], setup["page_ids"])
    bias = torch.randn(w.shape[0]).to(DEV) if biased else None
    qkv = torch.empty(n, w.shape[0], dtype=torch.bfloat16, device=DEV)
    ops.gemm_prefill_bf16(x, w, qkv, ops.EPI_STORE_BF16, bias=bias)
    if biased:
        plain_qkv = x.float() @ w.float().t() + bias
        assert float((qkv.float() - plain_qkv).abs().max()) <= 0.02 * float(plain_qkv.abs().max())
    q_two = torch.zeros(n, nq * d, dtype=torch.bfloat16, device=DEV)
    k_two, v_two = torch.zeros_like(setup["k_pool"]), torch.zeros_like(setup["v_pool"])
    ops.head_prep(qkv, q_two, k_two, v_two, *tail, **common)
    q_one = torch.zeros_like(q_two)
    k_one, v_one = torch.zeros_like(k_two), torch.zeros_like(v_two)
    block = ops.head_prep(None, q_one, k_one, v_one, *tail, **common)
    ops.gemm_prefill_bf16(x, w, None, ops.EPI_HEAD_PREP, head_prep=block, bias=bias)
    torch.cuda.synchronize()
    ops.raise_on_kernel_fault()
    assert torch.equal(v_one, v_two)
    for one, two in ((q_one, q_two), (k_one, k_two)):
        assert float(two.float().abs().sum()) > 0
        assert torch.equal(one == 0, two == 0) or float(((one == 0) != (two == 0)).float().mean()) < 1e-4
        differ = (one.float() - two.float()).abs()
        assert float(differ.max()) <= 0.02 * float(two.float().abs().max()) and float((differ > 0).float().mean()) < 0.02


def test_a_wait_that_runs_out_is_reported_and_leaves_the_gpu_usable():
    """Every barrier wait of the tensor-core kernels is bounded.  Here one runs out for real, safely: one tile of
    a build whose waits last about ten milliseconds, with a producer that requests no copy (nothing is in
    flight).  The MMA role gives up, the kernel frees its tensor memory and returns, the error word names that
    role, the host check raises once, and the next product on the same device is right."""
    ops.raise_on_kernel_fault()                      # start from a clean word
    code = ops.selftest_bounded_wait(DEV)
    assert code == 2, f"the MMA role's wait should have run out first (code 2), the word holds {code}"
    with pytest.raises(ops.KernelError, match="gemm_tcgen05: the MMA issuer"):
        ops.raise_on_kernel_fault()
    ops.raise_on_kernel_fault()                      # reported once
    torch.manual_seed(50)
    x = torch.randn(8, 512).bfloat16().to(DEV)
    w = (torch.randn(256, 512) / math.sqrt(512)).bfloat16().to(DEV)
    out = torch.empty(8, 256, dtype=torch.float32, device=DEV)
    ops.gemm_bf16(x, w, out, ops.EPI_STORE_F32)
    torch.cuda.synchronize()
    ops.raise_on_kernel_fault()
    assert torch.allclose(out.cpu(), (x.float() @ w.float().t()).cpu(), atol=1e-4, rtol=1e-4)


@pytest.mark.parametrize("tokens,N,K", [(2048, 4096, 4096), (2048, 4096, 12288), (5000, 1024, 136), (2100, 5120, 1000),
                                        (4500, 776, 72), (19000, 256, 64)])
def test_gemm_prefill_tcgen05_adds_a_tile_in_ordered_parts(tokens, N, K):
    """The residual product with every tile's k-blocks cut into parts that different CTA pairs add one after the
    other: the same result as whole tiles up to fp32 rounding, against fp32 torch, and the same bits every time
    (the order of a tile's adds is fixed); the counters are left zero."""
    torch.manual_seed(61)
    x = torch.randn(tokens, K).bfloat16().to(DEV)
    w = (torch.randn(N, K) / math.sqrt(K)).bfloat16().to(DEV)
    res = torch.randn(tokens, N)
    expected = res + (x.float() @ w.float().t()).cpu()
    outs = []
    bias = torch.randn(N).to(DEV)
    expected = expected + bias.cpu()
    for balance in (0, 4, 4, 1, 2, 3):
        out = res.clone().to(DEV)
        ops.gemm_prefill_bf16(x, w, out, ops.EPI_RESIDUAL, balance=balance, bias=bias)
        torch.cuda.synchronize()
        ops.raise_on_kernel_fault()
        assert torch.allclose(out.cpu(), expected, atol=1e-4, rtol=1e-4), (balance, float((out.cpu() - expected).abs().max()))
        outs.append(out)
    assert torch.equal(outs[1], outs[2]), "two runs in four parts differ: the order of a tile's adds is not fixed"
    assert float((outs[0] - outs[1]).abs().max()) <= 2e-5 * math.sqrt(K)
    _, tickets, _ = ops._gemm_buffers(torch.device(DEV), 0)
    assert int(tickets.abs().sum()) == 0, "a flag or ticket was left set"
