"""Each CUDA kernel alone against a plain float32 torch restatement of the same operation,
at sizes that differ from the engine's test configurations (widths and vocabularies that are
no power of two, odd head counts, page sizes 8/16/32)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def dev():
    return torch.device("cuda:0")


def rnd(shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(dev())


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    from dispec_b200 import ops
    table = rnd((301, 88), dtype, 1)
    ids = torch.tensor([0, 300, 5, 5, 17], dtype=torch.int32, device=dev())
    out = ops.embed(table, ids)
    assert torch.equal(out, table[ids.long()])
    table2 = rnd((50, 33), dtype, 2)  # row bytes not a multiple of 16
    out2 = ops.embed(table2, ids[:1] * 0 + 49)
    assert torch.equal(out2, table2[49:50])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hidden", [96, 1536, 200])
def test_rms_norm(dtype, hidden):
    from dispec_b200 import ops
    x = rnd((7, hidden), dtype, 3, 2.0)
    w = (1 + rnd((hidden,), torch.float32, 4, 0.1)).to(dtype)
    eps = 1e-5
    y = ops.rms_norm(x, w, eps)
    xf = x.float()
    n = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(dtype).float()
    ref = (w.float() * n).to(dtype)
    torch.testing.assert_close(y.float(), ref.float(), **tol(dtype))
    # fused residual sum, written back
    d = rnd((7, hidden), dtype, 5)
    x2 = x.clone()
    y2 = ops.rms_norm(x2, w, eps, delta=d, write_back=True)
    s = (x.float() + d.float()).to(dtype)
    assert torch.equal(x2, s)
    sf = s.float()
    n2 = (sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + eps)).to(dtype).float()
    torch.testing.assert_close(y2.float(), (w.float() * n2).to(dtype).float(), **tol(dtype))
    # gathered rows, nothing written back
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=dev())
    x3 = x.clone()
    y3 = ops.rms_norm(x3, w, eps, delta=d, rows=rows)
    assert torch.equal(x3, x)
    torch.testing.assert_close(y3.float(), y2[rows.long()].float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden", [(515, 1536), (700, 200), (513, 3584), (512, 1000), (600, 5120), (1029, 72)])
def test_rms_norm_of_many_rows(dtype, rows, hidden):
    """Hundreds of rows, as in a portion of a prompt, at widths of every kernel form (vectors that
    fit a CTA's registers, wider ones, widths that are no multiple of a vector): the same checks as
    for a few rows, and row for row the result of the same rows taken a hundred at a time."""
    from dispec_b200 import ops
    x = rnd((rows, hidden), dtype, 13, 2.0)
    w = (1 + rnd((hidden,), torch.float32, 14, 0.1)).to(dtype)
    eps = 1e-6
    y = ops.rms_norm(x, w, eps)
    xf = x.float()
    n = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(dtype).float()
    torch.testing.assert_close(y.float(), (w.float() * n).to(dtype).float(), **tol(dtype))
    few = torch.cat([ops.rms_norm(x[i:i + 100].contiguous(), w, eps) for i in range(0, rows, 100)])
    torch.testing.assert_close(y.float(), few.float(), **tol(dtype))
    d = rnd((rows, hidden), dtype, 15)
    x2 = x.clone()
    y2 = ops.rms_norm(x2, w, eps, delta=d, write_back=True)
    s = (x.float() + d.float()).to(dtype)
    assert torch.equal(x2, s)
    sf = s.float()
    n2 = (sf * torch.rsqrt(sf.pow(2).mean(-1, keepdim=True) + eps)).to(dtype).float()
    torch.testing.assert_close(y2.float(), (w.float() * n2).to(dtype).float(), **tol(dtype))
    picked = torch.randperm(rows, generator=torch.Generator().manual_seed(3))[:rows - 3].to(torch.int32).to(dev())
    x3 = x.clone()
    y3 = ops.rms_norm(x3, w, eps, delta=d, rows=picked)
    assert torch.equal(x3, x)
    torch.testing.assert_close(y3.float(), y2[picked.long()].float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_swiglu(dtype):
    from dispec_b200 import ops
    gu = rnd((5, 2 * 224), dtype, 6, 3.0)
    out = ops.swiglu(gu)
    g, u = gu[:, :224].float(), gu[:, 224:].float()
    ref = (g * torch.sigmoid(g) * u).to(dtype)
    torch.testing.assert_close(out.float(), ref.float(), **tol(dtype))
    # gates and ups alternating in blocks of 16 columns
    inter = gu.view(5, 2, 14, 16).permute(0, 2, 1, 3).reshape(5, 448).contiguous()
    torch.testing.assert_close(ops.swiglu(inter, block=16).float(), ref.float(), **tol(dtype))
    odd = rnd((3, 2 * 50), dtype, 7)  # a width the 16-byte path does not take
    g, u = odd[:, :50].float(), odd[:, 50:].float()
    torch.testing.assert_close(ops.swiglu(odd).float(), (g * torch.sigmoid(g) * u).to(dtype).float(), **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 100, 96), (5, 130, 224), (70, 257, 40), (33, 64, 1536)])
def test_gemm_fma(dtype, M, N, K):
    from dispec_b200.ops import gemm
    x = rnd((M, K), dtype, 7)
    w = rnd((N, K), dtype, 8, 0.1)
    b = rnd((N,), dtype, 9)
    r = rnd((M, N), dtype, 10)
    out = gemm.linear(x, w, b, r, backend="simt")
    ref = (x.double() @ w.double().T + b.double() + r.double())
    torch.testing.assert_close(out.double(), ref, **tol(dtype))
    out32 = gemm.linear(x, w, out_dtype=torch.float32, backend="simt")
    torch.testing.assert_close(out32.double(), x.double() @ w.double().T, atol=1e-4, rtol=1e-4)


def test_gemm_fma_rows_do_not_depend_on_batch():
    from dispec_b200.ops import gemm
    x = rnd((37, 200), torch.float32, 11)
    w = rnd((77, 200), torch.float32, 12)
    full = gemm.linear(x, w)
    one = gemm.linear(x[20:21].contiguous(), w)
    assert torch.equal(full[20:21], one)


def _rope_reference(x, pos, theta, rotary_dim):
    half = rotary_dim // 2
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
    ang = pos.float()[:, None] * inv[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., :half], x[..., half:rotary_dim]
    out[..., :half] = a * c - b * s
    out[..., half:rotary_dim] = b * c + a * s
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KVH,D,rot,page", [(3, 1, 32, 32, 8), (6, 2, 48, 48, 16), (4, 4, 16, 8, 32)])
def test_rope_kv_store(dtype, H, KVH, D, rot, page):
    from dispec_b200 import ops
    T, num_pages = 9, 7
    theta = 50000.0
    qkv = rnd((T, (H + 2 * KVH) * D), dtype, 13)
    # two sequences: seq 0 holds positions 14..18 (crosses a page edge), seq 1 positions 0..3
    pos = torch.tensor([14, 15, 16, 17, 18, 0, 1, 2, 3], dtype=torch.int32)
    seq = torch.tensor([0] * 5 + [1] * 4, dtype=torch.int32)
    table = torch.tensor([[5, 2, 6, 0], [3, -1, -1, -1]], dtype=torch.int32)
    kp = torch.full((num_pages, KVH, page, D), float("nan"), dtype=dtype, device=dev())
    vp = kp.clone()
    inv = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(dev())
    q0 = qkv.clone()
    ops.rope_kv_store(qkv, pos.to(dev()), seq.to(dev()), table.to(dev()), kp, vp, inv, H, KVH, D, rot)
    x = q0.float().cpu().view(T, H + 2 * KVH, D)
    ref_qk = _rope_reference(x[:, :H + KVH], pos, theta, rot)
    got = qkv.float().cpu().view(T, H + 2 * KVH, D)
    torch.testing.assert_close(got[:, :H + KVH], ref_qk.to(dtype).float(), **tol(dtype))
    assert torch.equal(got[:, H + KVH:], x[:, H + KVH:])
    for t in range(T):
        p, s = int(pos[t]), int(seq[t])
        pg = int(table[s, p // page])
        torch.testing.assert_close(kp[pg, :, p % page].float().cpu(), got[t, H:H + KVH], atol=0, rtol=0)
        torch.testing.assert_close(vp[pg, :, p % page].float().cpu(), got[t, H + KVH:], atol=0, rtol=0)
    # nothing else was touched
    written = torch.zeros((num_pages, page), dtype=torch.bool)
    for t in range(T):
        written[int(table[int(seq[t]), int(pos[t]) // page]), int(pos[t]) % page] = True
    assert torch.isnan(kp.float().cpu().permute(0, 2, 1, 3)[~written]).all()


def _attention_reference(q, k, v, positions, window, scale):
    """q [T,H,D] (T tokens of one sequence at ``positions``), k/v [ctx,KVH,D] in float64."""
    T, H, D = q.shape
    G = H // k.shape[1]
    out = torch.zeros(T, H, D, dtype=torch.float64)
    for t in range(T):
        p = int(positions[t])
        lo = max(0, p - window + 1) if window > 0 else 0
        for h in range(H):
            s = (k[lo:p + 1, h // G] @ q[t, h]) * scale
            out[t, h] = torch.softmax(s, 0) @ v[lo:p + 1, h // G]
    return out


def _paged(k, v, page, num_pages, dtype, seed, order="shuffled"):
    """Scatter contiguous k/v [ctx,KVH,D] into pools through a page table: shuffled; "ascending"
    (consecutive pages up to the pool's last one); or "runs": consecutive stretches of changing
    length, with breaks inside key tiles, a descending stretch and the pool's last page in use."""
    ctx, KVH, D = k.shape
    n = (ctx + page - 1) // page
    g = torch.Generator().manual_seed(seed)
    if order == "shuffled":
        perm = torch.randperm(num_pages, generator=g)[:n]
    elif order == "ascending":
        perm = torch.arange(num_pages - n, num_pages)
    else:
        assert order == "runs"
        free, perm, length = list(range(num_pages)), [], 1
        while len(perm) < n:  # stretches of 1, 2, ... 9, 1, ... pages taken from both ends in turn
            take = min(length, n - len(perm))
            if (length // 3) % 2 == 0:
                perm += free[-take:]
                del free[-take:]
            else:
                perm += free[:take]
                del free[:take]
            if length == 5:
                perm[-take:] = reversed(perm[-take:])
            length = length % 9 + 1
        perm = torch.tensor(perm)
    kp = torch.full((num_pages, KVH, page, D), float("nan"), dtype=dtype)
    vp = kp.clone()
    for b in range(ctx):
        kp[perm[b // page], :, b % page] = k[b].to(dtype)
        vp[perm[b // page], :, b % page] = v[b].to(dtype)
    return kp.to(dev()), vp.to(dev()), perm.to(torch.int32)


ATTN_CASES = [
    # H, KVH, D, page, ctx, q_len, window
    (4, 2, 16, 16, 33, 33, 0),
    (3, 1, 32, 8, 70, 5, 0),
    (6, 2, 48, 16, 300, 1, 0),
    (12, 2, 128, 16, 257, 17, 0),
    (4, 2, 16, 8, 90, 90, 12),
    (6, 2, 32, 16, 200, 3, 40),
    (9, 1, 64, 32, 140, 1, 64),
]


def run_attention(kind, dtype, H, KVH, D, page, ctx, q_len, window, plant=None, seed=0, prefill_kernel=None,
                  page_order="shuffled"):
    """One sequence, its last q_len positions as queries.  ``plant``: key index whose score is
    made to stand out for every query that can see it."""
    from dispec_b200.ops import attention as A
    g = torch.Generator().manual_seed(100 + seed)
    q = torch.randn(q_len, H, D, generator=g)
    k = torch.randn(ctx, KVH, D, generator=g)
    v = torch.randn(ctx, KVH, D, generator=g)
    if plant is not None:
        G = H // KVH
        for kvh in range(KVH):
            direction = q[:, kvh * G:(kvh + 1) * G].mean(dim=(0, 1))
            q[:, kvh * G:(kvh + 1) * G] += 3.0 * direction / direction.norm()
            k[plant, kvh] = 12.0 * direction / direction.norm()
    q, k, v = q.to(dtype).float(), k.to(dtype).float(), v.to(dtype).float()
    positions = torch.arange(ctx - q_len, ctx, dtype=torch.int32)
    scale = D ** -0.5
    ref = _attention_reference(q.double(), k.double(), v.double(), positions, window, scale)
    num_pages = (ctx + page - 1) // page + 3
    kp, vp, perm = _paged(k, v, page, num_pages, dtype, seed, page_order)
    table = perm.view(1, -1).to(dev())
    qd = q.to(dtype).reshape(q_len, H * D).to(dev())
    out = torch.empty((q_len, H * D), dtype=dtype, device=dev())
    seq = torch.zeros(q_len, dtype=torch.int32, device=dev())
    if kind == "generic":
        A.paged_attention_generic(qd, H * D, kp, vp, table, positions.to(dev()), seq, out, H, KVH, D,
                                  window, scale)
    else:
        A.paged_attention_tensor_core(qd, H * D, kp, vp, table, positions.to(dev()), seq, out, H, KVH,
                                      D, window, scale, q_lens=[q_len], ctx_lens=[ctx],
                                      prefill_kernel=prefill_kernel)
    return out.float().cpu().view(q_len, H, D).double(), ref


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ATTN_CASES)
def test_attention_generic(dtype, case):
    out, ref = run_attention("generic", dtype, *case)
    torch.testing.assert_close(out, ref, **(dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32
                                           else dict(atol=2e-2, rtol=2e-2)))


@pytest.mark.parametrize("plant", [0, 7, 8, 15, 16, 17, 127, 128, 255, 256])
def test_attention_generic_far_key_stands_out(plant):
    # one key among hundreds carries the result: a skipped or misplaced key (page edge, tile edge)
    # changes the output completely
    out, ref = run_attention("generic", torch.float32, 4, 2, 32, 16, 300, 2, 0, plant=plant, seed=plant)
    torch.testing.assert_close(out, ref, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("offset", [-1, 0, 1])
def test_attention_generic_window_edge(offset):
    # the planted key sits just outside (offset -1), on (0) and just inside (+1) the window's far
    # edge of the last query
    ctx, window = 150, 40
    plant = ctx - 1 - window + 1 + offset
    out, ref = run_attention("generic", torch.float32, 4, 2, 32, 16, ctx, 1, window, plant=plant, seed=5)
    torch.testing.assert_close(out, ref, atol=1e-5, rtol=1e-5)


def test_argmax_ties_go_to_the_lowest_index():
    from dispec_b200 import ops
    x = torch.randn(5, 1000, generator=torch.Generator().manual_seed(1))
    x[0, 700] = x[0, 20] = 9.0
    x[1, 999] = 10.0
    x[2, 0] = 10.0
    got = ops.argmax(x.to(dev())).cpu()
    assert got.tolist() == [20, 999, 0, int(x[3].argmax()), int(x[4].argmax())]
    # a large vocabulary that is no power of two
    y = torch.randn(3, 151937, generator=torch.Generator().manual_seed(2))
    assert ops.argmax(y.to(dev())).cpu().tolist() == y.argmax(-1).tolist()


def test_sampling_matches_plain_inverse_cdf():
    import plain_qwen2 as plain
    from dispec_b200 import ops
    V = 1003
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(8, V, generator=g) * 3
    cases = [(0.8, 0, 1.0), (1.3, 10, 1.0), (0.7, 0, 0.9), (1.0, 50, 0.5), (0.0, 0, 1.0),
             (2.0, 1, 1.0), (0.5, 0, 0.01), (1.0, 2000, 0.999)]
    us = [0.03, 0.5, 0.77, 0.999, 0.4, 0.6, 0.9, 0.25]
    t = torch.tensor([c[0] for c in cases], dtype=torch.float32, device=dev())
    k = torch.tensor([c[1] for c in cases], dtype=torch.int32, device=dev())
    p = torch.tensor([c[2] for c in cases], dtype=torch.float32, device=dev())
    u = torch.tensor(us, dtype=torch.float32, device=dev())
    got = ops.sample(logits.to(dev()), t, k, p, u).cpu().tolist()
    for r, (temp, tk, tp) in enumerate(cases):
        probs = plain.sampling_distribution(logits[r], temp, tk, tp)
        want = plain.draw_inverse_cdf(probs, us[r]) if temp > 0 else int(logits[r].argmax())
        assert probs[got[r]] > 0, (r, got[r])
        assert got[r] == want, (r, got[r], want)


@pytest.mark.parametrize("V", [151936, 152064])
def test_sampling_at_the_real_vocabulary_sizes(V):
    """The radix selection and the fixed-point mass of the sampling kernel at the vocabularies the
    benchmark shapes have, against the plain inverse CDF in float64: the cases of the small test,
    top-p at 0.999 over a flat tail behind a few heavy tokens, and top-k with thousands of ties."""
    import plain_qwen2 as plain
    from dispec_b200 import ops
    g = torch.Generator().manual_seed(V)
    cases = [(0.8, 0, 1.0), (1.3, 10, 1.0), (0.7, 0, 0.9), (1.0, 50, 0.5), (0.0, 0, 1.0),
             (2.0, 1, 1.0), (0.5, 0, 0.01), (1.0, 2000, 0.999), (1.0, 0, 0.999), (1.0, 0, 0.999), (1.5, 100, 1.0)]
    us = [0.03, 0.5, 0.77, 0.999, 0.4, 0.6, 0.9, 0.25, 0.9985, 0.31, 0.62]
    logits = torch.randn(len(cases), V, generator=g) * 3
    flat = torch.zeros(V)  # a flat tail (every token the same) behind three heavy tokens
    flat[[5, V // 2, V - 1]] = torch.tensor([14.0, 13.5, 13.0])
    logits[8] = logits[9] = flat
    ties = torch.full((V,), -2.0)  # 5,000 tokens tie at the top: top_k = 100 keeps all of them
    ties[torch.randperm(V, generator=g)[:5000]] = 1.0
    logits[10] = ties
    t = torch.tensor([c[0] for c in cases], dtype=torch.float32, device=dev())
    k = torch.tensor([c[1] for c in cases], dtype=torch.int32, device=dev())
    p = torch.tensor([c[2] for c in cases], dtype=torch.float32, device=dev())
    u = torch.tensor(us, dtype=torch.float32, device=dev())
    got = ops.sample(logits.to(dev()), t, k, p, u).cpu().tolist()
    exact = 0
    for r, (temp, tk, tp) in enumerate(cases):
        probs = plain.sampling_distribution(logits[r], temp, tk, tp)
        want = plain.draw_inverse_cdf(probs, float(u[r].item())) if temp > 0 else int(logits[r].argmax())
        assert probs[got[r]] > 0, (r, got[r])
        if got[r] == want:
            exact += 1
            continue
        # 32-bit exponentials against 64-bit ones: the draw may land on a neighbour only when the
        # uniform number is within 1e-6 of the mass of an edge of the cumulative distribution
        cdf = probs.cumsum(-1)
        assert float((cdf - float(u[r].item()) * cdf[-1]).abs().min()) < 1e-6, (r, got[r], want)
    assert exact >= len(cases) - 2
    kept = plain.sampling_distribution(logits[10], 1.5, 100, 1.0)
    assert int((kept > 0).sum()) == 5000


def test_sampling_distribution_is_the_masked_softmax():
    import plain_qwen2 as plain
    from dispec_b200 import ops
    V, n = 50, 4000
    logits = (torch.randn(V, generator=torch.Generator().manual_seed(4)) * 2)
    probs = plain.sampling_distribution(logits, 0.9, 12, 0.8)
    u = torch.rand(n, generator=torch.Generator().manual_seed(5))
    rows = logits[None].expand(n, V).contiguous().to(dev())
    got = ops.sample(rows, torch.full((n,), 0.9, device=dev()), torch.full((n,), 12, dtype=torch.int32, device=dev()),
                     torch.full((n,), 0.8, device=dev()), u.to(dev())).cpu()
    freq = torch.bincount(got.long(), minlength=V).double() / n
    assert (freq[probs == 0] == 0).all()
    assert (freq - probs).abs().max().item() < 4 * math.sqrt(0.25 / n)


def test_sampling_keeps_ties_at_the_kth_value():
    from dispec_b200 import ops
    logits = torch.full((1, 64), -5.0)
    logits[0, [3, 9, 40]] = 2.0  # three tokens tie for the top; top_k = 2 keeps all three
    seen = set()
    for u in [0.01, 0.34, 0.5, 0.67, 0.99]:
        got = ops.sample(logits.to(dev()), torch.tensor([1.0], device=dev()),
                         torch.tensor([2], dtype=torch.int32, device=dev()),
                         torch.tensor([1.0], device=dev()), torch.tensor([u], device=dev()))
        seen.add(int(got[0]))
    assert seen == {3, 9, 40}


def test_gemm_weight_streaming_is_deterministic_and_strided():
    from dispec_b200.ops import gemm
    big = rnd((8, 3 * 1536), torch.bfloat16, 25)
    x = big[:, 1536:2 * 1536]  # a strided view
    w = rnd((1536, 1536), torch.bfloat16, 26, 0.05)
    a = gemm.linear(x, w)
    for _ in range(3):
        assert torch.equal(a, gemm.linear(x, w))
    torch.testing.assert_close(a.double(), x.double() @ w.double().T, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M,I,K", [(1, 64, 96), (8, 8960, 1536), (13, 176, 80), (40, 224, 96), (64, 512, 776),
                                   (300, 512, 776), (2048, 1024, 1536)])
def test_gate_up_product_with_swiglu_epilogue(M, I, K):
    from dispec_b200 import ops
    from dispec_b200.ops import gemm
    x = rnd((M, K), torch.bfloat16, 41)
    wg, wu = rnd((I, K), torch.bfloat16, 42, 0.15), rnd((I, K), torch.bfloat16, 43, 0.15)
    b = gemm.SWIGLU_BLOCK
    w = torch.stack([wg.view(I // b, b, K), wu.view(I // b, b, K)], dim=1).reshape(2 * I, K).contiguous()
    g, u = x.double() @ wg.double().T, x.double() @ wu.double().T
    ref = g * torch.sigmoid(g) * u
    out = gemm.linear_gate_up_swiglu(x, w)
    torch.testing.assert_close(out.double(), ref, atol=3e-2, rtol=3e-2)
    # the unfused pair of kernels on the same interleaved weight
    unfused = ops.swiglu(gemm.linear(x, w, backend="simt"), block=b)
    torch.testing.assert_close(unfused.double(), ref, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("case", ATTN_CASES + [(28, 4, 128, 16, 1200, 1, 0), (5, 5, 80, 16, 130, 64, 0),
                                               (8, 1, 256, 16, 100, 9, 0), (12, 2, 128, 16, 700, 300, 0)])
def test_attention_tensor_core(case):
    out, ref = run_attention("tensor_core", torch.bfloat16, *case)
    torch.testing.assert_close(out, ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("plant", [0, 15, 16, 63, 64, 65, 255, 256, 511, 600])
@pytest.mark.parametrize("q_len", [1, 37])
def test_attention_tensor_core_far_key_stands_out(plant, q_len):
    out, ref = run_attention("tensor_core", torch.bfloat16, 12, 2, 64, 16, 700, q_len, 0, plant=plant,
                             seed=plant)
    torch.testing.assert_close(out, ref, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("offset", [-1, 0, 1])
@pytest.mark.parametrize("q_len", [1, 20])
def test_attention_tensor_core_window_edge(offset, q_len):
    ctx, window = 333, 100
    plant = ctx - 1 - window + 1 + offset
    out, ref = run_attention("tensor_core", torch.bfloat16, 6, 2, 32, 8, ctx, q_len, window, plant=plant,
                             seed=9)
    torch.testing.assert_close(out, ref, atol=3e-2, rtol=3e-2)


def test_attention_tensor_core_mixed_batch_matches_alone():
    """Single tokens (with key splits) beside a portion of a prompt, ragged lengths."""
    from dispec_b200.ops import attention as A
    H, KVH, D, page = 6, 2, 64, 16
    q_lens = [1, 1, 1, 23, 70]
    ctx_lens = [17, 300, 64, 23, 200]
    g = torch.Generator().manual_seed(11)
    num_pages = sum((c + page - 1) // page for c in ctx_lens) + 2
    kp = torch.full((num_pages, KVH, page, D), float("nan"), dtype=torch.bfloat16)
    vp = kp.clone()
    perm = torch.randperm(num_pages, generator=g).tolist()
    maxp = max((c + page - 1) // page for c in ctx_lens)
    table = torch.full((len(q_lens), maxp), -1, dtype=torch.int32)
    qs, refs, positions, seqs = [], [], [], []
    for s, (ql, cl) in enumerate(zip(q_lens, ctx_lens)):
        k = torch.randn(cl, KVH, D, generator=g).bfloat16().float()
        v = torch.randn(cl, KVH, D, generator=g).bfloat16().float()
        q = torch.randn(ql, H, D, generator=g).bfloat16().float()
        for j in range((cl + page - 1) // page):
            table[s, j] = perm.pop()
        for b in range(cl):
            kp[table[s, b // page], :, b % page] = k[b].bfloat16()
            vp[table[s, b // page], :, b % page] = v[b].bfloat16()
        pos = torch.arange(cl - ql, cl, dtype=torch.int32)
        refs.append(_attention_reference(q.double(), k.double(), v.double(), pos, 0, D ** -0.5))
        qs.append(q)
        positions.append(pos)
        seqs += [s] * ql
    qd = torch.cat(qs).bfloat16().reshape(-1, H * D).to(dev())
    out = torch.empty_like(qd)
    A.paged_attention_tensor_core(qd, H * D, kp.to(dev()), vp.to(dev()), table.to(dev()),
                                  torch.cat(positions).to(dev()),
                                  torch.tensor(seqs, dtype=torch.int32, device=dev()), out, H, KVH, D, 0,
                                  D ** -0.5, q_lens=q_lens, ctx_lens=ctx_lens, splits=4)
    got = out.float().cpu().view(-1, H, D).double()
    torch.testing.assert_close(got, torch.cat(refs), atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("pairs", [0, 1])
@pytest.mark.parametrize("M,N,K,bias,resid,out_dtype", [
    (128, 256, 64, False, False, torch.bfloat16),     # one tile, one k block
    (65, 100, 96, True, False, torch.bfloat16),       # ragged in every direction, k tail of 32
    (300, 777, 776, True, True, torch.bfloat16),
    (2048, 2048, 1536, False, True, torch.bfloat16),  # more tiles than SMs: the ring runs across tiles
    (257, 384, 224, False, False, torch.float32),     # 32-bit output (logits)
    (1000, 8960, 1536, False, False, torch.bfloat16),
])
def test_gemm_tcgen05(pairs, M, N, K, bias, resid, out_dtype):
    from dispec_b200.ops import gemm, library
    x = rnd((M, K), torch.bfloat16, 51)
    w = rnd((N, K), torch.bfloat16, 52, 0.1)
    b = rnd((N,), torch.bfloat16, 53) if bias else None
    r = rnd((M, N), out_dtype, 54) if resid else None
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=dev())
    gemm._tcgen05(x, w, b, r, out, pairs=pairs)
    assert library.device_error() == 0  # no bounded wait ran out
    ref = x.double() @ w.double().T
    if bias:
        ref = ref + b.double()
    if resid:
        ref = ref + r.double()
    if out_dtype == torch.float32:
        torch.testing.assert_close(out.double(), ref, atol=1e-3, rtol=1e-4)
    else:
        torch.testing.assert_close(out.double(), ref, atol=3e-2, rtol=2e-2)


def test_gemm_tcgen05_rows_do_not_depend_on_the_batch_and_repeat_exactly():
    from dispec_b200.ops import gemm
    x = rnd((700, 1536), torch.bfloat16, 55)
    w = rnd((2048, 1536), torch.bfloat16, 56, 0.05)
    full = gemm.linear(x, w, backend="tcgen05")
    assert torch.equal(full, gemm.linear(x, w, backend="tcgen05"))
    part = gemm.linear(x[300:500].contiguous(), w, backend="tcgen05")
    assert torch.equal(full[300:500], part)


@pytest.mark.parametrize("M,N,K,bias,resid,out_dtype,target", [
    (8, 128, 64, False, False, torch.bfloat16, 0),       # one block, one k block
    (1, 256, 1536, True, False, torch.bfloat16, 0),
    (8, 2048, 1536, True, True, torch.bfloat16, 0),      # K split across a cluster
    (16, 1536, 8960, False, True, torch.bfloat16, 148),
    (13, 300, 96, True, True, torch.bfloat16, 0),        # ragged rows of W, k tail of 32
    (40, 384, 776, False, False, torch.bfloat16, 0),     # 32 < M <= 64 columns
    (64, 1000, 1536, True, False, torch.bfloat16, 0),
    (5, 40000, 1536, False, False, torch.float32, 0),    # more blocks than CTAs: double-buffered accumulator
    (9, 301, 200, True, True, torch.bfloat16, 0),        # a width that rules out four outputs per store
    (37, 1001, 200, True, False, torch.float32, 0),
    (64, 151936, 64, False, False, torch.float32, 0),    # the output head's width, every row count's epilogue
    (20, 4096, 1536, True, True, torch.bfloat16, 0),     # 32 blocks: K split over 4 CTAs, 5 rows each
])
def test_gemm_stream_tcgen05(M, N, K, bias, resid, out_dtype, target):
    from dispec_b200.ops import gemm, library
    x = rnd((M, K), torch.bfloat16, 61)
    w = rnd((N, K), torch.bfloat16, 62, 0.1)
    b = rnd((N,), torch.bfloat16, 63) if bias else None
    r = rnd((M, N), out_dtype, 64) if resid else None
    out = torch.full((M, N), float("nan"), dtype=out_dtype, device=dev())
    gemm._stream(x, w, b, r, out, target_ctas=target)
    assert library.device_error() == 0
    ref = x.double() @ w.double().T
    if bias:
        ref = ref + b.double()
    if resid:
        ref = ref + r.double()
    if out_dtype == torch.float32:
        torch.testing.assert_close(out.double(), ref, atol=1e-3, rtol=1e-4)
    else:
        torch.testing.assert_close(out.double(), ref, atol=3e-2, rtol=2e-2)
    again = torch.empty_like(out)
    gemm._stream(x, w, b, r, again, target_ctas=target)
    assert torch.equal(out, again)  # the cluster sum runs in a fixed order


@pytest.mark.parametrize("M,I,K,target", [(8, 8960, 1536, 0), (3, 224, 96, 148), (33, 2048, 1536, 0), (64, 176, 80, 0),
                                          # an odd number of rows (the epilogue pairs them), every width of the tile of A
                                          (1, 8960, 1536, 0), (7, 512, 96, 0), (16, 512, 96, 0), (17, 512, 96, 0),
                                          (24, 8960, 1536, 0), (31, 224, 96, 0), (32, 512, 776, 0), (63, 512, 96, 0)])
def test_gemm_stream_tcgen05_swiglu_epilogue(M, I, K, target):
    from dispec_b200.ops import gemm, library
    x = rnd((M, K), torch.bfloat16, 65)
    wg, wu = rnd((I, K), torch.bfloat16, 66, 0.15), rnd((I, K), torch.bfloat16, 67, 0.15)
    b = gemm.SWIGLU_BLOCK
    w = torch.stack([wg.view(I // b, b, K), wu.view(I // b, b, K)], dim=1).reshape(2 * I, K).contiguous()
    out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=dev())
    gemm._stream(x, w, None, None, out, epilogue=gemm.EPI_SWIGLU, target_ctas=target)
    assert library.device_error() == 0
    g, u = x.double() @ wg.double().T, x.double() @ wu.double().T
    torch.testing.assert_close(out.double(), g * torch.sigmoid(g) * u, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("M,N,K,bias,resid,target", [
    (8, 2048, 1536, True, False, 0),      # K split over a cluster: the owners of the rows scale them
    (16, 1536, 1536, False, True, 0),     # two rows per owner
    (1, 256, 1536, True, True, 0),
    (5, 1000, 200, True, False, 0),       # ragged rows of W, K of 3 blocks and a tail
    (13, 40000, 96, False, False, 0),     # more blocks than CTAs: no split, every CTA scales all rows
    (3, 384, 3584, False, True, 148),
    (33, 2048, 1536, True, True, 0),      # more than 16 rows: the cluster reads its partial tiles
    (64, 1536, 1536, False, True, 0),
    (40, 40000, 96, True, False, 0),
    (6, 302, 96, True, False, 0),         # a width that rules out four outputs per store
])
def test_gemm_stream_norm_taken_apart(M, N, K, bias, resid, target):
    """The few-row product with a norm split around it: rows times the gain as the operand, the
    rsqrt factors formed by the kernel from the rows themselves; against the norm's formula in
    float64, and against the norm kernel followed by the plain product."""
    from dispec_b200 import ops
    from dispec_b200.ops import gemm, library
    eps = 3e-5
    h = rnd((M, K), torch.bfloat16, 161, 3.0)
    h[0] *= 40.0  # rows of very different size: a factor of the wrong row would show
    gain = (1.0 + rnd((K,), torch.float32, 162, 0.3)).bfloat16()
    w = rnd((N, K), torch.bfloat16, 163, 0.1)
    b = rnd((N,), torch.bfloat16, 164) if bias else None
    r = rnd((M, N), torch.bfloat16, 165) if resid else None
    scaled = (h.float() * gain.float()).bfloat16()
    normed = gemm.NormedRows(h, gain, eps, scaled)
    assert normed.splittable(w)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    gemm._stream(scaled, w, b, r, out, target_ctas=target, norm=normed)
    assert library.device_error() == 0
    hd = h.double()
    y = hd * torch.rsqrt((hd * hd).mean(dim=1, keepdim=True) + eps) * gain.double()
    ref = y @ w.double().T
    if bias:
        ref = ref + b.double()
    if resid:
        ref = ref + r.double()
    torch.testing.assert_close(out.double(), ref, atol=3e-2, rtol=2e-2)
    # no further from the truth than the norm kernel followed by the plain product (which rounds
    # the normalised rows twice, this path once)
    two = gemm.linear(ops.rms_norm(h, gain, eps), w, b, residual=r)
    assert (out.double() - ref).abs().max() <= 1.25 * (two.double() - ref).abs().max() + 1e-3
    # through linear(): the same kernel, the same bits
    assert torch.equal(gemm.linear(normed, w, b, residual=r), out) or target != 0


@pytest.mark.parametrize("M,I,K", [(8, 8960, 1536), (16, 224, 96), (3, 512, 776), (64, 8960, 1536), (17, 224, 96)])
def test_gemm_stream_norm_taken_apart_with_swiglu(M, I, K):
    from dispec_b200.ops import gemm, library
    eps = 1e-6
    h = rnd((M, K), torch.bfloat16, 171, 2.0)
    gain = (1.0 + rnd((K,), torch.float32, 172, 0.3)).bfloat16()
    wg, wu = rnd((I, K), torch.bfloat16, 173, 0.15), rnd((I, K), torch.bfloat16, 174, 0.15)
    blk = gemm.SWIGLU_BLOCK
    w = torch.stack([wg.view(I // blk, blk, K), wu.view(I // blk, blk, K)], dim=1).reshape(2 * I, K).contiguous()
    scaled = (h.float() * gain.float()).bfloat16()
    normed = gemm.NormedRows(h, gain, eps, scaled)
    out = gemm.linear_gate_up_swiglu(normed, w)
    assert library.device_error() == 0
    hd = h.double()
    rstd = torch.rsqrt((hd * hd).mean(dim=1, keepdim=True) + eps)
    # the kernel's own arithmetic: the operand it is given (rows times gain, rounded), the factors
    # of the rows, the activation
    g, u = scaled.double() @ wg.double().T * rstd, scaled.double() @ wu.double().T * rstd
    torch.testing.assert_close(out.double(), g * torch.sigmoid(g) * u, atol=3e-2, rtol=3e-2)
    # and against the norm's formula: no further off than the norm kernel followed by the product
    y = hd * rstd * gain.double()
    g, u = y @ wg.double().T, y @ wu.double().T
    ref = g * torch.sigmoid(g) * u
    from dispec_b200 import ops
    two = gemm.linear_gate_up_swiglu(ops.rms_norm(h, gain, eps), w)
    assert (out.double() - ref).abs().max() <= 1.25 * (two.double() - ref).abs().max() + 1e-3


@pytest.mark.parametrize("M,N,K,target", [(8, 1536, 8960, 0), (16, 300, 96, 0), (2, 40000, 64, 0), (33, 512, 96, 0),
                                          (64, 1536, 8960, 0), (70, 512, 96, 0)])
def test_gemm_stream_scaled_second_output(M, N, K, target):
    """linear(then_norm=): beside its result the product stores the rounded result times the next
    norm's gain; with more rows it stores nothing and the norm kernel runs."""
    from dispec_b200 import ops
    from dispec_b200.ops import gemm, library
    x = rnd((M, K), torch.bfloat16, 181)
    w = rnd((N, K), torch.bfloat16, 182, 0.1)
    r = rnd((M, N), torch.bfloat16, 183)
    gain = (1.0 + rnd((N,), torch.float32, 184, 0.3)).bfloat16()
    plain = gemm.linear(x, w, residual=r)
    out, nxt = gemm.linear(x, w, residual=r, then_norm=(gain, 1e-6))
    assert library.device_error() == 0
    assert torch.equal(out, plain) and nxt.source is out
    if M <= gemm.NORM_SPLIT_MAX_ROWS:
        assert torch.equal(nxt.scaled, (out.float() * gain.float()).bfloat16())
    else:
        assert nxt.scaled is None
    torch.testing.assert_close(nxt.materialize().float(), ops.rms_norm(out, gain, 1e-6).float())


@pytest.mark.parametrize("decode_kernel", [True, False])
@pytest.mark.parametrize("splits", [1, 3, 8, 12])
def test_attention_tensor_core_single_token_splits(splits, decode_kernel):
    """One decoded token over 900 keys: no split, splits merged on chip by the cluster (up to 8),
    and splits merged from global scratch by the combine kernel (above 8)."""
    from dispec_b200.ops import attention as A
    # decode_kernel: the warp-parallel kernel (any number of splits up to 8) or the tile kernel
    H, KVH, D, page, ctx = 12, 2, 128, 16, 900
    g = torch.Generator().manual_seed(70 + splits)
    q = torch.randn(1, H, D, generator=g).bfloat16().float()
    k = torch.randn(ctx, KVH, D, generator=g).bfloat16().float()
    v = torch.randn(ctx, KVH, D, generator=g).bfloat16().float()
    ref = _attention_reference(q.double(), k.double(), v.double(), torch.tensor([ctx - 1]), 0, D ** -0.5)
    kp, vp, perm = _paged(k, v, page, (ctx + page - 1) // page + 2, torch.bfloat16, splits)
    out = torch.empty((1, H * D), dtype=torch.bfloat16, device=dev())
    A.paged_attention_tensor_core(q.bfloat16().reshape(1, H * D).to(dev()), H * D, kp, vp, perm.view(1, -1).to(dev()),
                                  None, None, out, H, KVH, D, 0, D ** -0.5, q_lens=[1], ctx_lens=[ctx], splits=splits,
                                  decode_kernel=decode_kernel)
    torch.testing.assert_close(out.float().cpu().view(1, H, D).double(), ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("out_dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("tokens,H,D,splits", [(1, 12, 128, 16), (3, 5, 16, 1), (2, 14, 48, 7), (4, 2, 256, 32)])
def test_attention_combine_alone(tokens, H, D, splits, out_dtype):
    """The kernel that merges split attention, against the same formula in float64; some splits saw
    no key (maximum -inf, sum 0, output never written), one row saw none at all."""
    from dispec_b200.ops import library as L
    g = torch.Generator().manual_seed(100 + splits)
    rows = tokens * H
    o = torch.randn(rows, splits, D, generator=g)
    m = torch.randn(rows, splits, generator=g) * 6
    l = torch.rand(rows, splits, generator=g) * 50 + 0.1
    dead = torch.rand(rows, splits, generator=g) < 0.3
    dead[0] = True  # a padding row
    if rows > 1:
        dead[1] = False
    m[dead], l[dead] = float("-inf"), 0.0
    o[dead] = float("nan")
    w = torch.where(dead, torch.zeros(()), torch.exp2(m - m.max(1, keepdim=True).values).nan_to_num(0.0)).double()
    num = (w[..., None] * o.nan_to_num(0.0).double()).sum(1)
    den = (w * l.double()).sum(1, keepdim=True)
    ref = torch.where(den > 0, num / den.clamp_min(1e-300), torch.zeros(())).view(tokens, H * D)
    out = torch.full((tokens, H * D), float("nan"), dtype=out_dtype, device=dev())
    ml = torch.stack([m, l], -1).contiguous().to(dev())
    od = o.contiguous().to(dev())
    L.check(L.core().dsp_attn_combine(L.ptr(od), L.ptr(ml), L.ptr(out), L.i64(out.stride(0)), tokens, H, D, splits,
                                      L.dtype_code(out_dtype), L.stream_handle()))
    torch.cuda.synchronize()
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    torch.testing.assert_close(out.double().cpu(), ref, atol=tol, rtol=tol)


TCGEN05_CASES = [
    # H, KVH, D, page, ctx, q_len, window: portions of prompts on the tcgen05 kernel
    (12, 2, 128, 16, 700, 300, 0),   # several query tiles, group of 6 (126 of 128 rows used)
    (14, 2, 64, 8, 333, 333, 0),     # whole prompt, group of 7, small pages
    (4, 4, 128, 32, 520, 130, 0),    # no sharing of keys between heads
    (8, 1, 64, 64, 1000, 77, 0),     # one page per key tile
    (6, 2, 128, 16, 900, 200, 150),  # window: first key tile of most query tiles starts before it
    (6, 3, 64, 8, 400, 2, 70),       # two tokens
    (64, 1, 64, 16, 150, 5, 0),      # a group that fills half a tile per token
]


@pytest.mark.parametrize("backend", ["tcgen05", "mma"])
@pytest.mark.parametrize("case", TCGEN05_CASES)
def test_attention_prefill_backends(case, backend):
    """The same portions of prompts on the tcgen05 kernel and on the mma.sync kernel (which serves
    the other head sizes)."""
    from dispec_b200.ops import attention as A
    assert A.tcgen05_supported(case[2], case[0] // case[1], case[3], torch.bfloat16)
    out, ref = run_attention("tensor_core", torch.bfloat16, *case, prefill_kernel=backend)
    torch.testing.assert_close(out, ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("case", TCGEN05_CASES + [(12, 2, 128, 16, 2048, 1100, 0), (14, 2, 64, 8, 1500, 640, 300)])
@pytest.mark.parametrize("order", ["ascending", "runs"])
def test_attention_tcgen05_pages_in_runs(case, order, monkeypatch):
    """Key tiles whose pages follow each other in the pool are fetched with one request per operand;
    the result is, bit for bit, that of the same keys on scattered pages and that of a build
    which fetches page by page."""
    out, ref = run_attention("tensor_core", torch.bfloat16, *case, prefill_kernel="tcgen05", page_order=order)
    torch.testing.assert_close(out, ref, atol=2e-2, rtol=2e-2)
    scattered, _ = run_attention("tensor_core", torch.bfloat16, *case, prefill_kernel="tcgen05")
    assert torch.equal(out, scattered)
    monkeypatch.setenv("DISPEC_B200_PAGE_RUNS", "0")
    by_page, _ = run_attention("tensor_core", torch.bfloat16, *case, prefill_kernel="tcgen05", page_order=order)
    assert torch.equal(out, by_page)


@pytest.mark.parametrize("plant", [0, 63, 64, 200, 511, 699])
def test_attention_tcgen05_far_key_stands_out_on_pages_in_runs(plant):
    out, ref = run_attention("tensor_core", torch.bfloat16, 12, 2, 128, 16, 700, 150, 0, plant=plant, seed=plant,
                             page_order="ascending")
    torch.testing.assert_close(out, ref, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("plant", [0, 15, 16, 63, 64, 65, 127, 128, 255, 256, 511, 600, 699])
def test_attention_tcgen05_far_key_stands_out(plant):
    out, ref = run_attention("tensor_core", torch.bfloat16, 12, 2, 128, 16, 700, 150, 0, plant=plant, seed=plant)
    torch.testing.assert_close(out, ref, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("H,KVH,D,splits", [(16, 1, 128, 8), (16, 1, 64, 3), (12, 1, 80, 5), (9, 1, 128, 2),
                                            (32, 2, 64, 8), (7, 1, 96, 7), (3, 3, 128, 8)])
def test_decode_attention_cluster_merge_paths(H, KVH, D, splits):
    """The ways the cluster's CTAs put their partial rows together, by group size and split count:
    rows sent to their owners (one or several rows per owner, owners without a row, more rows
    than warps) and, where the owners' inboxes would not hold them, partials read from the other
    CTAs.  Two rows: a long one with a far key that stands out, and one of three keys."""
    from dispec_b200 import ops
    from dispec_b200.ops import attention as A
    page, ctx_lens, plant = 16, [1500, 3], [77, 1]
    B = len(ctx_lens)
    g = torch.Generator().manual_seed(1000 * H + splits)
    pages_per = [(c + page - 1) // page for c in ctx_lens]
    num_pages = sum(pages_per) + 2
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((B, max(pages_per)), -1, dtype=torch.int32)
    kp = torch.full((num_pages, KVH, page, D), float("nan"), dtype=torch.bfloat16)
    vp = kp.clone()
    q = torch.randn(B, H, D, generator=g).bfloat16()
    refs = []
    for s, c in enumerate(ctx_lens):
        k = torch.randn(c, KVH, D, generator=g).bfloat16()
        v = torch.randn(c, KVH, D, generator=g).bfloat16()
        k[plant[s]] = (q[s, ::H // KVH] * 4.0).bfloat16()
        for j in range(pages_per[s]):
            table[s, j] = perm.pop()
        for b in range(c):
            kp[table[s, b // page], :, b % page] = k[b]
            vp[table[s, b // page], :, b % page] = v[b]
        refs.append(_attention_reference(q[s:s + 1].double(), k.double(), v.double(), torch.tensor([c - 1]),
                                         0, D ** -0.5)[0])
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    out = torch.full((B, H * D), float("nan"), dtype=torch.bfloat16, device=dev())
    A.paged_attention_tiles(q.reshape(B, H * D).to(dev()), H * D, kp.to(dev()), vp.to(dev()), table.to(dev()),
                            i32(list(range(B + 1))), i32(ctx_lens), i32(list(range(B))), i32([0] * B), B, B, out,
                            H, KVH, D, 0, D ** -0.5, splits)
    torch.cuda.synchronize()
    ops.raise_on_device_error("decode attention, cluster merge")
    got = out.float().cpu().view(B, H, D)
    for s, ref in enumerate(refs):
        torch.testing.assert_close(got[s].double(), ref, atol=2e-2, rtol=2e-2, msg=lambda m: f"row {s}: {m}")


@pytest.mark.parametrize("offset", [-1, 0, 1])
@pytest.mark.parametrize("q_len", [2, 40])
def test_attention_tcgen05_window_edge(offset, q_len):
    ctx, window = 333, 100
    plant = ctx - 1 - window + 1 + offset
    out, ref = run_attention("tensor_core", torch.bfloat16, 6, 2, 64, 8, ctx, q_len, window, plant=plant, seed=9)
    torch.testing.assert_close(out, ref, atol=3e-2, rtol=3e-2)


@pytest.mark.parametrize("splits,outer", [(8, 2), (8, 5), (3, 4), (1, 3)])
@pytest.mark.parametrize("H,KVH,D,page,window", [(12, 2, 128, 16, 0), (6, 3, 64, 8, 700), (14, 2, 48, 32, 0)])
def test_decode_attention_with_key_ranges_beyond_the_cluster(splits, outer, H, KVH, D, page, window):
    """Single tokens whose keys are cut into ``outer`` ranges of ``splits`` CTAs each, merged by a
    second kernel: long and short rows side by side (ranges without a key, a row of one key, a
    padding row of length 0), with one far key made to stand out in every row."""
    from dispec_b200 import ops
    from dispec_b200.ops import attention as A
    ctx_lens = [2500, 1, 0, 40, 1023, 1025]
    plant = [1300, 0, 0, 17, 3, 1024]
    B = len(ctx_lens)
    g = torch.Generator().manual_seed(11 * splits + outer)
    pages_per = [(c + page - 1) // page for c in ctx_lens]
    num_pages = sum(pages_per) + 2
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((B, max(pages_per)), -1, dtype=torch.int32)
    kp = torch.full((num_pages, KVH, page, D), float("nan"), dtype=torch.bfloat16)
    vp = kp.clone()
    q = torch.randn(B, H, D, generator=g).bfloat16()
    refs = []
    for s, c in enumerate(ctx_lens):
        if c == 0:
            refs.append(None)
            continue
        k = torch.randn(c, KVH, D, generator=g).bfloat16()
        v = torch.randn(c, KVH, D, generator=g).bfloat16()
        # the planted key is the query of the group's first head, enlarged: that head sees little else
        k[plant[s]] = (q[s, ::H // KVH] * 4.0).bfloat16()
        for j in range(pages_per[s]):
            table[s, j] = perm.pop()
        for b in range(c):
            kp[table[s, b // page], :, b % page] = k[b]
            vp[table[s, b // page], :, b % page] = v[b]
        refs.append(_attention_reference(q[s:s + 1].double(), k.double(), v.double(), torch.tensor([c - 1]),
                                         window, D ** -0.5)[0])
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    out = torch.full((B, H * D), float("nan"), dtype=torch.bfloat16, device=dev())
    A.paged_attention_tiles(q.reshape(B, H * D).to(dev()), H * D, kp.to(dev()), vp.to(dev()), table.to(dev()),
                            i32(list(range(B + 1))), i32(ctx_lens), i32(list(range(B))), i32([0] * B), B, B, out,
                            H, KVH, D, window, D ** -0.5, splits, outer=outer)
    torch.cuda.synchronize()
    ops.raise_on_device_error("decode attention with key ranges")
    got = out.float().cpu().view(B, H, D)
    for s, ref in enumerate(refs):
        if ref is None:
            continue
        torch.testing.assert_close(got[s].double(), ref, atol=2e-2, rtol=2e-2, msg=lambda m: f"row {s}: {m}")


@pytest.mark.parametrize("H,KVH,D,rot,page,window,outer", [(12, 2, 128, 128, 16, 0, 1), (6, 3, 64, 32, 8, 40, 1),
                                                           (4, 4, 16, 16, 32, 0, 1), (14, 2, 48, 48, 16, 0, 1),
                                                           (12, 2, 128, 128, 16, 0, 3), (6, 3, 64, 32, 8, 40, 2)])
def test_decode_attention_that_rotates_and_stores_itself(H, KVH, D, rot, page, window, outer):
    """Single tokens: the kernel that rotates q and the token's key and writes key and value to the
    cache against the rotation kernel followed by the plain attention kernel: the same outputs and
    the same cache, for tokens at a page's first and last offset and in the middle."""
    from dispec_b200 import ops
    from dispec_b200.ops import attention as A
    ctx_lens = [page * 3, page * 2 + 1, 77, 1, 300]
    B = len(ctx_lens)
    g = torch.Generator().manual_seed(5)
    pages_per = [(c + page - 1) // page for c in ctx_lens]
    num_pages = sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((B, max(pages_per)), -1, dtype=torch.int32)
    for s in range(B):
        for j in range(pages_per[s]):
            table[s, j] = perm.pop()
    pool = torch.randn(2, num_pages, KVH, page, D, generator=g).bfloat16()
    for s, c in enumerate(ctx_lens):  # the slot of the newest position is not in the cache yet
        pool[:, table[s, (c - 1) // page], :, (c - 1) % page] = float("nan")
    qkv = torch.randn(B, (H + 2 * KVH) * D, generator=g).bfloat16().to(dev())
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(dev())
    positions = torch.tensor([c - 1 for c in ctx_lens], dtype=torch.int32, device=dev())
    seq = torch.arange(B, dtype=torch.int32, device=dev())
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=dev())
    q_start, ctx_len = i32(list(range(B + 1))), i32(ctx_lens)
    ts, t0 = i32(list(range(B))), i32([0] * B)
    table_d = table.to(dev())
    results = []
    for fused in (False, True):
        kp, vp = pool[0].clone().to(dev()), pool[1].clone().to(dev())
        rows = qkv.clone()
        out = torch.empty((B, H * D), dtype=torch.bfloat16, device=dev())
        if not fused:
            ops.rope_kv_store(rows, positions, seq, table_d, kp, vp, inv_freq, H, KVH, D, rot)
        for splits in (3,):
            A.paged_attention_tiles(rows, rows.stride(0), kp, vp, table_d, q_start, ctx_len, ts, t0, B, B, out, H,
                                    KVH, D, window, D ** -0.5, splits,
                                    fused_rope=(inv_freq, rot, True) if fused else None, outer=outer)
        torch.cuda.synchronize()
        results.append((out.float().cpu(), kp.float().cpu(), vp.float().cpu()))
    (o0, k0, v0), (o1, k1, v1) = results
    assert torch.isfinite(o0).all() and torch.isfinite(o1).all()
    torch.testing.assert_close(o1, o0, atol=2e-2, rtol=2e-2)
    written = torch.zeros(num_pages, page, dtype=torch.bool)
    for s, c in enumerate(ctx_lens):
        written[table[s, (c - 1) // page], (c - 1) % page] = True
    for a, b in ((k0, k1), (v0, v1)):
        a, b = a.permute(0, 2, 1, 3), b.permute(0, 2, 1, 3)  # [page, offset, kvh, d]
        torch.testing.assert_close(b[written], a[written], atol=1e-2, rtol=1e-2)
        assert torch.equal(b[~written], a[~written])  # nothing else was touched
    ops.raise_on_device_error("decode attention with rotation")


# ------------------------------------------------------------------ counter-based random fill

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape", [(1,), (7, 13), (1023,), (3, 5, 17), (257, 96)])
def test_fill_normal_equals_the_cpu_generator_bit_for_bit(dtype, shape):
    import numpy as np
    import plain_qwen2 as plain
    from dispec_b200 import ops
    from dispec_b200.weights import counter_rng
    seed, ordinal, std, mean = 2 ** 35 + 11, 41, 0.02, 1.0
    out = ops.fill_normal(torch.empty(shape, dtype=dtype, device=dev()), seed, ordinal, std, mean)
    want = torch.from_numpy(counter_rng.normal(seed, ordinal, shape, std, mean))
    assert torch.equal(out.cpu(), want.to(dtype))
    z = ops.fill_normal(torch.empty(shape, dtype=torch.float32, device=dev()), seed, ordinal, 1.0, 0.0).cpu().flatten()
    for i in sorted({0, z.numel() // 2, z.numel() - 1}):
        assert np.float32(z[i].item()) == plain.counter_normal_element(seed, ordinal, i)
    # rounded through bfloat16 into a float32 buffer: what loading a bfloat16 file into the 32-bit engine gives
    via = ops.fill_normal(torch.empty(shape, dtype=torch.float32, device=dev()), seed, ordinal, std, mean, through_bf16=True)
    assert torch.equal(via.cpu(), want.to(torch.bfloat16).float())


def test_fill_normal_of_a_large_tensor_is_fast_and_any_slice_can_be_recomputed():
    """The output matrix of the largest shape (152,064 x 5,120, 1.5 GB in bfloat16) is filled in
    place on the device; slices anywhere in it equal the CPU generator started at that element."""
    import time
    from dispec_b200 import ops
    from dispec_b200.weights import counter_rng
    rows, cols = 152064, 5120
    out = torch.empty((rows, cols), dtype=torch.bfloat16, device=dev())
    ops.fill_normal(out[:8], 4, 290, 0.02)  # first call: library load
    torch.cuda.synchronize()
    t0 = time.time()
    ops.fill_normal(out, 4, 290, 0.02)
    torch.cuda.synchronize()
    assert time.time() - t0 < 2.0
    flat = out.view(-1)
    for start in (0, 5119, 123_456_789, rows * cols - 1000):
        want = torch.from_numpy(np_f32(counter_rng.standard_normal(4, 290, 1000, start=start)) * np_f32(0.02))
        assert torch.equal(flat[start:start + 1000].cpu(), want.to(torch.bfloat16)), start
    sample = flat[::997].float()
    assert abs(sample.mean().item()) < 2e-4 and abs(sample.std().item() - 0.02) < 2e-4


def np_f32(x):
    import numpy as np
    return np.float32(x) if not hasattr(x, "dtype") else x.astype(np.float32, copy=False)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_random_model_filled_on_the_device_equals_the_written_folder(tmp_path, dtype):
    """load_random_model (device fill) and write_random_model (CPU generator) + load_model give
    the same weights, hence the same logits bit for bit."""
    import replay_util as ru
    from dispec_b200 import load_model, load_model_config
    from dispec_b200.engine import ModelRunner, SeqEntry
    from dispec_b200.weights import load_random_model, write_random_model
    cfg = load_model_config(ru.CONFIG_B)
    overrides = {"lm_head.weight": 0.5}
    write_random_model(cfg, str(tmp_path), seed=1, std=0.05, dtype="bfloat16", overrides=overrides)
    from_file = load_model(str(tmp_path), dtype, dev())
    on_device = load_random_model(cfg, 1, 0.05, dtype, dev(), overrides=overrides)
    assert torch.equal(from_file.embedding.weight, on_device.embedding.weight)
    assert torch.equal(from_file.layers[2].mixer.w_qkv, on_device.layers[2].mixer.w_qkv)
    assert torch.equal(from_file.layers[1].mixer_norm.weight, on_device.layers[1].mixer_norm.weight)
    ids = ru.random_ids(21, ru.CONFIG_B["vocab_size"], 3)
    logits = []
    for model in (from_file, on_device):
        runner = ModelRunner(model, page_size=8, num_pages=8, max_num_seqs=2)
        runner.admit("s")
        logits.append(runner.step([SeqEntry("s", ids, 0, list(range(len(ids))))]))
    assert torch.equal(logits[0], logits[1])
    # a folder written from device-filled tensors is the same file content
    write_random_model(cfg, str(tmp_path / "dev"), seed=1, std=0.05, dtype="bfloat16", overrides=overrides, device=dev())
    a = open(tmp_path / "model.safetensors", "rb").read()
    b = open(tmp_path / "dev" / "model.safetensors", "rb").read()
    assert a == b


@pytest.mark.parametrize("M", [130, 200, 256])
def test_linear_runs_narrow_long_products_in_chunks_of_rows(M):
    """A few hundred rows, a narrow product with a long K (the down projection's shape): the
    few-row kernel per 128 rows instead of eight tiles of the many-row kernel; a norm handed on
    from it runs as a kernel."""
    from dispec_b200 import ops
    from dispec_b200.ops import gemm, library, tuning
    N, K, eps = 1536, 8960, 1e-6
    assert tuning.rows_in_chunks_is_faster(M, N, K, torch.device(dev()), gemm.STREAM_MAX_ROWS)
    assert not tuning.rows_in_chunks_is_faster(M, 17920, 1536, torch.device(dev()), gemm.STREAM_MAX_ROWS)
    x = rnd((M, K), torch.bfloat16, 201)
    w = rnd((N, K), torch.bfloat16, 202, 0.05)
    b = rnd((N,), torch.bfloat16, 203)
    r = rnd((M, N), torch.bfloat16, 204)
    gain = (1.0 + rnd((N,), torch.float32, 205, 0.3)).bfloat16()
    out, nxt = gemm.linear(x, w, b, residual=r, then_norm=(gain, eps))
    assert library.device_error() == 0
    ref = x.double() @ w.double().T + b.double() + r.double()
    torch.testing.assert_close(out.double(), ref, atol=3e-2, rtol=2e-2)
    assert nxt.scaled is None and nxt.source is out
    w2 = rnd((1024, N), torch.bfloat16, 207, 0.1)
    assert torch.equal(gemm.linear(nxt, w2), gemm.linear(ops.rms_norm(out, gain, eps), w2))


@pytest.mark.parametrize("M,N,K,bias,resid,swiglu", [(65, 2048, 1536, True, False, False), (128, 1536, 8960, False, True, False),
                                                     (100, 17920, 1536, False, False, True), (128, 1000, 200, True, True, False),
                                                     (97, 40000, 96, True, False, False), (128, 4096, 1536, False, False, True)])
def test_gemm_stream_up_to_128_rows(M, N, K, bias, resid, swiglu):
    """65 to 128 rows of A in the few-row kernel: the accumulator of 128 columns is taken in two
    windows of 64 by the epilogues (K split over a cluster, and not)."""
    from dispec_b200.ops import gemm, library
    x = rnd((M, K), torch.bfloat16, 211)
    x[M - 1] *= 3.0  # the last row, in the second window
    if swiglu:
        I = N // 2
        wg, wu = rnd((I, K), torch.bfloat16, 212, 0.15), rnd((I, K), torch.bfloat16, 213, 0.15)
        blk = gemm.SWIGLU_BLOCK
        w = torch.stack([wg.view(I // blk, blk, K), wu.view(I // blk, blk, K)], dim=1).reshape(N, K).contiguous()
        out = torch.full((M, I), float("nan"), dtype=torch.bfloat16, device=dev())
        gemm._stream(x, w, None, None, out, epilogue=gemm.EPI_SWIGLU)
        g, u = x.double() @ wg.double().T, x.double() @ wu.double().T
        assert library.device_error() == 0
        torch.testing.assert_close(out.double(), g * torch.sigmoid(g) * u, atol=3e-2, rtol=3e-2)
        return
    w = rnd((N, K), torch.bfloat16, 214, 0.1)
    b = rnd((N,), torch.bfloat16, 215) if bias else None
    r = rnd((M, N), torch.bfloat16, 216) if resid else None
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev())
    gemm._stream(x, w, b, r, out)
    assert library.device_error() == 0
    ref = x.double() @ w.double().T
    if bias:
        ref = ref + b.double()
    if resid:
        ref = ref + r.double()
    torch.testing.assert_close(out.double(), ref, atol=3e-2, rtol=2e-2)
    again = torch.empty_like(out)
    gemm._stream(x, w, b, r, again)
    assert torch.equal(out, again)


def test_measurement_entries_run_and_refuse_bad_arguments():
    """The two measurement kernels that `bench.py --only mma-rate | tma-rate` call: they run with
    bounded waits, report that no wait ran out, and refuse arguments outside their ranges."""
    import ctypes
    from dispec_b200.ops import library as L
    core = L.core()
    out = torch.zeros(3, dtype=torch.int64, device=dev())
    L.check(core.dsp_selftest_mma_issue_rate(16, 2, 50, ctypes.c_void_p(out.data_ptr()), L.stream_handle()))
    issue, done, ok = out.tolist()
    assert ok == 1 and issue > 0 and done >= issue
    assert core.dsp_selftest_mma_issue_rate(24, 1, 50, ctypes.c_void_p(out.data_ptr()), L.stream_handle()) != 0
    matrix = torch.zeros((1280, 1536), dtype=torch.bfloat16, device=dev())
    cycles = torch.zeros(4, dtype=torch.int64, device=dev())
    flag = torch.ones(1, dtype=torch.int32, device=dev())
    for stages, boxes, k_blocks in ((3, 2, 2), (6, 1, 1)):
        L.check(core.dsp_selftest_tma_rate(L.ptr(matrix), 1280, stages, boxes, k_blocks, 4, 50, L.ptr(cycles), L.ptr(flag),
                                           L.stream_handle()))
        torch.cuda.synchronize()
        assert int(flag.item()) == 1 and int(cycles.min()) > 0
    assert core.dsp_selftest_tma_rate(L.ptr(matrix), 1280, 3, 2, 5, 4, 50, L.ptr(cycles), L.ptr(flag), L.stream_handle()) != 0
    assert core.dsp_selftest_tma_rate(L.ptr(matrix), 1000, 3, 2, 2, 4, 50, L.ptr(cycles), L.ptr(flag), L.stream_handle()) != 0
    assert L.device_error() == 0
