"""The kernels' error reporting, shown to work: a bad token id, a bad page id and a bounded wait
that runs out each set their bit of the device error word, do no harm, and leave the context
usable.  Every case is built so that no memory outside an allocation can be touched: the tables
and pools are allocated with one row or page more than the kernels are told about, and the
"bad" id names exactly that extra one; the wait is the kernels' own bounded wait with a limit of
a few hundred tries on a barrier at which nothing arrives."""
import ctypes

import pytest
import torch

from test_kernels_gpu import _attention_reference, _paged, dev, rnd

pytestmark = pytest.mark.gpu

BAD_PAGE, BAD_TOKEN, WAIT_LIMIT = 1, 2, 4


def error_word():
    from dispec_b200.ops import library as L
    return L.device_error()


def test_bad_token_id_gives_a_zero_row_and_sets_its_bit():
    from dispec_b200 import ops
    from dispec_b200.ops import library as L
    vocab, hidden = 37, 48
    table = rnd((vocab + 1, hidden), torch.bfloat16, 1)  # one row more than the kernel is told about
    ids = torch.tensor([3, vocab, 0], dtype=torch.int32, device=dev())  # vocab is one past the end
    out = torch.full((3, hidden), 7.0, dtype=torch.bfloat16, device=dev())
    assert error_word() == 0
    L.check(L.core().dsp_embed(L.ptr(table), L.ptr(ids), L.ptr(out), 3, hidden, vocab, L.dtype_code(table.dtype),
                               L.stream_handle()))
    torch.cuda.synchronize()
    assert torch.equal(out[0], table[3]) and torch.equal(out[2], table[0])
    assert (out[1] == 0).all()  # not the extra row's contents
    with pytest.raises(ops.KernelError, match="token id outside the vocabulary"):
        ops.raise_on_device_error("embedding")
    assert error_word() == 0  # the read cleared it
    assert torch.equal(ops.embed(table, torch.tensor([vocab], dtype=torch.int32, device=dev()))[0], table[vocab])
    assert error_word() == 0  # the same id is fine for a table that has the row


def test_token_fed_from_a_row_that_does_not_exist_sets_its_bit():
    from dispec_b200.ops import library as L
    prev = torch.tensor([11, 12, 13, 99], dtype=torch.int32, device=dev())  # the kernel is told about 3
    ids = torch.tensor([5, 5, 5], dtype=torch.int32, device=dev())
    src = torch.tensor([2, 3, -1], dtype=torch.int32, device=dev())
    L.check(L.core().dsp_feed_tokens(L.ptr(ids), L.ptr(src), L.ptr(prev), 3, 3, L.stream_handle()))
    assert ids.tolist() == [13, 5, 5]
    assert error_word() == BAD_TOKEN and error_word() == 0


def _pools_with_a_spare_page(k, v, page, dtype, seed):
    """Pools of P + 1 pages of which the kernels see the first P (a view): page id P is outside the
    pool they know and inside the allocation."""
    ctx = k.shape[0]
    P = (ctx + page - 1) // page + 2
    kp, vp, perm = _paged(k, v, page, P + 1, dtype, seed)
    perm = perm.clone()
    assert int(perm.max()) <= P
    # keep every real page below P: swap whichever logical page landed on page P with a free one
    used = set(perm.tolist())
    if P in used:
        free = next(i for i in range(P) if i not in used)
        where = perm.tolist().index(P)
        kp[free], vp[free] = kp[P].clone(), vp[P].clone()
        perm[where] = free
    kp[P], vp[P] = 1000.0, 1000.0  # would dominate every output if it were read
    return kp, vp, perm, P


@pytest.mark.parametrize("kind,dtype,H,KVH,D,page,ctx,q_len", [
    ("generic", torch.float32, 4, 2, 32, 16, 150, 3),
    ("generic", torch.bfloat16, 6, 2, 48, 8, 90, 1),
    ("tensor_core", torch.bfloat16, 6, 2, 48, 16, 200, 37),   # mma.sync tiles (head size 48)
    ("tensor_core", torch.bfloat16, 12, 2, 128, 16, 700, 1),  # the single-token kernel
    ("tensor_core", torch.bfloat16, 12, 2, 128, 16, 700, 150),  # tcgen05 tiles
    ("tensor_core", torch.bfloat16, 14, 2, 64, 8, 333, 200),    # tcgen05 tiles, small pages
])
def test_bad_page_id_is_skipped_and_sets_its_bit(kind, dtype, H, KVH, D, page, ctx, q_len):
    """One logical page of the table names a page outside the pool: its keys are skipped (the
    output is the attention over the other keys), bit 1 is set, and the same launch with the
    table repaired is right afterwards."""
    from dispec_b200.ops import attention as A
    g = torch.Generator().manual_seed(ctx + q_len)
    q = torch.randn(q_len, H, D, generator=g).to(dtype).float()
    k = torch.randn(ctx, KVH, D, generator=g).to(dtype).float()
    v = torch.randn(ctx, KVH, D, generator=g).to(dtype).float()
    kp, vp, perm, P = _pools_with_a_spare_page(k, v, page, dtype, 5)
    positions = torch.arange(ctx - q_len, ctx, dtype=torch.int32)
    scale = D ** -0.5
    victim = 2  # logical page 2: keys 2 * page .. 3 * page - 1, which every query sees
    broken = perm.clone()
    broken[victim] = P
    keep = torch.ones(ctx, dtype=torch.bool)
    keep[victim * page:(victim + 1) * page] = False

    def launch(table):
        out = torch.empty((q_len, H * D), dtype=dtype, device=dev())
        qd = q.to(dtype).reshape(q_len, H * D).to(dev())
        seq = torch.zeros(q_len, dtype=torch.int32, device=dev())
        t = table.view(1, -1).to(dev())
        if kind == "generic":
            A.paged_attention_generic(qd, H * D, kp[:P], vp[:P], t, positions.to(dev()), seq, out, H, KVH, D, 0, scale)
        else:
            A.paged_attention_tensor_core(qd, H * D, kp[:P], vp[:P], t, positions.to(dev()), seq, out, H, KVH, D, 0,
                                          scale, q_lens=[q_len], ctx_lens=[ctx])
        torch.cuda.synchronize()
        return out.float().cpu().view(q_len, H, D).double()

    assert error_word() == 0
    got = launch(broken)
    assert error_word() == BAD_PAGE
    assert torch.isfinite(got).all() and got.abs().max().item() < 50  # page P (filled with 1000) was not read
    # the reference without the victim's keys: positions shift, so mask by hand
    ref = torch.empty_like(got)
    G = H // KVH
    for j in range(H):
        s = (q[:, j].double() @ k[:, j // G].double().T) * scale
        hidden = (torch.arange(ctx)[None, :] > positions[:, None]) | ~keep[None, :]
        ref[:, j] = torch.softmax(s.masked_fill(hidden, float("-inf")), dim=-1) @ v[:, j // G].double()
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    torch.testing.assert_close(got, ref, atol=tol, rtol=tol)
    fixed = launch(perm)
    assert error_word() == 0
    torch.testing.assert_close(fixed, _attention_reference(q.double(), k.double(), v.double(), positions, 0, scale),
                               atol=tol, rtol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_key_value_write_to_a_bad_page_is_dropped_and_sets_its_bit(dtype):
    from dispec_b200 import ops
    H, KVH, D, page, P = 4, 2, 32, 8, 3
    pool_k = torch.zeros((P + 1, KVH, page, D), dtype=dtype, device=dev())
    pool_v = torch.zeros_like(pool_k)
    T = 5
    qkv = rnd((T, (H + 2 * KVH) * D), dtype, 3)
    positions = torch.arange(6, 6 + T, dtype=torch.int32, device=dev())  # logical pages 0 and 1
    seq = torch.zeros(T, dtype=torch.int32, device=dev())
    table = torch.tensor([[1, P, 0]], dtype=torch.int32, device=dev())  # logical page 1 names page P
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))).to(dev())
    before = qkv.clone()
    ops.rope_kv_store(qkv, positions, seq, table, pool_k[:P], pool_v[:P], inv_freq, H, KVH, D, D)
    torch.cuda.synchronize()
    assert error_word() == BAD_PAGE
    assert (pool_k[P] == 0).all() and (pool_v[P] == 0).all()  # nothing was written there
    assert (pool_k[1, :, 6:8] != 0).any()  # positions 6 and 7 went to page 1
    assert (pool_k[0] == 0).all() and (pool_k[2] == 0).all()
    assert not torch.equal(qkv[:, :H * D], before[:, :H * D])  # q was rotated all the same


def test_decode_kernel_that_stores_the_new_key_itself_drops_a_bad_page():
    """The single-token kernel that rotates q and k and writes the token's key and value: the page
    of the new token is outside the pool, so nothing is written, bit 1 is set, and the token's own
    key is hidden like every key of such a page: the output is the attention over the older keys."""
    from dispec_b200.ops import attention as A
    H, KVH, D, page, ctx = 12, 2, 128, 16, 40
    g = torch.Generator().manual_seed(8)
    k = torch.randn(ctx - 1, KVH, D, generator=g).bfloat16().float()
    v = torch.randn(ctx - 1, KVH, D, generator=g).bfloat16().float()
    P = 5
    kp = torch.zeros((P + 1, KVH, page, D), dtype=torch.bfloat16, device=dev())
    vp = torch.zeros_like(kp)
    table = torch.tensor([[3, 0, P]], dtype=torch.int32, device=dev())  # position 39 lives on logical page 2
    for pos in range(32):  # the older keys of the two good pages; positions 32..38 would lie on the bad one
        kp[table[0, pos // page], :, pos % page] = k[pos].bfloat16().to(dev())
        vp[table[0, pos // page], :, pos % page] = v[pos].bfloat16().to(dev())
    qkv = (torch.randn(1, (H + 2 * KVH) * D, generator=g)).bfloat16().to(dev())
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))).to(dev())
    out = torch.empty((1, H * D), dtype=torch.bfloat16, device=dev())
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=dev())
    A.paged_attention_tiles(qkv, qkv.stride(0), kp[:P], vp[:P], table, i32([0, 1]), i32([ctx]), i32([0]), i32([0]), 1, 1,
                            out, H, KVH, D, 0, D ** -0.5, splits=1, fused_rope=(inv_freq, D, True))
    torch.cuda.synchronize()
    assert error_word() == BAD_PAGE
    assert (kp[P] == 0).all() and (vp[P] == 0).all()
    assert torch.isfinite(out.float()).all()
    # rotate q by hand and attend over the 32 keys of the two good pages (positions 0..31; 32..38 lie
    # on the bad page as well)
    import plain_qwen2 as plain
    cos, sin = plain.rope_tables(torch.tensor([ctx - 1]), D, 1e6)
    qr = plain.apply_rope(qkv[:, :H * D].float().cpu().view(1, H, D), cos, sin).to(torch.bfloat16).double()
    G = H // KVH
    ref = torch.empty(1, H, D, dtype=torch.float64)
    for j in range(H):
        sc = (qr[:, j] @ k[:32, j // G].double().T) * D ** -0.5
        ref[:, j] = torch.softmax(sc, dim=-1) @ v[:32, j // G].double()
    torch.testing.assert_close(out.float().cpu().view(1, H, D).double(), ref, atol=2e-2, rtol=2e-2)


def test_a_bounded_wait_that_runs_out_sets_its_bit_and_the_context_goes_on():
    """The kernels' own bounded wait on a barrier at which nothing arrives, with a limit of 300
    tries: the kernel returns, bit 4 is set, and ordinary kernels run afterwards."""
    from dispec_b200 import ops
    from dispec_b200.ops import library as L
    ran_out = torch.zeros(1, dtype=torch.int32, device=dev())
    assert error_word() == 0
    L.check(L.core().dsp_selftest_wait_limit(300, L.ptr(ran_out), L.stream_handle()))
    torch.cuda.synchronize()
    assert int(ran_out.item()) == 1
    with pytest.raises(ops.KernelError, match="a bounded wait ran out"):
        ops.raise_on_device_error("self test")
    assert error_word() == 0
    x = rnd((8, 1536), torch.bfloat16, 1)
    w = rnd((256, 1536), torch.bfloat16, 2, 0.05)
    torch.testing.assert_close(ops.linear(x, w).double(), x.double() @ w.double().T, atol=3e-2, rtol=3e-2)
    assert error_word() == 0
    assert L.core().dsp_selftest_wait_limit(0, L.ptr(ran_out), L.stream_handle()) != 0  # refused, with a message
    assert b"tries" in L.core().dsp_last_error()
