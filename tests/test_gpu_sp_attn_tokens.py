"""GPU parity of the sp_attn operator (key-token lists at the reference granularity)."""
import pytest
import torch

from helpers import GOLDEN_CASES, OUT_MAX_ABS, OUT_MEAN_ABS, load_golden

pytestmark = pytest.mark.gpu


def _capi():
    from fgattn_tk_cuda_b200 import capi
    return capi


def _close(o, ref, mx=OUT_MAX_ABS, mean=OUT_MEAN_ABS):
    d = (o.float().cpu() - torch.as_tensor(ref).float().cpu()).abs()
    assert torch.isfinite(o.float()).all()
    assert d.max().item() <= mx, d.max().item()
    assert d.mean().item() <= mean, d.mean().item()


@pytest.mark.parametrize("S,D", [(1000, 128), (777, 64), (128, 128)])
def test_identity_and_permuted_lists_equal_dense(S, D):
    """All keys listed, in order and in random order, must reproduce dense attention
    (test/test_sparseattn_asyncgatherload_padded.cu:37-62, python/test/test_extension.py:65-88)."""
    capi = _capi()
    B, H = 1, 2
    g = torch.Generator().manual_seed(S)
    q, k, v = (torch.randn(B, H, S, D, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    dense = torch.empty_like(q)
    capi.full_attn(dense, q, k, v)
    nb, stride = (S + 127) // 128, 128 * ((S + 127) // 128)
    idx = torch.empty(B, H, nb, stride, dtype=torch.int32, device="cuda")
    cnt = torch.empty(B, H, nb, dtype=torch.int32, device="cuda")
    capi.all_index_mask(idx, cnt, B, H, nb, S)
    o = torch.full_like(q, float("nan"))
    capi.sp_attn(o, q, k, v, idx, cnt)
    capi.check()
    _close(o, dense, 8e-3, 5e-4)
    perm = torch.cat([torch.randperm(S, generator=g), torch.full((stride - S,), stride)]).to(torch.int32)
    idx2 = perm.cuda().expand(B, H, nb, stride).contiguous()
    o2 = torch.full_like(q, float("nan"))
    capi.sp_attn(o2, q, k, v, idx2, cnt)
    capi.check()
    _close(o2, dense, 8e-3, 5e-4)


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_threshold_token_lists_golden(name):
    """The reference's own token lists (blocksz 128) drive the gather kernel; output against the
    oracle's renormalising sparse attention."""
    from oracle import fgattn_oracle as orc
    capi = _capi()
    g = load_golden(name)
    q, k, v = (g[t].cuda() for t in "qkv")
    idx = torch.from_numpy(g["index_128"]).cuda().contiguous()
    cnt = torch.from_numpy(g["count_128"]).cuda().contiguous()
    o = torch.full_like(q, float("nan"))
    capi.sp_attn(o, q, k, v, idx, cnt)
    capi.check()
    _close(o, orc.sp_attn_tokens(g["q"], g["k"], g["v"], idx.cpu(), cnt.cpu(), 128))


def test_ragged_counts_empty_lists_and_bad_entries():
    from oracle import fgattn_oracle as orc
    capi = _capi()
    B, H, S, D = 1, 2, 900, 128
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(B, H, S, D, generator=g).to(torch.bfloat16) for _ in range(3))
    nb, stride = (S + 127) // 128, 1024
    idx = torch.full((B, H, nb, stride), stride, dtype=torch.int32)
    cnt = torch.zeros(B, H, nb, dtype=torch.int32)
    for h in range(H):
        for b in range(nb):
            n = int(torch.randint(0, 700, (1,), generator=g))
            if (h, b) == (0, 1):
                n = 0                                   # empty list -> zero rows
            sel = torch.randperm(S, generator=g)[:n].to(torch.int32)
            if n > 10:
                sel[5] = stride                         # out-of-range entry inside the count: ignored
            idx[0, h, b, :n] = sel
            cnt[0, h, b] = n
    o = torch.full((B, H, S, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.sp_attn(o, q.cuda(), k.cuda(), v.cuda(), idx.cuda(), cnt.cuda())
    capi.check()
    _close(o, orc.sp_attn_tokens(q, k, v, idx, cnt, 128))
    # the order in which the thread blocks take the query blocks changes nothing in the result
    o_st = torch.full_like(o, float("nan"))
    capi.sp_attn(o_st, q.cuda(), k.cuda(), v.cuda(), idx.cuda(), cnt.cuda(), ordered=False)
    capi.check()
    assert torch.equal(o_st, o)
    # with the block route switched on the well-filled lists go through whole tiles: same result within rounding
    capi.set_tuning("token_block_route", 1)
    try:
        o_b = torch.full_like(o, float("nan"))
        capi.sp_attn(o_b, q.cuda(), k.cuda(), v.cuda(), idx.cuda(), cnt.cuda(), block_route=True)
        capi.check()
    finally:
        capi.set_tuning("token_block_route", -1)
    _close(o_b, orc.sp_attn_tokens(q, k, v, idx, cnt, 128))


def _routes(capi, ws, B, H, S):
    """Route flags (1 = block route) that the call left in its workspace, per (unit, 128-row query block)."""
    small = (capi.sp_attn_workspace_bytes(B, H, S) + 255) // 256 * 256
    n_rows = B * H * ((S + 127) // 128)
    off = 2 * small + (n_rows * 4 + 255) // 256 * 256
    return ws[off:off + n_rows * 4].view(torch.int32).view(B * H, -1).cpu()


def _lists_from_mask(tm, stride):
    from oracle import fgattn_oracle as orc
    idx, cnt = orc.bitmask_to_indexmask(tm)
    out = torch.full((*idx.shape[:3], stride), stride, dtype=torch.int32)
    n = idx.shape[-1]
    out[..., :n] = torch.where(idx >= n, torch.full_like(idx, stride), idx)
    return out, cnt


@pytest.mark.parametrize("S,D,kv", [(1000, 128, None), (1500, 64, None), (640, 128, 900)])
def test_block_route_mixed_with_row_gather(S, D, kv):
    """Lists that fill the 64-key blocks they touch (what a threshold mask produces) go through whole
    K/V tiles with column masks, scattered lists and lists that name a token twice stay on the row
    gather -- in one call; every query block against the oracle."""
    from oracle import fgattn_oracle as orc
    capi = _capi()
    B, H = 1, 2
    n_kv = kv or S
    g = torch.Generator().manual_seed(S + D)
    q = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16)
    k, v = (torch.randn(B, H, n_kv, D, generator=g).to(torch.bfloat16) for _ in range(2))
    nb, nkb = (S + 127) // 128, (n_kv + 63) // 64
    stride = 128 * ((n_kv + 127) // 128)
    # block-structured mask: a third of the key blocks, 90 % of their columns (ragged last block included)
    blocks = torch.rand(B, H, nb, nkb, generator=g) < 0.35
    tm = blocks.repeat_interleave(64, dim=-1)[..., :n_kv] & (torch.rand(B, H, nb, n_kv, generator=g) < 0.9)
    tm[0, 0, 1] = torch.rand(n_kv, generator=g) < 0.08          # scattered list: row gather
    tm[0, 1, 0] = False                                         # empty list: zero rows
    idx, cnt = _lists_from_mask(tm, stride)
    dup_row = (0, 1, 2)
    n = int(cnt[dup_row])
    if n >= 2:
        idx[dup_row][n - 1] = idx[dup_row][0]                   # a token listed twice: row gather (counts twice)
    ref = orc.sp_attn_tokens(q, k, v, idx, cnt, 128)
    qc, kc, vc, idxc, cntc = q.cuda(), k.cuda(), v.cuda(), idx.cuda(), cnt.cuda()
    ws = torch.empty(capi.sp_attn_token_workspace_bytes(B, H, S, n_kv), dtype=torch.uint8, device="cuda")
    o = torch.full_like(qc, float("nan"))
    capi.set_tuning("token_block_route", 1)
    try:
        capi.sp_attn(o, qc, kc, vc, idxc, cntc, workspace=ws)
        capi.check()
    finally:
        capi.set_tuning("token_block_route", -1)
    _close(o, ref)
    routes = _routes(capi, ws, B, H, S)
    assert routes[0, 1] == 0 and routes[1, 0] == 0              # scattered / empty
    if n >= 2:
        assert routes[1, 2] == 0                                # duplicate
    assert routes.sum() >= 3                                    # well-filled lists took the block route
    # the row gather alone gives the same within rounding
    o_g = torch.full_like(qc, float("nan"))
    capi.sp_attn(o_g, qc, kc, vc, idxc, cntc, block_route=False)
    capi.check()
    _close(o_g, ref)
    assert (o.float() - o_g.float()).abs().max().item() <= 1.6e-2


def test_block_route_large_scores_rerun():
    """Query norms large enough that the sampled exponent hint misses some rows by more than the safe
    range: those query blocks are recomputed by the running-maximum kernel, result unchanged."""
    from oracle import fgattn_oracle as orc
    capi = _capi()
    B, H, S, D = 1, 1, 512, 128
    g = torch.Generator().manual_seed(4)
    q = (torch.randn(B, H, S, D, generator=g) * 12.0).to(torch.bfloat16)
    k = (torch.randn(B, H, S, D, generator=g) * 12.0).to(torch.bfloat16)
    v = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16)
    tm = torch.rand(B, H, 4, S, generator=g) < 0.95
    idx, cnt = _lists_from_mask(tm, S)
    ref = orc.sp_attn_tokens(q, k, v, idx, cnt, 128)
    ws = torch.empty(capi.sp_attn_token_workspace_bytes(B, H, S, S), dtype=torch.uint8, device="cuda")
    o = torch.full((B, H, S, D), float("nan"), dtype=torch.bfloat16, device="cuda")
    capi.set_tuning("token_block_route", 1)
    try:
        capi.sp_attn(o, q.cuda(), k.cuda(), v.cuda(), idx.cuda(), cnt.cuda(), workspace=ws)
        capi.check()
    finally:
        capi.set_tuning("token_block_route", -1)
    _close(o, ref)
    assert _routes(capi, ws, B, H, S).sum() == 4
