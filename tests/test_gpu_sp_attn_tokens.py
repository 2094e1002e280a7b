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
