"""Key / value tensors whose length differs from the query length (kv_rows != seq) through every
entry point that takes k / v, plus kv_seq_len < kv_rows on top.  The reference only has the
same-length case with a shorter kv_seq_len hard-coded per shape (python/cuda_attn.cu:28-31)."""
import pytest
import torch

from helpers import OUT_MAX_ABS, OUT_MEAN_ABS, TAU_REL

pytestmark = pytest.mark.gpu

SHAPES = [  # B, H, S_q, S_kv, D, kv_seq_len
    (1, 3, 300, 520, 128, None),
    (2, 2, 512, 200, 64, None),
    (1, 2, 257, 1000, 128, 777),
    (1, 2, 640, 130, 64, 100),
    (1, 2, 300, 2500, 64, 2345),       # more than 2048 keys: the one-item kernels of the max / denominator pass
]


def _capi():
    from fgattn_tk_cuda_b200 import capi
    return capi


def _close(o, ref):
    d = (o.float().cpu() - torch.as_tensor(ref).float()).abs()
    assert torch.isfinite(o.float()).all()
    assert d.max().item() <= OUT_MAX_ABS, d.max().item()
    assert d.mean().item() <= OUT_MEAN_ABS, d.mean().item()


def _inputs(B, H, S, Skv, D, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, H, Skv, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, H, Skv, D, generator=g).to(torch.bfloat16)
    return q, k, v


@pytest.mark.parametrize("B,H,S,Skv,D,kv", SHAPES)
def test_dense_family(B, H, S, Skv, D, kv):
    from oracle import fgattn_oracle as orc
    capi = _capi()
    q, k, v = _inputs(B, H, S, Skv, D, S + Skv)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    s_pad = 128 * ((S + 127) // 128)
    o = torch.full_like(qc, float("nan"))
    capi.full_attn(o, qc, kc, vc, kv_seq_len=kv)
    ref = orc.full_attn(q, k, v, kv_seq_len=kv)
    _close(o, ref)
    o2 = torch.full_like(qc, float("nan"))
    m = torch.empty(B, H, 1, s_pad, device="cuda")
    l = torch.empty_like(m)
    capi.fullattn_maxq_denom(o2, m, l, qc, kc, vc, kv_seq_len=kv)
    m2, l2 = torch.empty_like(m), torch.empty_like(m)
    capi.maxq_denom(m2, l2, qc, kc, kv_seq_len=kv)
    capi.check()
    assert torch.equal(o, o2)
    rm, rl = orc.maxq_denom(q, k, kv_seq_len=kv)
    for mm, ll in ((m, l), (m2, l2)):
        assert (mm[..., :S].cpu() - rm[..., :S]).abs().max() <= 2e-3
        assert ((ll[..., :S].cpu() - rl[..., :S]).abs() / rl[..., :S]).max() <= 2e-3


@pytest.mark.parametrize("B,H,S,Skv,D,kv", [(1, 4, 15000, 300, 64, None), (2, 3, 13000, 1024, 128, 1000),
                                             (1, 5, 9999, 128, 128, None)])
def test_few_keys_many_query_tiles(B, H, S, Skv, D, kv):
    """Up to 1024 keys the dense family runs persistent CTAs that walk several (unit, query tile pair)
    items each; these shapes have more items than the GPU has SMs."""
    from oracle import fgattn_oracle as orc
    capi = _capi()
    assert B * H * ((S + 255) // 256) > torch.cuda.get_device_properties(0).multi_processor_count
    q, k, v = _inputs(B, H, S, Skv, D, S + 3 * Skv)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    s_pad = 128 * ((S + 127) // 128)
    o = torch.full_like(qc, float("nan"))
    capi.full_attn(o, qc, kc, vc, kv_seq_len=kv)
    o2 = torch.full_like(qc, float("nan"))
    m = torch.full((B, H, 1, s_pad), float("nan"), device="cuda")
    l = torch.full_like(m, float("nan"))
    capi.fullattn_maxq_denom(o2, m, l, qc, kc, vc, kv_seq_len=kv)
    m2, l2 = torch.full_like(m, float("nan")), torch.full_like(m, float("nan"))
    capi.maxq_denom(m2, l2, qc, kc, kv_seq_len=kv)
    capi.check()
    _close(o, orc.full_attn(q, k, v, kv_seq_len=kv))
    assert torch.equal(o, o2)
    rm, rl = orc.maxq_denom(q, k, kv_seq_len=kv)
    for mm, ll in ((m, l), (m2, l2)):
        assert (mm[..., :S].cpu() - rm[..., :S]).abs().max() <= 2e-3
        assert ((ll[..., :S].cpu() - rl[..., :S]).abs() / rl[..., :S]).max() <= 2e-3
        assert (mm[..., S:] == 0).all() and torch.isinf(ll[..., S:]).all()


@pytest.mark.parametrize("B,H,S,Skv,D,kv", SHAPES)
def test_block_pipeline(B, H, S, Skv, D, kv):
    from oracle import fgattn_oracle as orc
    capi = _capi()
    q, k, v = _inputs(B, H, S, Skv, D, 7 * S + Skv)
    q = (q.float() * 1.5).to(torch.bfloat16)                   # peakier rows: a real mix of kept / dropped blocks
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    n_kv = kv or Skv
    pmax = orc.qk_block_pmax(q, k, 64, 64, kv_seq_len=kv)
    tau = float(pmax.median())                                  # about half of the blocks kept
    nqb, nkb = (S + 63) // 64, (n_kv + 63) // 64
    s_pad = 128 * ((S + 127) // 128)
    idx = torch.full((B, H, nqb, nkb), -5, device="cuda", dtype=torch.int32)
    cnt = torch.full((B, H, nqb), -5, device="cuda", dtype=torch.int32)
    m = torch.empty(B, H, 1, s_pad, device="cuda")
    l = torch.empty_like(m)
    scratch = torch.empty(capi.block_scratch_bytes(B, H, S, n_kv) // 4, device="cuda")
    o = torch.full_like(qc, float("nan"))
    capi.block_index_lists(idx, cnt, m, l, qc, kc, tau, scratch, o=o, v=vc, kv_seq_len=kv)
    capi.check()
    _close(o, orc.full_attn(q, k, v, kv_seq_len=kv))
    live = torch.arange(nkb)[None, None, None, :] < cnt.cpu()[..., None]
    got = torch.zeros(B, H, nqb, nkb + 1, dtype=torch.bool)
    got.scatter_(3, torch.where(live, idx.cpu().long(), torch.full_like(idx.cpu().long(), nkb)), True)
    got = got[..., :nkb]
    bad = (got ^ (pmax > tau)) & ~orc.near_threshold(pmax, tau, TAU_REL)
    assert not bad.any(), int(bad.sum())
    assert 0 < int(got.sum()) < got.numel()
    o_ml = torch.full_like(qc, float("nan"))
    capi.sp_attn_blocks_ml(o_ml, qc, kc, vc, idx, cnt, m, l, kv_seq_len=kv)
    o_rn = torch.full_like(qc, float("nan"))
    capi.sp_attn_blocks(o_rn, qc, kc, vc, idx, cnt, kv_seq_len=kv)
    capi.check()
    _close(o_ml, orc.block_masked_attn(q, k, v, got, kv_seq_len=kv))
    _close(o_rn, orc.sp_attn_blocks(q, k, v, idx.cpu(), cnt.cpu(), kv_seq_len=kv))


@pytest.mark.parametrize("B,H,S,Skv,D,kv", SHAPES[:3])
def test_token_path_and_topk(B, H, S, Skv, D, kv):
    from oracle import fgattn_oracle as orc
    capi = _capi()
    q, k, v = _inputs(B, H, S, Skv, D, 3 * S + Skv)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    n_kv = kv or Skv
    nblk = (S + 127) // 128
    sel = max(1, n_kv // 5)
    stride = 128 * ((sel + 127) // 128)
    idx = torch.full((B, H, nblk, stride), -1, dtype=torch.int32, device="cuda")
    cnt = torch.full((B, H, nblk), -1, dtype=torch.int32, device="cuda")
    capi.topk_indices(idx, cnt, qc, kc, sel, blocksz=128, kv_seq_len=kv)
    capi.check()
    ridx, rcnt = orc.topk_indices(q, k, sel, 128, kv_seq_len=kv)
    assert torch.equal(cnt.cpu(), rcnt)
    # same key sets (order may differ between near-equal scores)
    a = torch.sort(idx[..., :sel].cpu(), dim=-1).values
    b = torch.sort(ridx, dim=-1).values
    assert (a != b).float().mean().item() < 0.01
    assert int(idx[..., :sel].max()) < n_kv
    o = torch.full_like(qc, float("nan"))
    capi.sp_attn(o, qc, kc, vc, idx, cnt)
    capi.check()
    _close(o, orc.sp_attn_tokens(q, k, v, idx.cpu(), cnt.cpu(), 128))
    # the threshold mask at the reference granularity
    s_pad = 128 * ((S + 127) // 128)
    m = torch.empty(B, H, 1, s_pad, device="cuda")
    l = torch.empty_like(m)
    capi.maxq_denom(m, l, qc, kc, kv_seq_len=kv)
    mstride = 128 * ((n_kv + 127) // 128)
    mask = torch.full((B, H, nblk, mstride), 7, dtype=torch.int32, device="cuda")
    tau = 4.0 / n_kv
    capi.booleanmask_128(mask, m, l, qc, kc, tau, kv_seq_len=kv)
    capi.check()
    pm = orc.qk_token_pmax(q, k, 128, kv_seq_len=kv)
    got = mask[..., :n_kv].cpu() > 0
    bad = (got ^ (pm > tau)) & ~orc.near_threshold(pm, tau, TAU_REL)
    assert not bad.any(), int(bad.sum())
    assert not (mask[..., n_kv:] != 0).any()


def test_operator_boundary_takes_shorter_keys():
    """Through torch.ops.cuda_attn the k / v length comes from the tensors themselves."""
    import fgattn_tk_cuda_b200.spattn  # noqa: F401  registers the operators
    from oracle import fgattn_oracle as orc
    q, k, v = _inputs(2, 3, 384, 139, 128, 5)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    o = torch.empty_like(qc)
    torch.ops.cuda_attn.full_attn(o, qc, kc, vc)
    _close(o, orc.full_attn(q, k, v))
    m = torch.empty(2, 3, 1, 384, device="cuda")
    l = torch.empty_like(m)
    torch.ops.cuda_attn.fullattn_maxq_denom(o, m, l, qc, kc, vc)
    rm, rl = orc.maxq_denom(q, k)
    assert (m.cpu() - rm).abs().max() <= 2e-3 and ((l.cpu() - rl).abs() / rl).max() <= 2e-3
