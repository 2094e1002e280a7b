"""The renormalising block-sparse kernel with a per-row exponent hint (fgattn_sp_attn_blocks_hint)
through the C ABI: same results as the oracle's softmax over the kept keys whatever the hint is --
an exact one, a stale one, and hints so far off that rows overflow / underflow and their query blocks
go through the re-run pass."""
import pytest
import torch

from helpers import OUT_MAX_ABS, OUT_MEAN_ABS

pytestmark = pytest.mark.gpu


def _close(o, ref):
    d = (o.float().cpu() - torch.as_tensor(ref).float()).abs()
    assert torch.isfinite(o.float()).all()
    assert d.max().item() <= OUT_MAX_ABS, d.max().item()
    assert d.mean().item() <= OUT_MEAN_ABS, d.mean().item()


def _redo_flags(capi, ws, B, H, S):
    """The re-run flags sit behind the queue header and the item order in the workspace."""
    n_items = B * H * ((S + 127) // 128)
    return ws.view(torch.int32)[4 + n_items:4 + 2 * n_items]


def _case(S, D, kv, seed, scale_q=1.0):
    from oracle import fgattn_oracle as orc
    B, H = 1, 2
    n_kv = kv or S
    nqb, nkb = (S + 63) // 64, (n_kv + 63) // 64
    g = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(B, H, S, D, generator=g).to(torch.bfloat16) for _ in range(3))
    q = (q.float() * scale_q).to(torch.bfloat16)
    bm = torch.rand(B, H, nqb, nkb, generator=g) < 0.35
    bm[0, 0, 0] = False                       # empty list next to a listed one (rows with nothing kept -> 0)
    if nqb > 3:
        bm[0, 1, 2] = False
        bm[0, 1, 3] = False                   # whole pair empty
        bm[0, 0, 1] = True
    idx, cnt = orc.bitmask_to_indexmask(bm)
    return q, k, v, idx, cnt


@pytest.mark.parametrize("S,D,kv", [(640, 128, None), (1000, 64, None), (1000, 128, 900), (130, 128, None),
                                    (2048, 64, None)])
def test_hint_kernel_matches_oracle_for_any_hint(S, D, kv):
    from fgattn_tk_cuda_b200 import capi
    from oracle import fgattn_oracle as orc
    q, k, v, idx, cnt = _case(S, D, kv, seed=S + D)
    B, H = q.shape[:2]
    ref = orc.sp_attn_blocks(q, k, v, idx, cnt, kv_seq_len=kv)
    qc, kc, vc, idxc, cntc = q.cuda(), k.cuda(), v.cuda(), idx.cuda(), cnt.cuda()
    s_pad = 128 * ((S + 127) // 128)
    m = torch.empty(B, H, 1, s_pad, device="cuda")
    l = torch.empty(B, H, 1, s_pad, device="cuda")
    capi.maxq_denom(m, l, qc, kc, kv_seq_len=kv)                 # row maxima over ALL keys: an upper estimate
    c = (D ** -0.5) * 1.4426950408889634
    hints = {
        "max over all keys": (m, False),
        "stale (off by +-20 in the exponent)": (m + torch.where(torch.rand_like(m) < 0.5, -20.0, 20.0) / c, False),
        "zero": (torch.zeros_like(m), False),
        "far too high (underflow)": (m + 300.0 / c, True),
        "far too low (overflow)": (m - 300.0 / c, True),
        "NaN": (torch.full_like(m, float("nan")), True),
    }
    for name, (hint, must_redo) in hints.items():
        o = torch.full_like(qc, float("nan"))
        ws = capi.sp_attn_blocks_hint(o, qc, kc, vc, idxc, cntc, hint.contiguous(), kv_seq_len=kv)
        capi.check()
        _close(o, ref)
        redo = int(_redo_flags(capi, ws, B, H, S).sum().item())
        if must_redo:
            assert redo > 0, name
        elif name != "zero":
            assert redo == 0, (name, redo)
    # same bits as the running-maximum kernel would be too strict (different summation order), but the
    # two renormalising kernels must agree closely
    o_rn = torch.full_like(qc, float("nan"))
    capi.sp_attn_blocks(o_rn, qc, kc, vc, idxc, cntc, kv_seq_len=kv)
    o_h = torch.full_like(qc, float("nan"))
    capi.sp_attn_blocks_hint(o_h, qc, kc, vc, idxc, cntc, m, kv_seq_len=kv)
    capi.check()
    assert (o_rn.float() - o_h.float()).abs().max().item() <= 1.6e-2


def test_hint_kernel_partial_redo_with_large_scores():
    """Large query norms (scores in the hundreds): a hint that is right for one head and far off for
    the other re-runs only the second head's items."""
    from fgattn_tk_cuda_b200 import capi
    from oracle import fgattn_oracle as orc
    S, D = 768, 128
    q, k, v, idx, cnt = _case(S, D, None, seed=5, scale_q=6.0)
    ref = orc.sp_attn_blocks(q, k, v, idx, cnt)
    qc, kc, vc, idxc, cntc = q.cuda(), k.cuda(), v.cuda(), idx.cuda(), cnt.cuda()
    m = torch.empty(1, 2, 1, S, device="cuda")
    l = torch.empty_like(m)
    capi.maxq_denom(m, l, qc, kc)
    c = (D ** -0.5) * 1.4426950408889634
    hint = m.clone()
    hint[0, 1] += 400.0 / c
    o = torch.full_like(qc, float("nan"))
    ws = capi.sp_attn_blocks_hint(o, qc, kc, vc, idxc, cntc, hint)
    capi.check()
    _close(o, ref)
    flags = _redo_flags(capi, ws, 1, 2, S).view(2, -1)
    assert int(flags[0].sum().item()) == 0
    assert int(flags[1].sum().item()) > 0


def test_cached_block_mask_replay_uses_the_hint_kernel():
    """cached_attn_cuda in the 64x64 mode keeps max_q with the cached lists and the replay step hands
    it to sp_attn_blocks_hint (python/spattn/sparseattn_functionals.py:95-113 is the flow)."""
    from fgattn_tk_cuda_b200 import synth
    from fgattn_tk_cuda_b200.spattn import mask_utils as mu, sparseattn_functionals as sf
    from oracle import fgattn_oracle as orc
    w = synth.Workload("t", 1, 2, 1100, 128, "clustered", centroids=16, run=128, tau=1e-4, seed=91)
    q, k, v = synth.make_qkv(w, device="cuda")
    cache = mu.NaiveMaskCache([0])
    sf.cached_attn_cuda(q, k, v, 0, 0, thresh=w.tau, blocksz=64, mask_cache=cache)
    assert len(cache.get_mask_from_cache(0)) == 3
    q2 = (q.float() * 1.05 + 0.02).to(torch.bfloat16)
    k2 = (k.float() * 0.97).to(torch.bfloat16)
    o1 = sf.cached_attn_cuda(q2, k2, v, 0, 1, thresh=w.tau, blocksz=64, mask_cache=cache)
    idx, cnt = cache.get_mask_from_cache(0)[:2]
    _close(o1, orc.sp_attn_blocks(q2.cpu(), k2.cpu(), v.cpu(), idx.cpu(), cnt.cpu()))
    o2 = sf.sparse_attn_from_cache_cuda(q2, k2, v, mask_cache=cache, current_layer=0, blocksz=64)
    assert torch.equal(o1, o2)


def test_half_index_lists_entry_point():
    """attn_2xmask_cuda (python/spattn/sparseattn_functionals.py:137-153): every other key."""
    from fgattn_tk_cuda_b200.spattn import mask_utils as mu, sparseattn_functionals as sf
    from oracle import fgattn_oracle as orc
    g = torch.Generator().manual_seed(12)
    q, k, v = (torch.randn(1, 2, 640, 128, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    o = sf.attn_2xmask_cuda(q, k, v, 0, 0, blocksz=128)
    idx, cnt = mu.halfindex_mask(1, 2, 640, 128)
    _close(o, orc.sp_attn_tokens(q.cpu(), k.cpu(), v.cpu(), idx.cpu(), cnt.cpu(), 128))
