"""GPU parity of the 64x64 block pipeline through the C ABI: one-pass m/l + key-block lists, and
the gather sparse attention in both softmax modes."""
import numpy as np
import pytest
import torch

from helpers import GOLDEN_CASES, OUT_MAX_ABS, OUT_MEAN_ABS, TAU_REL, load_golden

pytestmark = pytest.mark.gpu


def _capi():
    from fgattn_tk_cuda_b200 import capi
    return capi


def _close(o, ref):
    d = (o.float().cpu() - torch.as_tensor(ref).float()).abs()
    assert torch.isfinite(o.float()).all()
    assert d.max().item() <= OUT_MAX_ABS, d.max().item()
    assert d.mean().item() <= OUT_MEAN_ABS, d.mean().item()


def lists_to_bitmap(idx, cnt, nkb):
    idx, cnt = idx.cpu().long(), cnt.cpu().long()
    B, H, nqb, stride = idx.shape
    bm = torch.zeros(B, H, nqb, nkb + 1, dtype=torch.bool)
    ar = torch.arange(stride)[None, None, None, :]
    live = ar < cnt[..., None]
    bm.scatter_(3, torch.where(live, idx, torch.full_like(idx, nkb)), True)
    return bm[..., :nkb]


def run_lists(q, k, tau, v=None, kv=None, scratch_heads=None, stride_extra=0):
    capi = _capi()
    B, H, S, D = q.shape
    n_kv = kv or S
    nqb, nkb = (S + 63) // 64, (n_kv + 63) // 64
    s_pad = 128 * ((S + 127) // 128)
    idx = torch.full((B, H, nqb, nkb + stride_extra), -5, device="cuda", dtype=torch.int32)
    cnt = torch.full((B, H, nqb), -5, device="cuda", dtype=torch.int32)
    m = torch.empty(B, H, 1, s_pad, device="cuda")
    l = torch.empty(B, H, 1, s_pad, device="cuda")
    nbytes = capi.block_scratch_bytes(B, H, S, n_kv)
    if scratch_heads:
        nbytes = nbytes // (B * H) * scratch_heads
    scratch = torch.empty(nbytes // 4, device="cuda", dtype=torch.float32)
    o = torch.full_like(q, float("nan")) if v is not None else None
    capi.block_index_lists(idx, cnt, m, l, q, k, tau, scratch, o=o, v=v, kv_seq_len=kv)
    capi.check()
    return idx, cnt, m, l, o


def check_lists(idx, cnt, q_cpu, k_cpu, tau, kv=None):
    """Bit-exact against the oracle except blocks whose score is within TAU_REL of tau."""
    from oracle import fgattn_oracle as orc
    pmax = orc.qk_block_pmax(q_cpu, k_cpu, 64, 64, kv_seq_len=kv)
    nkb = pmax.shape[-1]
    want = pmax > tau
    got = lists_to_bitmap(idx, cnt, nkb)
    diff = got ^ want
    exempt = orc.near_threshold(pmax, tau, TAU_REL)
    assert not (diff & ~exempt).any(), int((diff & ~exempt).sum())
    # list format: ascending, count, sentinel fill (checked on the GPU's own bitmap)
    ridx, rcnt = orc.bitmask_to_indexmask(got)
    stride = idx.shape[3]
    assert torch.equal(cnt.cpu(), rcnt)
    assert torch.equal(idx.cpu()[..., :nkb], ridx)
    if stride > nkb:
        assert torch.all(idx.cpu()[..., nkb:] == nkb)
    return got, int(diff.sum())


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_block_pipeline(name):
    from oracle import fgattn_oracle as orc
    capi = _capi()
    g = load_golden(name)
    q, k, v = (g[t].cuda() for t in "qkv")
    tau = g["tau"]
    S = q.shape[2]
    idx, cnt, m, l, o = run_lists(q, k, tau, v=v)
    got, _ = check_lists(idx, cnt, g["q"], g["k"], tau)
    _close(o, g["sdpa"])
    np.testing.assert_allclose(m[:, :, 0, :S].cpu().numpy(), g["max_q"], rtol=0, atol=2e-3)
    np.testing.assert_allclose(l[:, :, 0, :S].cpu().numpy(), g["denom"], rtol=2e-3, atol=0)
    # the 64x64 block map must be the OR over 64-key groups of the reference's blocksz-64 token map
    n = g["k"].shape[2]
    tok = torch.from_numpy(np.unpackbits(g["bitmask_64"], axis=-1)[..., :n].astype(bool))
    nkb = (n + 63) // 64
    want = torch.nn.functional.pad(tok, (0, nkb * 64 - n)).view(*tok.shape[:3], nkb, 64).any(-1)
    pmax = orc.qk_block_pmax(g["q"], g["k"])
    assert not ((got ^ want) & ~orc.near_threshold(pmax, tau, TAU_REL)).any()

    # masked attention with the precomputed m, l (no renormalisation)
    o_ml = torch.full_like(q, float("nan"))
    capi.sp_attn_blocks_ml(o_ml, q, k, v, idx, cnt, m, l)
    capi.check()
    _close(o_ml, orc.block_masked_attn(g["q"], g["k"], g["v"], got))
    # renormalising softmax over the kept blocks
    o_rn = torch.full_like(q, float("nan"))
    capi.sp_attn_blocks(o_rn, q, k, v, idx, cnt)
    capi.check()
    _close(o_rn, orc.sp_attn_blocks(g["q"], g["k"], g["v"], idx.cpu(), cnt.cpu()))


@pytest.mark.parametrize("B,H,S,D,kv", [(1, 2, 1000, 128, None), (2, 1, 1536, 64, None), (1, 2, 1024, 128, 779)])
def test_lists_only_and_chunked_scratch(B, H, S, D, kv):
    from fgattn_tk_cuda_b200 import synth
    w = synth.Workload("t", B, H, S, D, "clustered", centroids=8, run=64, tau=1e-3, seed=S + D)
    q, k, v = synth.make_qkv(w)
    qc, kc = q.cuda(), k.cuda()
    idx, cnt, m, l, _ = run_lists(qc, kc, w.tau, kv=kv, stride_extra=3)
    _, ndiff = check_lists(idx, cnt, q, k, w.tau, kv=kv)
    idx2, cnt2, m2, l2, _ = run_lists(qc, kc, w.tau, kv=kv, scratch_heads=1, stride_extra=3)
    assert torch.equal(idx, idx2) and torch.equal(cnt, cnt2) and torch.equal(m, m2) and torch.equal(l, l2)
    dens = cnt.float().mean().item() / idx.shape[3]
    assert 0.0 < dens < 0.9


@pytest.mark.parametrize("S,D,kv", [(640, 128, None), (1000, 64, None), (1000, 128, 900), (130, 128, None)])
def test_random_lists_both_modes(S, D, kv):
    """Arbitrary lists: empty ones, lists that differ between the two query blocks of a pair, odd
    union sizes, a ragged last block."""
    from oracle import fgattn_oracle as orc
    capi = _capi()
    B, H = 1, 2
    n_kv = kv or S
    nqb, nkb = (S + 63) // 64, (n_kv + 63) // 64
    g = torch.Generator().manual_seed(S + D)
    q, k, v = (torch.randn(B, H, S, D, generator=g).to(torch.bfloat16) for _ in range(3))
    bm = torch.rand(B, H, nqb, nkb, generator=g) < 0.35
    bm[0, 0, 0] = False                       # empty list
    if nqb > 3:
        bm[0, 1, 2] = False
        bm[0, 1, 3] = False                   # whole pair empty
        bm[0, 0, 1] = True                    # full list next to an empty one
    idx, cnt = orc.bitmask_to_indexmask(bm)
    qc, kc, vc, idxc, cntc = q.cuda(), k.cuda(), v.cuda(), idx.cuda(), cnt.cuda()
    s_pad = 128 * ((S + 127) // 128)
    m = torch.empty(B, H, 1, s_pad, device="cuda")
    l = torch.empty(B, H, 1, s_pad, device="cuda")
    capi.maxq_denom(m, l, qc, kc, kv_seq_len=kv)
    o_ml = torch.full_like(qc, float("nan"))
    capi.sp_attn_blocks_ml(o_ml, qc, kc, vc, idxc, cntc, m, l, kv_seq_len=kv)
    capi.check()
    _close(o_ml, orc.block_masked_attn(q, k, v, bm, kv_seq_len=kv))
    o_rn = torch.full_like(qc, float("nan"))
    capi.sp_attn_blocks(o_rn, qc, kc, vc, idxc, cntc, kv_seq_len=kv)
    capi.check()
    _close(o_rn, orc.sp_attn_blocks(q, k, v, idx, cnt, kv_seq_len=kv))
    # the order in which the thread blocks take the query blocks changes nothing in the result
    o_st = torch.full_like(qc, float("nan"))
    capi.sp_attn_blocks(o_st, qc, kc, vc, idxc, cntc, kv_seq_len=kv, ordered=False)
    capi.check()
    assert torch.equal(o_st, o_rn)


def test_identity_lists_equal_dense():
    """The reference's main sparse check: with every key listed the sparse kernel reproduces the
    dense one (test/test_sparseattn_asyncgatherload_padded.cu:37-62)."""
    capi = _capi()
    B, H, S, D = 1, 2, 1111, 128
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(B, H, S, D, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    nqb = nkb = (S + 63) // 64
    idx = torch.arange(nkb, dtype=torch.int32, device="cuda").expand(B, H, nqb, nkb).contiguous()
    cnt = torch.full((B, H, nqb), nkb, dtype=torch.int32, device="cuda")
    dense = torch.empty_like(q)
    s_pad = 128 * ((S + 127) // 128)
    m = torch.empty(B, H, 1, s_pad, device="cuda")
    l = torch.empty(B, H, 1, s_pad, device="cuda")
    capi.fullattn_maxq_denom(dense, m, l, q, k, v)
    for fn in ("ml", "rn"):
        o = torch.full_like(q, float("nan"))
        if fn == "ml":
            capi.sp_attn_blocks_ml(o, q, k, v, idx, cnt, m, l)
        else:
            capi.sp_attn_blocks(o, q, k, v, idx, cnt)
        capi.check()
        d = (o.float() - dense.float()).abs()
        assert d.max().item() <= 8e-3 and d.mean().item() <= 5e-4, (fn, d.max().item(), d.mean().item())


@pytest.mark.parametrize("group", [1, 2, 0])
def test_thread_block_order_with_several_head_groups(group):
    """The longest-first order is built per group of heads (the "group_heads" tuning knob overrides the
    group size; 0 = built-in choice); whatever the grouping, every item must be visited exactly once:
    same output as storage order."""
    from oracle import fgattn_oracle as orc
    capi = _capi()
    capi.set_tuning("group_heads", group)
    try:
        _order_case(capi, orc)
    finally:
        capi.set_tuning("group_heads", -1)


def _order_case(capi, orc):
    B, H, S, D = 1, 5, 1500, 64
    nqb = nkb = (S + 63) // 64
    g = torch.Generator().manual_seed(77)
    q, k, v = (torch.randn(B, H, S, D, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    dens = torch.rand(B, H, nqb, 1, generator=g)                     # list lengths from empty to full
    bm = torch.rand(B, H, nqb, nkb, generator=g) < dens
    idx, cnt = orc.bitmask_to_indexmask(bm)
    idx, cnt = idx.cuda(), cnt.cuda()
    o_st = torch.full_like(q, float("nan"))
    o_or = torch.full_like(q, float("nan"))
    capi.sp_attn_blocks(o_st, q, k, v, idx, cnt, ordered=False)
    capi.sp_attn_blocks(o_or, q, k, v, idx, cnt)
    capi.check()
    assert torch.equal(o_st, o_or)
    # token lists: the same block lists expanded to tokens, 128-row query blocks
    nb = (S + 127) // 128
    tm = bm[:, :, 0::2].repeat_interleave(64, dim=-1)[..., :S]
    tidx, tcnt = orc.bitmask_to_indexmask(tm)
    stride = 128 * ((tidx.shape[-1] + 127) // 128)
    pad = torch.full((B, H, nb, stride), stride, dtype=torch.int32)
    pad[..., :tidx.shape[-1]] = torch.where(tidx >= S, torch.full_like(tidx, stride), tidx)
    t_st = torch.full_like(q, float("nan"))
    t_or = torch.full_like(q, float("nan"))
    capi.sp_attn(t_st, q, k, v, pad.cuda(), tcnt.cuda(), ordered=False)
    capi.sp_attn(t_or, q, k, v, pad.cuda(), tcnt.cuda())
    capi.check()
    assert torch.equal(t_st, t_or)
    assert torch.isfinite(t_or.float()).all()


@pytest.mark.parametrize("S,D,kv", [(1000, 128, None), (1536, 64, 1400)])
def test_lists_for_another_threshold_from_kept_maxima(S, D, kv):
    """block_lists_from_maxima: the threshold step alone on the block maxima that block_index_lists left in a
    scratch sized for all units.  The same threshold gives the same lists; another threshold gives the lists of a
    fresh pass with that threshold."""
    from fgattn_tk_cuda_b200 import capi, synth
    w = synth.Workload("t", 2, 3, S, D, "clustered", centroids=10, run=80, tau=1e-3, seed=77)
    q, k, _ = synth.make_qkv(w, device="cuda")
    B, H = q.shape[:2]
    n_kv = kv or S
    nqb, nkb = (S + 63) // 64, (n_kv + 63) // 64
    s_pad = 128 * ((S + 127) // 128)
    def fresh(tau):
        idx = torch.full((B, H, nqb, nkb), -7, dtype=torch.int32, device="cuda")
        cnt = torch.full((B, H, nqb), -7, dtype=torch.int32, device="cuda")
        m = torch.empty(B, H, 1, s_pad, device="cuda")
        l = torch.empty_like(m)
        scratch = torch.empty(capi.block_scratch_bytes(B, H, S, n_kv) // 4, device="cuda")
        capi.block_index_lists(idx, cnt, m, l, q, k, tau, scratch, kv_seq_len=kv)
        capi.check()
        return idx, cnt, m, l, scratch
    idx, cnt, m, l, scratch = fresh(w.tau)
    for tau in (w.tau, 3e-2):
        idx2 = torch.full_like(idx, -9)
        cnt2 = torch.full_like(cnt, -9)
        capi.block_lists_from_maxima(idx2, cnt2, scratch, m, l, q.shape, tau, kv_seq_len=kv)
        capi.check()
        ref_idx, ref_cnt = (idx, cnt) if tau == w.tau else fresh(tau)[:2]
        assert torch.equal(cnt2, ref_cnt) and torch.equal(idx2, ref_idx)
        # the same through the torch operator
        import fgattn_tk_cuda_b200.spattn  # noqa: F401  (registers torch.ops.cuda_attn)
        idx3, cnt3 = torch.full_like(idx, -9), torch.full_like(cnt, -9)
        torch.ops.cuda_attn.block_lists_from_maxima(idx3, cnt3, scratch, m, l, S, D, n_kv, tau)
        assert torch.equal(cnt3, ref_cnt) and torch.equal(idx3, ref_idx)
    assert cnt2.sum().item() < cnt.sum().item()          # the higher threshold keeps fewer blocks
