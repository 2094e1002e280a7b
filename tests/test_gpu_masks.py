"""GPU parity of the integer mask kernels and of the reference-granularity threshold mask."""
import numpy as np
import pytest
import torch

from helpers import GOLDEN, GOLDEN_CASES, TAU_REL, load_golden

pytestmark = pytest.mark.gpu


def _capi():
    from fgattn_tk_cuda_b200 import capi
    return capi


@pytest.mark.parametrize("B,H,SB,stride,seq,dens", [(1, 2, 3, 384, 384, 0.3), (2, 1, 5, 1280, 1201, 0.05),
                                                     (1, 1, 2, 37, 30, 0.5), (1, 1, 4, 4096, 4096, 0.0),
                                                     (1, 1, 4, 2048, 2048, 1.0)])
def test_mask_to_index(B, H, SB, stride, seq, dens):
    from oracle import fgattn_oracle as orc
    capi = _capi()
    g = torch.Generator().manual_seed(stride)
    mask = (torch.rand(B, H, SB, stride, generator=g) < dens).to(torch.int32) * torch.randint(1, 9, (B, H, SB, stride), generator=g, dtype=torch.int32)
    idx = torch.full((B, H, SB, stride), -1, dtype=torch.int32, device="cuda")
    cnt = torch.full((B, H, SB), -1, dtype=torch.int32, device="cuda")
    capi.booleanmask_to_indexmask(idx, cnt, mask.cuda(), seq)
    capi.check()
    live = mask.clone()
    live[..., seq:] = 0
    ridx, rcnt = orc.bitmask_to_indexmask(live)
    assert torch.equal(cnt.cpu(), rcnt) and torch.equal(idx.cpu(), ridx)


def test_compaction_golden_fixture():
    capi = _capi()
    z = np.load(GOLDEN / "compaction_9x37.npz")
    mask = torch.from_numpy(z["mask"].astype(np.int32))[None, None].cuda()
    idx = torch.empty(1, 1, 9, 37, dtype=torch.int32, device="cuda")
    cnt = torch.empty(1, 1, 9, dtype=torch.int32, device="cuda")
    capi.booleanmask_to_indexmask(idx, cnt, mask, 37)
    capi.check()
    assert np.array_equal(idx[0, 0].cpu().numpy(), z["index"]) and np.array_equal(cnt[0, 0].cpu().numpy(), z["count"])


def test_all_index_mask():
    from oracle import fgattn_oracle as orc
    capi = _capi()
    B, H, S, stride = 2, 3, 1000, 1024
    nb = (S + 127) // 128
    idx = torch.empty(B, H, nb, stride, dtype=torch.int32, device="cuda")
    cnt = torch.empty(B, H, nb, dtype=torch.int32, device="cuda")
    capi.all_index_mask(idx, cnt, B, H, nb, S)
    capi.check()
    ridx, rcnt = orc.allindex_mask(B, H, stride, S, 128)
    assert torch.equal(idx.cpu(), ridx) and torch.equal(cnt.cpu(), rcnt)


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_booleanmask_128_golden(name):
    """Token mask at the reference granularity against the reference's own qk_bitmask output."""
    from oracle import fgattn_oracle as orc
    capi = _capi()
    g = load_golden(name)
    q, k = g["q"].cuda(), g["k"].cuda()
    B, H, S, D = q.shape
    tau = g["tau"]
    s_pad = 128 * ((S + 127) // 128)
    m = torch.empty(B, H, 1, s_pad, device="cuda")
    l = torch.empty(B, H, 1, s_pad, device="cuda")
    capi.maxq_denom(m, l, q, k)
    nqb = (S + 127) // 128
    mask = torch.full((B, H, nqb, s_pad), 3, dtype=torch.int32, device="cuda")
    capi.booleanmask_128(mask, m, l, q, k, tau)
    capi.check()
    got = mask.cpu()[..., :S] > 0
    assert torch.all(mask.cpu()[..., S:] == 0)
    want = torch.from_numpy(np.unpackbits(g["bitmask_128"], axis=-1)[..., :S].astype(bool))
    pmax = orc.qk_token_pmax(g["q"], g["k"], 128)
    bad = (got ^ want) & ~orc.near_threshold(pmax, tau, TAU_REL)
    assert not bad.any(), int(bad.sum())
    # and through the compaction: same lists as the reference's qk_indexmask where masks agree
    idx = torch.empty(B, H, nqb, s_pad, dtype=torch.int32, device="cuda")
    cnt = torch.empty(B, H, nqb, dtype=torch.int32, device="cuda")
    capi.booleanmask_to_indexmask(idx, cnt, mask, S)
    capi.check()
    if not (got ^ want).any():
        assert np.array_equal(cnt.cpu().numpy(), g["count_128"])
        ref = g["index_128"].copy()
        ref[ref == S] = s_pad                       # sentinel = list width (mask_stride here)
        assert np.array_equal(idx.cpu().numpy()[..., :S], ref)


@pytest.mark.parametrize("S,D,kv", [(1024, 128, None), (900, 64, None), (1536, 128, 1400)])
def test_token_mask_inside_kept_blocks(S, D, kv):
    """booleanmask_128_listed: the token mask computed only inside the 64x64 blocks that the one-pass
    block lists kept.  Checked against the oracle like booleanmask_128, and against booleanmask_128
    itself (they may differ only on tokens within rounding of the threshold)."""
    from fgattn_tk_cuda_b200 import synth
    from oracle import fgattn_oracle as orc
    capi = _capi()
    w = synth.Workload("t", 1, 3, S, D, "clustered", centroids=12, run=96, tau=2e-3, seed=31)
    q, k, _ = synth.make_qkv(w, device="cuda")
    B, H = q.shape[:2]
    n_kv = kv or S
    nqb, nkb, nblk = (S + 63) // 64, (n_kv + 63) // 64, (S + 127) // 128
    s_pad = 128 * ((S + 127) // 128)
    idx = torch.empty(B, H, nqb, nkb, dtype=torch.int32, device="cuda")
    cnt = torch.empty(B, H, nqb, dtype=torch.int32, device="cuda")
    m = torch.empty(B, H, 1, s_pad, device="cuda")
    l = torch.empty_like(m)
    scratch = torch.empty(capi.block_scratch_bytes(B, H, S, n_kv) // 4, device="cuda")
    capi.block_index_lists(idx, cnt, m, l, q, k, w.tau, scratch, kv_seq_len=kv)
    mstride = 128 * ((n_kv + 127) // 128)
    listed = torch.full((B, H, nblk, mstride), 9, dtype=torch.int32, device="cuda")
    plain = torch.full_like(listed, 9)
    capi.booleanmask_128_listed(listed, m, l, q, k, w.tau, idx, cnt, kv_seq_len=kv)
    capi.booleanmask_128(plain, m, l, q, k, w.tau, kv_seq_len=kv)
    capi.check()
    dens = cnt.sum().item() / (B * H * nqb * nkb)
    assert 0.02 < dens < 0.9, dens                       # the lists really skip something
    pm = orc.qk_token_pmax(q.cpu(), k.cpu(), 128, kv_seq_len=kv)
    near = orc.near_threshold(pm, w.tau, TAU_REL)
    for got in (listed, plain):
        g = got[..., :n_kv].cpu() > 0
        assert not ((g ^ (pm > w.tau)) & ~near).any()
        assert not (got[..., n_kv:] != 0).any()
    diff = (listed[..., :n_kv].cpu() > 0) ^ (plain[..., :n_kv].cpu() > 0)
    assert not (diff & ~near).any()
    # the mask over all key tiles has two kernels (two threads per row by default, "maxq_wide" = 0: the dense
    # family's mode); same comparison against the same threshold, so the same mask bit for bit
    narrow = torch.full_like(listed, 9)
    capi.set_tuning("maxq_wide", 0)
    try:
        capi.booleanmask_128(narrow, m, l, q, k, w.tau, kv_seq_len=kv)
        capi.check()
    finally:
        capi.set_tuning("maxq_wide", -1)
    assert torch.equal(narrow, plain)
    # thread blocks in storage order instead of longest lists first: the same mask
    unordered = torch.full_like(listed, 9)
    capi.booleanmask_128_listed(unordered, m, l, q, k, w.tau, idx, cnt, kv_seq_len=kv, ordered=False)
    capi.check()
    assert torch.equal(unordered, listed)


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_python_mask_pipeline_reference_granularity(name):
    """spattn.mask_utils.qk_bitmask_cuda / qk_indexmask_cuda (blocksz 128) against the reference's own
    qk_bitmask / qk_indexmask outputs (python/spattn/mask_utils.py:206-245), and the model-facing
    entry points with a token-list cache against the oracle's renormalising sparse attention."""
    from helpers import unpack_bitmask, OUT_MAX_ABS, OUT_MEAN_ABS
    from fgattn_tk_cuda_b200.spattn import mask_utils as mu, sparseattn_functionals as sf
    from oracle import fgattn_oracle as orc
    g = load_golden(name)
    q, k, v = g["q"].cuda(), g["k"].cuda(), g["v"].cuda()
    S, tau = q.shape[2], g["tau"]
    want = unpack_bitmask(g["bitmask_128"], S)
    pm = orc.qk_token_pmax(g["q"], g["k"], 128)
    near = orc.near_threshold(pm, tau, TAU_REL)
    got = mu.qk_bitmask_cuda(q, k, tau, blocksz=128)[..., :S].cpu()
    assert not ((got ^ want) & ~near).any()
    idx, cnt = mu.qk_indexmask_cuda(q, k, tau, blocksz=128)
    ridx, rcnt = orc.bitmask_to_indexmask(got)
    live = torch.arange(S)[None, None, None, :] < rcnt[..., None]
    assert torch.equal(cnt.cpu(), rcnt) and torch.equal(idx.cpu()[..., :S][live], ridx[live])
    assert (idx.cpu()[..., :S][~live] == idx.shape[3]).all()          # unused slots = list stride
    if not (got ^ want).any():                           # no near-threshold flips: bit-exact with the reference
        ref_idx = torch.from_numpy(g["index_128"])
        assert torch.equal(cnt.cpu(), torch.from_numpy(g["count_128"])) and torch.equal(ridx[live], ref_idx[live])
    for fn, cache in ((sf.cached_attn_cuda, mu.NaiveMaskCache([0])), (sf.bitmaskcached_attn_cuda, mu.CompressedBitMaskCache([0]))):
        o0 = fn(q, k, v, 0, 0, thresh=tau, blocksz=128, mask_cache=cache)
        d = (o0.float().cpu() - torch.from_numpy(g["sdpa"])).abs()
        assert d.max() < OUT_MAX_ABS and d.mean() < OUT_MEAN_ABS
        o1 = fn(q, k, v, 0, 1, thresh=tau, blocksz=128, mask_cache=cache)
        ci, cc = cache.get_mask_from_cache(0)[:2]
        ref = orc.sp_attn_tokens(g["q"], g["k"], g["v"], ci.cpu(), cc.cpu(), 128)
        d = (o1.float().cpu() - ref).abs()
        assert d.max() < OUT_MAX_ABS and d.mean() < OUT_MEAN_ABS
