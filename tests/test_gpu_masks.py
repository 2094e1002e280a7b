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
