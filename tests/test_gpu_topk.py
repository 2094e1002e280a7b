"""GPU parity of the top-k key selector (python/spattn/mask_utils.py:389-417 of the reference)."""
import numpy as np
import pytest
import torch

from helpers import GOLDEN, OUT_MAX_ABS, OUT_MEAN_ABS

pytestmark = pytest.mark.gpu

# Scores are fp32 sums of 64..128 products on both sides but in different orders, so two keys whose
# scores differ by less than this (relative to the score scale) may swap places.
SCORE_TOL = 2e-5


def _capi():
    from fgattn_tk_cuda_b200 import capi
    return capi


def _check_lists(idx, cnt, scores, select_k, n_valid):
    """idx [R, stride], cnt [R] from the GPU against fp32 oracle scores [R, n]: exactly select_k
    distinct valid keys; every listed key scores at least the oracle's k-th largest minus the
    tolerance and every unlisted one at most that plus the tolerance; listed in descending order."""
    R = scores.shape[0]
    assert (cnt == select_k).all()
    tol = SCORE_TOL * max(1.0, float(scores.abs().max()))
    kth = torch.sort(scores, dim=-1, descending=True).values[:, select_k - 1]
    for r in range(R):
        sel = idx[r, :select_k].long()
        assert sel.min() >= 0 and sel.max() < n_valid
        assert sel.unique().numel() == select_k
        s_sel = scores[r, sel]
        assert (s_sel >= kth[r] - tol).all()
        rest = torch.ones(scores.shape[1], dtype=torch.bool)
        rest[sel] = False
        assert (scores[r, rest] <= kth[r] + tol).all()
        assert (s_sel[1:] <= s_sel[:-1] + tol).all()
        assert (idx[r, select_k:] == idx.shape[1]).all()


def test_topk_golden_fixture():
    """The fixture made by the reference (ragged last query block); random normal inputs have no
    near-ties at this size, so the lists must match index for index."""
    capi = _capi()
    z = np.load(GOLDEN / "topk_s300_d64_k40.npz")
    q = torch.from_numpy(z["q_bf16"]).view(torch.bfloat16).cuda()
    k = torch.from_numpy(z["k_bf16"]).view(torch.bfloat16).cuda()
    K = int(z["select_k"])
    idx = torch.full((1, 2, 3, 128), -1, dtype=torch.int32, device="cuda")
    cnt = torch.full((1, 2, 3), -1, dtype=torch.int32, device="cuda")
    capi.topk_indices(idx, cnt, q, k, K, blocksz=128)
    capi.check()
    assert np.array_equal(cnt.cpu().numpy(), z["count"])
    assert np.array_equal(idx[..., :K].cpu().numpy(), z["index"])
    assert (idx[..., K:] == 128).all()


@pytest.mark.parametrize("B,H,S,D,blocksz,select_k,kv", [(1, 2, 1024, 128, 128, 100, None), (2, 1, 777, 64, 128, 64, None),
                                                        (1, 1, 2048, 128, 64, 1, None), (1, 2, 1500, 128, 128, 1500, None),
                                                        (1, 1, 4096, 64, 128, 3000, 4000), (1, 3, 640, 128, 256, 333, 600)])
def test_topk_vs_oracle(B, H, S, D, blocksz, select_k, kv):
    from oracle import fgattn_oracle as orc
    capi = _capi()
    g = torch.Generator().manual_seed(S + select_k)
    q = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, H, S, D, generator=g).to(torch.bfloat16)
    nblk = (S + blocksz - 1) // blocksz
    stride = 128 * ((select_k + 127) // 128)
    idx = torch.full((B, H, nblk, stride), -1, dtype=torch.int32, device="cuda")
    cnt = torch.full((B, H, nblk), -1, dtype=torch.int32, device="cuda")
    capi.topk_indices(idx, cnt, q.cuda(), k.cuda(), select_k, blocksz=blocksz, kv_seq_len=kv)
    capi.check()
    sc = orc.topk_scores(q, k, blocksz, kv_seq_len=kv)
    _check_lists(idx.cpu().view(-1, stride), cnt.cpu().view(-1), sc.reshape(-1, sc.shape[-1]), select_k, kv or S)


def test_topk_ties_take_the_smallest_indices():
    """All keys equal: every score ties, so the list is 0 .. select_k-1 in order."""
    capi = _capi()
    B, H, S, D, K = 1, 1, 512, 64, 37
    q = torch.randn(B, H, S, D).to(torch.bfloat16).cuda()
    k = torch.ones(B, H, S, D, dtype=torch.bfloat16, device="cuda")
    idx = torch.empty(B, H, 4, 128, dtype=torch.int32, device="cuda")
    cnt = torch.empty(B, H, 4, dtype=torch.int32, device="cuda")
    capi.topk_indices(idx, cnt, q, k, K, blocksz=128)
    capi.check()
    assert torch.equal(idx[..., :K].cpu(), torch.arange(K, dtype=torch.int32).expand(B, H, 4, K))


def test_topk_attention_flow():
    """attn_topkmask_cuda (python/spattn/sparseattn_functionals.py:39-48): top-k lists into the
    token-list sparse kernel; select_k = S keeps every key, i.e. dense attention."""
    from fgattn_tk_cuda_b200.spattn import sparseattn_functionals as sf, mask_utils as mu
    from oracle import fgattn_oracle as orc
    g = torch.Generator().manual_seed(3)
    B, H, S, D = 1, 2, 640, 128
    q, k, v = (torch.randn(B, H, S, D, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    o = sf.attn_topkmask_cuda(q, k, v, 0, 0, select_k=200, blocksz=128)
    idx, cnt = mu.qk_topkmask_indices(q, k, 200, blocksz=128)
    ref = orc.sp_attn_tokens(q.cpu(), k.cpu(), v.cpu(), idx.cpu(), cnt.cpu(), 128)
    d = (o.float().cpu() - ref).abs()
    assert d.max() < OUT_MAX_ABS and d.mean() < OUT_MEAN_ABS
    o_all = sf.attn_topkmask_cuda(q, k, v, 0, 0, select_k=None, blocksz=128)
    d = (o_all.float().cpu() - orc.full_attn(q.cpu(), k.cpu(), v.cpu())).abs()
    assert d.max() < OUT_MAX_ABS and d.mean() < OUT_MEAN_ABS


def test_topk_argument_checks():
    capi = _capi()
    q = torch.zeros(1, 1, 256, 64, dtype=torch.bfloat16, device="cuda")
    idx = torch.empty(1, 1, 2, 128, dtype=torch.int32, device="cuda")
    cnt = torch.empty(1, 1, 2, dtype=torch.int32, device="cuda")
    for bad_k in (0, 257, 129):                      # none, more than the keys, more than the list stride
        with pytest.raises(capi.FgattnError):
            capi.topk_indices(idx, cnt, q, q, bad_k)
