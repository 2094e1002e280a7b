"""GPU parity of the dense family (full_attn, fullattn_maxq_denom, maxq_denom) through the C ABI
against the golden fixtures and the CPU oracle."""
import numpy as np
import pytest
import torch

from helpers import GOLDEN_CASES, OUT_MAX_ABS, OUT_MEAN_ABS, load_golden

pytestmark = pytest.mark.gpu


def _capi():
    from fgattn_tk_cuda_b200 import capi
    return capi


def _close(o, ref):
    d = (o.float().cpu() - torch.as_tensor(ref).float()).abs()
    assert torch.isfinite(o.float()).all()
    assert d.max().item() <= OUT_MAX_ABS, d.max().item()
    assert d.mean().item() <= OUT_MEAN_ABS, d.mean().item()


def _ml_buffers(B, H, S):
    s_pad = 128 * ((S + 127) // 128)
    m = torch.full((B, H, 1, s_pad), 7.0, device="cuda", dtype=torch.float32)
    l = torch.full((B, H, 1, s_pad), 7.0, device="cuda", dtype=torch.float32)
    return m, l


def _check_ml(m, l, ref_m, ref_l, S):
    m, l = m.cpu(), l.cpu()
    np.testing.assert_allclose(m[:, :, 0, :S].numpy(), np.asarray(ref_m), rtol=0, atol=2e-3)
    np.testing.assert_allclose(l[:, :, 0, :S].numpy(), np.asarray(ref_l), rtol=2e-3, atol=0)
    assert torch.all(m[:, :, 0, S:] == 0) and torch.all(torch.isneginf(l[:, :, 0, S:]))


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_golden_dense(name):
    capi = _capi()
    g = load_golden(name)
    q, k, v = (g[t].cuda() for t in "qkv")
    B, H, S, D = q.shape
    o = torch.full_like(q, float("nan"))
    capi.full_attn(o, q, k, v)
    capi.check()
    _close(o, g["sdpa"])

    o2 = torch.full_like(q, float("nan"))
    m, l = _ml_buffers(B, H, S)
    capi.fullattn_maxq_denom(o2, m, l, q, k, v)
    capi.check()
    _close(o2, g["sdpa"])
    _check_ml(m, l, g["max_q"], g["denom"], S)

    m2, l2 = _ml_buffers(B, H, S)
    capi.maxq_denom(m2, l2, q, k)
    capi.check()
    _check_ml(m2, l2, g["max_q"], g["denom"], S)


@pytest.mark.parametrize("B,H,S,D,kv", [(1, 3, 1000, 128, None), (2, 2, 777, 64, None), (1, 2, 1024, 128, 779),
                                       (1, 1, 64, 64, None), (1, 2, 2048, 64, None)])
def test_dense_vs_oracle(B, H, S, D, kv):
    from oracle import fgattn_oracle as orc
    capi = _capi()
    g = torch.Generator().manual_seed(S * 7 + D)
    q, k, v = (torch.randn(B, H, S, D, generator=g).to(torch.bfloat16) for _ in range(3))
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    o = torch.full_like(qc, float("nan"))
    m, l = _ml_buffers(B, H, S)
    capi.fullattn_maxq_denom(o, m, l, qc, kc, vc, kv_seq_len=kv)
    capi.check()
    _close(o, orc.full_attn(q, k, v, kv_seq_len=kv))
    rm, rl = orc.maxq_denom(q, k, kv_seq_len=kv)
    _check_ml(m, l, rm[:, :, 0, :S], rl[:, :, 0, :S], S)
    o1 = torch.full_like(qc, float("nan"))
    capi.full_attn(o1, qc, kc, vc, kv_seq_len=kv)
    capi.check()
    assert torch.equal(o1, o)          # same arithmetic with and without the m/l epilogue


def test_large_scores_rescale_path():
    """Scores that keep growing along the key axis force the running-maximum rescale."""
    from oracle import fgattn_oracle as orc
    capi = _capi()
    B, H, S, D = 1, 1, 512, 128
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, H, S, D, generator=g)
    k = torch.randn(B, H, S, D, generator=g) * torch.linspace(0.2, 3.0, S)[None, None, :, None]
    v = torch.randn(B, H, S, D, generator=g)
    q, k, v = (t.to(torch.bfloat16) for t in (q, k, v))
    o = torch.empty_like(q, device="cuda")
    m, l = _ml_buffers(B, H, S)
    capi.fullattn_maxq_denom(o, m, l, q.cuda(), k.cuda(), v.cuda())
    capi.check()
    _close(o, orc.full_attn(q, k, v))
    rm, rl = orc.maxq_denom(q, k)
    _check_ml(m, l, rm[:, :, 0, :S], rl[:, :, 0, :S], S)


def test_argument_errors():
    capi = _capi()
    q = torch.zeros(1, 1, 64, 96, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(capi.FgattnError) as e:
        capi.full_attn(torch.empty_like(q), q, q, q)
    assert e.value.status == 2
    q = torch.zeros(1, 1, 64, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(capi.FgattnError) as e:
        capi.full_attn(torch.empty_like(q), q, q, q, kv_seq_len=65)
    assert e.value.status == 1
    with pytest.raises(capi.FgattnError):
        capi.full_attn(torch.empty_like(q), q.float(), q, q)


@pytest.mark.parametrize("B,H,S,D,kv", [(1, 2, 1500, 128, None),      # ragged last tile, 28 keys in its second half
                                       (1, 2, 1664, 64, 1590),       # last tile's second half has no live key
                                       (1, 30, 1280, 128, None),     # 150 items: the last wave's two are cut in halves
                                       (2, 1, 2304, 64, 2111)])
def test_maxq_two_threads_per_row(B, H, S, D, kv):
    """Above 1024 keys maxq_denom runs the kernel that shares a row between two threads (one per 64-key block
    of a score tile, partial (m, l) merged at the end); "maxq_wide" = 0 sends it through the dense family.
    Both against the oracle, maxima identical, and the key-block lists built on either are the same."""
    from oracle import fgattn_oracle as orc
    capi = _capi()
    g = torch.Generator().manual_seed(S + D)
    q = torch.randn(B, H, S, D, generator=g)
    k = torch.randn(B, H, S, D, generator=g) * torch.linspace(0.3, 2.5, S)[None, None, :, None]   # maxima keep growing
    q, k = q.to(torch.bfloat16), k.to(torch.bfloat16)
    qc, kc = q.cuda(), k.cuda()
    rm, rl = orc.maxq_denom(q[:, :4], k[:, :4], kv_seq_len=kv)
    nqb = nkb = (S + 63) // 64
    out = {}
    try:
        capi.set_tuning("dense_persist", 0)      # up to 2048 keys maxq_denom alone would take the persistent form
        for wide in (1, 0):
            capi.set_tuning("maxq_wide", wide)
            m, l = _ml_buffers(B, H, S)
            capi.maxq_denom(m, l, qc, kc, kv_seq_len=kv)
            capi.check()
            _check_ml(m[:, :4], l[:, :4], rm[:, :, 0, :S], rl[:, :, 0, :S], S)
            idx = torch.empty(B, H, nqb, nkb, dtype=torch.int32, device="cuda")
            cnt = torch.empty(B, H, nqb, dtype=torch.int32, device="cuda")
            m2, l2 = _ml_buffers(B, H, S)
            scratch = torch.empty(capi.block_scratch_bytes(B, H, S) // 4, device="cuda")
            capi.block_index_lists(idx, cnt, m2, l2, qc, kc, 1e-3, scratch, kv_seq_len=kv)
            capi.check()
            assert torch.equal(m2, m)
            out[wide] = (m.cpu(), l.cpu(), idx.cpu(), cnt.cpu())
    finally:
        capi.set_tuning("maxq_wide", -1)
        capi.set_tuning("dense_persist", -1)
    assert torch.equal(out[0][0], out[1][0])
    np.testing.assert_allclose(out[0][1][..., :S].numpy(), out[1][1][..., :S].numpy(), rtol=5e-4)   # approximate exponentials, different summation order
    # a block whose probability lies within 1e-3 of the threshold may flip with the summation order of l
    assert (out[0][3] != out[1][3]).float().mean().item() <= 0.01
