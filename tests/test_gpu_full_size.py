"""Full-size BASELINE configurations on the GPU, checked against the CPU oracle.

Every configuration runs at its full shape.  The oracle (fp32 torch on the CPU, pinned to the
reference's own functions by the golden fixtures) checks
  * whole heads where the CPU finishes them in seconds (all of C1; the last head of C3),
  * windows of two neighbouring 64-row query blocks (one 128-row tile of the sparse kernel) on
    several heads of each configuration, the first and the last head included: the first, a middle and
    the last window of the sequence, plus the window whose two blocks' lists differ the most (the
    one-sided entries of the union walk),
and size-independent properties cover the rest (determinism, list format, all-blocks-listed == dense).
Tolerances are BASELINE's: lists bit-exact except blocks whose score lies within 1e-3 * tau of tau;
outputs within max-abs 2e-2 and mean-abs 2e-3 (bf16 inputs, fp32 accumulation)."""
import dataclasses

import pytest
import torch

from helpers import OUT_MAX_ABS, OUT_MEAN_ABS, TAU_REL

pytestmark = pytest.mark.gpu


def _close(o, ref, mx=OUT_MAX_ABS, mean=OUT_MEAN_ABS):
    d = (o.float().cpu() - torch.as_tensor(ref).float().cpu()).abs()
    assert torch.isfinite(o.float()).all()
    assert d.max().item() <= mx, d.max().item()
    assert d.mean().item() <= mean, d.mean().item()


def _bitmap(idx, cnt, nkb):
    live = torch.arange(idx.shape[3], device=idx.device)[None, None, None, :] < cnt[..., None]
    bm = torch.zeros(*idx.shape[:3], nkb + 1, dtype=torch.bool, device=idx.device)
    bm.scatter_(3, torch.where(live, idx.long(), torch.full_like(idx, nkb).long()), True)
    return bm[..., :nkb]


def _pipeline(w, heads=None):
    from fgattn_tk_cuda_b200 import capi, synth
    import fgattn_tk_cuda_b200.spattn as spattn
    q, k, v = synth.make_qkv(w, device="cuda", heads=heads)
    out = spattn.mask_utils.qk_block_indexmask_cuda(q, k, w.tau, v=v)
    capi.check()
    return (q, k, v) + tuple(out)


def _list_format(idx, cnt, nkb):
    bm = _bitmap(idx, cnt, nkb)
    assert torch.equal(bm.sum(-1).int(), cnt)
    live = torch.arange(idx.shape[3], device=idx.device)[None, None, None, :] < cnt[..., None]
    assert torch.all(idx[~live] == nkb)
    asc = (idx[..., 1:] > idx[..., :-1]) | ~live[..., 1:]
    assert asc.all()
    return bm


def _most_different_pair(bm, b, h):
    """Index of the pair of neighbouring query blocks of unit (b, h) whose lists differ in the most
    entries (found on the GPU), and that number."""
    rows = bm[b, h]
    n = rows.shape[0] // 2
    diff = (rows[0:2 * n:2] ^ rows[1:2 * n:2]).sum(-1)
    p = int(diff.argmax().item())
    return p, int(diff[p].item())


def _check_window(orc, tau, S, q, k, v, bm, b, h, r0, r1, o_sparse=None, o_dense=None, m=None, l=None):
    """Rows [r0, r1) of unit (b, h): the block map, max_q / denom, the dense and the sparse output
    against the oracle on the same inputs."""
    qs, ks, vs = q[b:b + 1, h:h + 1, r0:r1].cpu(), k[b:b + 1, h:h + 1].cpu(), v[b:b + 1, h:h + 1].cpu()
    pmax = orc.qk_block_pmax(qs, ks, 64, 64, kv_seq_len=S)
    got = bm[b:b + 1, h:h + 1, r0 // 64:(r1 + 63) // 64].cpu()
    bad = (got ^ (pmax > tau)) & ~orc.near_threshold(pmax, tau, TAU_REL)
    assert not bad.any(), (b, h, r0, int(bad.sum()))
    if o_sparse is not None:
        _close(o_sparse[b:b + 1, h:h + 1, r0:r1], orc.block_masked_attn(qs, ks, vs, got, kv_seq_len=S))
    if o_dense is not None:
        _close(o_dense[b:b + 1, h:h + 1, r0:r1], orc.full_attn(qs, ks, vs, kv_seq_len=S))
    if m is not None:
        rm, rl = orc.maxq_denom(qs, ks, kv_seq_len=S)
        n = r1 - r0
        assert (m[b, h, 0, r0:r1].cpu() - rm[0, 0, 0, :n]).abs().max() <= 2e-3
        assert ((l[b, h, 0, r0:r1].cpu() - rl[0, 0, 0, :n]).abs() / rl[0, 0, 0, :n]).max() <= 2e-3


def _windows(S):
    """First, middle and last 128-row window of a sequence (the last may be ragged)."""
    last = (S - 1) // 128 * 128
    mid = (S // 2) // 128 * 128
    return [(0, 128), (mid, mid + 128), (last, S)]


def test_c1_cpu_config():
    """BASELINE's CPU-runnable configuration (B=1 H=4 S=1024 D=64, N(0,1), tau=1e-3, 64x64 blocks):
    the fp32 inputs are rounded to bf16 and the GPU path is compared with the fp32 oracle on the same
    rounded inputs, the way the reference compares its kernels with SDPA
    (python/test/test_extension.py:16-20) -- the whole output, every list, m and l."""
    from fgattn_tk_cuda_b200 import capi, synth
    from oracle import fgattn_oracle as orc
    w = synth.WORKLOADS["c1"]
    q32, k32, v32 = synth.make_qkv(w)
    assert q32.dtype == torch.float32 and q32.shape == (1, 4, 1024, 64)
    qb, kb, vb = (t.to(torch.bfloat16) for t in (q32, k32, v32))
    q, k, v = qb.cuda(), kb.cuda(), vb.cuda()
    import fgattn_tk_cuda_b200.spattn as spattn
    idx, cnt, m, l, o_dense = spattn.mask_utils.qk_block_indexmask_cuda(q, k, w.tau, v=v)
    capi.check()
    nkb = 16
    bm = _list_format(idx, cnt, nkb).cpu()
    pmax = orc.qk_block_pmax(qb, kb)
    bad = (bm ^ (pmax > w.tau)) & ~orc.near_threshold(pmax, w.tau, TAU_REL)
    assert not bad.any(), int(bad.sum())
    ridx, rcnt = orc.bitmask_to_indexmask(bm)
    assert torch.equal(idx.cpu(), ridx) and torch.equal(cnt.cpu(), rcnt)
    rm, rl = orc.maxq_denom(qb, kb)
    assert (m.cpu() - rm).abs().max() <= 2e-3
    assert ((l.cpu() - rl).abs() / rl).max() <= 2e-3
    _close(o_dense, orc.full_attn(qb, kb, vb))
    o = torch.full_like(q, float("nan"))
    capi.sp_attn_blocks_ml(o, q, k, v, idx, cnt, m, l)
    capi.check()
    _close(o, orc.block_masked_attn(qb, kb, vb, bm))
    o_rn = torch.full_like(q, float("nan"))
    capi.sp_attn_blocks(o_rn, q, k, v, idx, cnt)
    capi.check()
    _close(o_rn, orc.sp_attn_blocks(qb, kb, vb, idx.cpu(), cnt.cpu()))


def test_c2_dense_full_size():
    """B=2 H=16 S=4096 D=64 dense attention: four whole heads (first and last of each batch entry)
    against the oracle, all heads against the fused m/l variant."""
    from fgattn_tk_cuda_b200 import capi, synth
    from oracle import fgattn_oracle as orc
    w = synth.WORKLOADS["c2"]
    q, k, v = synth.make_qkv(w, device="cuda")
    o = torch.empty_like(q)
    capi.full_attn(o, q, k, v)
    o2 = torch.empty_like(q)
    s_pad = 128 * ((w.S + 127) // 128)
    m = torch.empty(w.B, w.H, 1, s_pad, device="cuda")
    l = torch.empty_like(m)
    capi.fullattn_maxq_denom(o2, m, l, q, k, v)
    capi.check()
    assert torch.equal(o, o2)
    for b, h in ((0, 0), (0, 15), (1, 7), (1, 15)):
        qs, ks, vs = (t[b:b + 1, h:h + 1].cpu() for t in (q, k, v))
        _close(o[b:b + 1, h:h + 1], orc.full_attn(qs, ks, vs))
        rm, rl = orc.maxq_denom(qs, ks)
        assert (m[b, h, 0].cpu() - rm[0, 0, 0]).abs().max() <= 2e-3
        assert ((l[b, h, 0].cpu() - rl[0, 0, 0]).abs() / rl[0, 0, 0]).max() <= 2e-3


def test_c3_headline_full_size():
    """B=1 H=32 S=16384 D=128 clustered, all 32 heads on the GPU: density band, determinism, list
    format; oracle windows (first / middle / last / most-different pair) on heads 0, 5, 13, 31;
    the all-blocks-listed property (sparse == dense)."""
    from fgattn_tk_cuda_b200 import capi, synth
    from oracle import fgattn_oracle as orc
    w = synth.WORKLOADS["c3"]
    q, k, v, idx, cnt, m, l, o_dense = _pipeline(w)
    B, H, S, D = q.shape
    nqb = nkb = S // 64
    dens = cnt.sum().item() / (B * H * nqb * nkb)
    assert 0.05 <= dens <= 0.20, dens
    # determinism: a second pass gives bit-identical lists and m/l
    _, _, _, idx2, cnt2, m2, l2, _ = _pipeline(w)
    assert torch.equal(idx, idx2) and torch.equal(cnt, cnt2) and torch.equal(m, m2) and torch.equal(l, l2)
    bm = _list_format(idx, cnt, nkb)
    # sparse pass
    o = torch.full_like(q, float("nan"))
    capi.sp_attn_blocks_ml(o, q, k, v, idx, cnt, m, l)
    capi.check()
    assert torch.isfinite(o.float()).all()
    n_onesided = 0
    for h in (0, 5, 13, 31):
        p, nd = _most_different_pair(bm, 0, h)
        n_onesided += nd
        for r0, r1 in _windows(S) + [(p * 128, p * 128 + 128)]:
            _check_window(orc, w.tau, S, q, k, v, bm, 0, h, r0, r1, o_sparse=o, o_dense=o_dense, m=m, l=l)
    assert n_onesided > 0          # some checked window did walk entries kept by one half only
    # every block listed -> the gather kernel reproduces dense attention
    full_idx = torch.arange(nkb, dtype=torch.int32, device="cuda").expand(1, 4, nqb, nkb).contiguous()
    full_cnt = torch.full((1, 4, nqb), nkb, dtype=torch.int32, device="cuda")
    o4 = torch.empty_like(q[:, :4])
    capi.sp_attn_blocks_ml(o4, q[:, :4].contiguous(), k[:, :4].contiguous(), v[:, :4].contiguous(), full_idx, full_cnt,
                           m[:, :4].contiguous(), l[:, :4].contiguous())
    capi.check()
    d = (o4.float() - o_dense[:, :4].float()).abs()
    assert d.max().item() <= 1e-2 and d.mean().item() <= 5e-4


def test_c3_whole_last_head_against_oracle():
    """Head 31 of C3 in full (all 256 query blocks, 16384 x 16384 scores on the CPU): block map,
    lists, max_q / denom and the sparse output."""
    from fgattn_tk_cuda_b200 import capi, synth
    from oracle import fgattn_oracle as orc
    w = synth.WORKLOADS["c3"]
    q, k, v, idx, cnt, m, l, _ = _pipeline(w, heads=range(31, 32))
    S = w.S
    nkb = S // 64
    bm = _list_format(idx, cnt, nkb)
    o = torch.full_like(q, float("nan"))
    capi.sp_attn_blocks_ml(o, q, k, v, idx, cnt, m, l)
    capi.check()
    qc, kc, vc = q.cpu(), k.cpu(), v.cpu()
    pmax = orc.qk_block_pmax(qc, kc)
    got = bm.cpu()
    bad = (got ^ (pmax > w.tau)) & ~orc.near_threshold(pmax, w.tau, TAU_REL)
    assert not bad.any(), int(bad.sum())
    ridx, rcnt = orc.bitmask_to_indexmask(got)
    assert torch.equal(idx.cpu(), ridx) and torch.equal(cnt.cpu(), rcnt)
    _close(o, orc.block_masked_attn(qc, kc, vc, got))
    rm, rl = orc.maxq_denom(qc, kc)
    assert (m.cpu() - rm).abs().max() <= 2e-3
    assert ((l.cpu() - rl).abs() / rl).max() <= 2e-3


def test_c3_renormalising_full_size():
    """The renormalising block kernels (lists replayed from a cache) on 8 heads of C3 with perturbed
    queries: oracle windows on three heads; all blocks listed -> dense attention; rows of the
    ragged C4 shape against the oracle."""
    from fgattn_tk_cuda_b200 import capi, synth
    from oracle import fgattn_oracle as orc
    w = synth.WORKLOADS["c3"]
    q, k, v, idx, cnt, m, l, o_dense = _pipeline(w, heads=range(8))
    B, H, S, D = q.shape
    nqb = nkb = S // 64
    bm = _bitmap(idx, cnt, nkb)
    q2 = (q.float() * 1.1 - 0.03).to(torch.bfloat16)          # the cached lists meet new queries
    o = torch.full_like(q, float("nan"))
    capi.sp_attn_blocks(o, q2, k, v, idx, cnt)
    capi.check()
    assert torch.isfinite(o.float()).all()
    for h in (0, 3, 7):
        p, _ = _most_different_pair(bm, 0, h)
        for r0, r1 in _windows(S) + [(p * 128, p * 128 + 128)]:
            ref = orc.sp_attn_blocks(q2[:, h:h + 1, r0:r1].cpu(), k[:, h:h + 1].cpu(), v[:, h:h + 1].cpu(),
                                     idx[:, h:h + 1, r0 // 64:r1 // 64].cpu(), cnt[:, h:h + 1, r0 // 64:r1 // 64].cpu())
            _close(o[:, h:h + 1, r0:r1], ref)
    # every block listed -> dense attention
    full_idx = torch.arange(nkb, dtype=torch.int32, device="cuda").expand(1, 2, nqb, nkb).contiguous()
    full_cnt = torch.full((1, 2, nqb), nkb, dtype=torch.int32, device="cuda")
    o2 = torch.empty_like(q[:, :2])
    capi.sp_attn_blocks(o2, q[:, :2].contiguous(), k[:, :2].contiguous(), v[:, :2].contiguous(), full_idx, full_cnt)
    capi.check()
    d = (o2.float() - o_dense[:, :2].float()).abs()
    assert d.max().item() <= 1e-2 and d.mean().item() <= 5e-4
    # ragged shape (S = 12345, D = 64): last query blocks of one head
    w4 = dataclasses.replace(synth.WORKLOADS["c4"], B=1, H=3)
    q, k, v, idx, cnt, m, l, _ = _pipeline(w4)
    o = torch.full_like(q, float("nan"))
    capi.sp_attn_blocks(o, q, k, v, idx, cnt)
    capi.check()
    h, r0 = 1, 12032
    ref = orc.sp_attn_blocks(q[:, h:h + 1, r0:].cpu(), k[:, h:h + 1].cpu(), v[:, h:h + 1].cpu(),
                             idx[:, h:h + 1, r0 // 64:].cpu(), cnt[:, h:h + 1, r0 // 64:].cpu())
    _close(o[:, h:h + 1, r0:], ref)


def test_c4_ragged_full_size():
    """B=4 H=24 S=12345 (not a multiple of 64) D=64 in full: list format over all 96 units, oracle
    windows on units of the first and the last batch entry including the last, partial query / key
    blocks (the final block has 57 rows), tails of max_q / denom."""
    from fgattn_tk_cuda_b200 import capi, synth
    from oracle import fgattn_oracle as orc
    w = synth.WORKLOADS["c4"]
    q, k, v, idx, cnt, m, l, o_dense = _pipeline(w)
    B, H, S, D = q.shape
    assert (B, H, S, D) == (4, 24, 12345, 64)
    nkb = (S + 63) // 64
    assert idx.shape[2] == 193 and nkb == 193
    bm = _list_format(idx, cnt, nkb)
    dens = cnt.sum().item() / (B * H * 193 * nkb)
    assert 0.01 <= dens <= 0.30, dens
    o = torch.full_like(q, float("nan"))
    capi.sp_attn_blocks_ml(o, q, k, v, idx, cnt, m, l)
    capi.check()
    assert torch.isfinite(o.float()).all()
    for b, h in ((0, 0), (0, 23), (2, 11), (3, 0), (3, 23)):
        p, _ = _most_different_pair(bm, b, h)
        for r0, r1 in _windows(S) + [(p * 128, min(S, p * 128 + 128))]:
            _check_window(orc, w.tau, S, q, k, v, bm, b, h, r0, r1, o_sparse=o, o_dense=o_dense, m=m, l=l)
    # the last five query blocks of one unit in one piece (rows 12032 .. 12344)
    _check_window(orc, w.tau, S, q, k, v, bm, 1, 2, 188 * 64, S, o_sparse=o, o_dense=o_dense, m=m, l=l)
    assert torch.all(m[:, :, 0, S:] == 0) and torch.all(torch.isneginf(l[:, :, 0, S:]))


def test_c5_long_context_shape():
    """S=65536, D=128 with the long-context construction on 8 of the 512 units (the first four and
    the last four of the flattened batch x head order): chunked scratch (two units at a time), density
    band, oracle windows on every one of them including the last query rows."""
    from fgattn_tk_cuda_b200 import capi, synth
    from oracle import fgattn_oracle as orc
    w = synth.WORKLOADS["c5"]
    units = list(range(0, 4)) + list(range(508, 512))
    q, k, v = synth.make_qkv(w, device="cuda", heads=units)
    S, D = w.S, w.D
    n = len(units)
    nqb = nkb = S // 64
    idx = torch.empty(1, n, nqb, nkb, dtype=torch.int32, device="cuda")
    cnt = torch.empty(1, n, nqb, dtype=torch.int32, device="cuda")
    m = torch.empty(1, n, 1, S, device="cuda")
    l = torch.empty_like(m)
    scratch = torch.empty(capi.block_scratch_bytes(1, 2, S) // 4, device="cuda")      # two units per chunk
    capi.block_index_lists(idx, cnt, m, l, q, k, w.tau, scratch)
    capi.check()
    dens = cnt.sum().item() / (n * nqb * nkb)
    # measured: ~12.6 % (most query runs have no key run with their centroid among the 128 key runs
    # drawn from 256 centroids, so their probability mass spreads over many blocks)
    assert 0.005 <= dens <= 0.25, dens
    bm = _list_format(idx, cnt, nkb)
    o = torch.full_like(q, float("nan"))
    capi.sp_attn_blocks_ml(o, q, k, v, idx, cnt, m, l)
    capi.check()
    assert torch.isfinite(o.float()).all()
    for h in range(n):
        p, _ = _most_different_pair(bm, 0, h)
        wins = [(S - 128, S), (p * 128, p * 128 + 128)]
        if h in (0, n - 1):
            wins += _windows(S)[:2]
        for r0, r1 in wins:
            _check_window(orc, w.tau, S, q, k, v, bm, 0, h, r0, r1, o_sparse=o, m=m, l=l)
