"""GPU parity (bit-exact) of the one-bit-per-entry mask kernels and of the caches built on them."""
import numpy as np
import pytest
import torch

from helpers import GOLDEN

pytestmark = pytest.mark.gpu


def _capi():
    from fgattn_tk_cuda_b200 import capi
    return capi


def test_pack_unpack_golden_fixture():
    """pack / unpack / compressed-cache lists against vectors made by the reference
    (python/spattn/mask_utils.py:421-440, :89-93)."""
    capi = _capi()
    z = np.load(GOLDEN / "packed_2x3x5x136.npz")
    for src in (torch.from_numpy(z["mask"]), torch.from_numpy(z["mask"].astype(np.uint8)),
                torch.from_numpy(z["mask"].astype(np.int32) * 5)):
        packed = torch.full(z["packed"].shape, 0xAA, dtype=torch.uint8, device="cuda")
        capi.pack_mask(packed, src.cuda())
        assert np.array_equal(packed.cpu().numpy(), z["packed"])
    for dt in (torch.bool, torch.uint8, torch.int32):
        mask = torch.empty(z["mask"].shape, dtype=dt, device="cuda")
        capi.unpack_mask(mask, torch.from_numpy(z["packed"]).cuda())
        assert np.array_equal(mask.cpu().numpy().astype(bool), z["mask"])
        assert int(mask.to(torch.int32).max()) == 1
    idx = torch.full(z["index"].shape, -1, dtype=torch.int32, device="cuda")
    cnt = torch.full(z["count"].shape, -1, dtype=torch.int32, device="cuda")
    capi.packedmask_to_indexmask(idx, cnt, torch.from_numpy(z["packed"]).cuda(), 136)
    assert np.array_equal(idx.cpu().numpy(), z["index"]) and np.array_equal(cnt.cpu().numpy(), z["count"])
    back = torch.full(z["packed"].shape, 0x55, dtype=torch.uint8, device="cuda")
    capi.indexmask_to_packedmask(back, idx, cnt)
    assert np.array_equal(back.cpu().numpy(), z["packed"])


@pytest.mark.parametrize("rows,width,dens", [(7, 8, 0.5), (3, 40, 0.3), (5, 4096, 0.08), (2, 75648, 0.02),
                                              (4, 1024, 0.0), (4, 1024, 1.0), (300, 256, 0.15)])
def test_pack_unpack_roundtrip(rows, width, dens):
    from oracle import fgattn_oracle as orc
    capi = _capi()
    g = torch.Generator().manual_seed(rows * 131 + width)
    mask = torch.rand(rows, width, generator=g) < dens
    packed = torch.empty(rows, width // 8, dtype=torch.uint8, device="cuda")
    capi.pack_mask(packed, (mask.to(torch.int32) * 7).cuda())
    assert np.array_equal(packed.cpu().numpy(), orc.pack_mask(mask))
    out = torch.empty(rows, width, dtype=torch.int32, device="cuda")
    capi.unpack_mask(out, packed)
    assert torch.equal(out.cpu(), mask.to(torch.int32))


@pytest.mark.parametrize("rows,width,stride,n_valid,dens", [(6, 384, 384, 384, 0.3), (5, 1280, 1280, 1201, 0.05),
                                                             (3, 40, 40, 33, 0.5), (2, 32768, 32768, 32760, 0.1),
                                                             (4, 256, 256, 256, 0.0), (4, 256, 256, 256, 1.0),
                                                             (9, 264, 260, 257, 0.4), (2, 75648, 75648, 75600, 0.03)])
def test_packed_to_index_and_back(rows, width, stride, n_valid, dens):
    from oracle import fgattn_oracle as orc
    capi = _capi()
    g = torch.Generator().manual_seed(width + rows)
    mask = torch.rand(rows, width, generator=g) < dens
    packed_np = orc.pack_mask(mask)
    packed = torch.from_numpy(packed_np).cuda()
    idx = torch.full((rows, stride), -1, dtype=torch.int32, device="cuda")
    cnt = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
    capi.packedmask_to_indexmask(idx, cnt, packed, n_valid)
    ridx, rcnt = orc.packedmask_to_indexmask(packed_np, n_valid=n_valid, stride=stride)
    assert np.array_equal(cnt.cpu().numpy(), rcnt) and np.array_equal(idx.cpu().numpy(), ridx)
    # lists -> bits reproduces the live part of the mask
    back = torch.full((rows, 4 * ((width + 31) // 32)), 0xFF, dtype=torch.uint8, device="cuda")
    capi.indexmask_to_packedmask(back, idx, cnt)
    assert np.array_equal(back.cpu().numpy(), orc.indexmask_to_packedmask(ridx, rcnt, width))
    live = mask.clone()
    live[:, n_valid:] = False
    assert np.array_equal(orc.unpack_mask(back.cpu().numpy())[:, :width], live.numpy())


def test_argument_checks():
    capi = _capi()
    packed = torch.empty(4, 5, dtype=torch.uint8, device="cuda")
    with pytest.raises(capi.FgattnError):
        capi.pack_mask(packed, torch.zeros(4, 40, dtype=torch.float32, device="cuda"))   # dtype
    with pytest.raises(capi.FgattnError):
        capi.pack_mask(packed, torch.zeros(4, 44, dtype=torch.int32, device="cuda"))     # width % 8


def test_compressed_caches_match_plain_caches():
    """CompressedBitMaskCache / CompressedListCache hand back exactly the lists the uncompressed
    caches do (python/spattn/mask_utils.py:70-98)."""
    from fgattn_tk_cuda_b200.spattn import mask_utils as mu
    g = torch.Generator().manual_seed(5)
    B, H, SB, W, S = 1, 3, 4, 512, 500
    mask = ((torch.rand(B, H, SB, W, generator=g) < 0.1).to(torch.int32) * 3).cuda()
    plain, comp = mu.BitMaskCache([0]), mu.CompressedBitMaskCache([0])
    plain.update_cache(0, mask, S)
    comp.update_cache(0, mask, S)
    assert comp.cache[0][0].numel() * 8 == mask.numel()             # one bit per entry instead of 32
    (i0, c0), (i1, c1) = plain.get_mask_from_cache(0), comp.get_mask_from_cache(0)
    assert torch.equal(i0, i1) and torch.equal(c0, c1)
    # block lists: 37 key blocks, list stride 37
    nqb = nkb = 37
    bm = torch.rand(2, 2, nqb, nkb, generator=g) < 0.2
    from oracle import fgattn_oracle as orc
    ridx, rcnt = orc.bitmask_to_indexmask(bm)
    lc = mu.CompressedListCache([0])
    lc.update_cache(3, ridx.cuda(), rcnt.cuda(), nkb)
    i2, c2 = lc.get_mask_from_cache(3)
    assert torch.equal(i2.cpu(), ridx) and torch.equal(c2.cpu(), rcnt)


def test_cached_attention_flow_block_mode():
    """cached_attn_cuda (python/spattn/sparseattn_functionals.py:95-113) in the 64x64 mode: the run that
    builds the mask returns dense attention; a later run with DIFFERENT q / k reuses the cached
    lists and must renormalise over the kept blocks (oracle: softmax restricted to kept keys)."""
    from fgattn_tk_cuda_b200 import synth
    from fgattn_tk_cuda_b200.spattn import mask_utils as mu, sparseattn_functionals as sf
    from oracle import fgattn_oracle as orc
    from helpers import OUT_MAX_ABS, OUT_MEAN_ABS
    w = synth.Workload("t", 1, 2, 1024, 128, "clustered", centroids=16, run=128, tau=1e-4, seed=77)
    q, k, v = synth.make_qkv(w, device="cuda")
    for cache in (mu.NaiveMaskCache([0]), mu.CompressedListCache([0])):
        o0 = sf.cached_attn_cuda(q, k, v, 0, 0, thresh=w.tau, blocksz=64, mask_cache=cache)
        ref0 = orc.full_attn(q.cpu(), k.cpu(), v.cpu())
        assert (o0.float().cpu() - ref0).abs().max() < OUT_MAX_ABS
        q2 = (q.float() * 1.05 + 0.02).to(torch.bfloat16)
        o1 = sf.cached_attn_cuda(q2, k, v, 0, 1, thresh=w.tau, blocksz=64, mask_cache=cache)
        idx, cnt = cache.get_mask_from_cache(0)[:2]
        ref1 = orc.sp_attn_blocks(q2.cpu(), k.cpu(), v.cpu(), idx.cpu(), cnt.cpu())
        d = (o1.float().cpu() - ref1).abs()
        assert d.max() < OUT_MAX_ABS and d.mean() < OUT_MEAN_ABS
