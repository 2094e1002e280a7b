"""Pin the CPU oracle to outputs of the reference's own PyTorch functions (tests/golden/*.npz,
made by tests/golden/make_golden.py from the unmodified reference)."""
import numpy as np
import pytest
import torch

from oracle import fgattn_oracle as orc
from helpers import GOLDEN, GOLDEN_CASES, load_golden, unpack_bitmask


@pytest.mark.parametrize("name", GOLDEN_CASES)
@pytest.mark.parametrize("bs", [64, 128])
def test_token_masks_and_lists(name, bs):
    g = load_golden(name)
    n = g["k"].shape[2]
    bit = orc.qk_bitmask(g["q"], g["k"], g["tau"], bs)
    assert torch.equal(bit, unpack_bitmask(g[f"bitmask_{bs}"], n))
    idx, cnt = orc.qk_indexmask(g["q"], g["k"], g["tau"], bs)
    assert idx.dtype == torch.int32 and cnt.dtype == torch.int32
    assert np.array_equal(idx.numpy(), g[f"index_{bs}"])
    assert np.array_equal(cnt.numpy(), g[f"count_{bs}"])


@pytest.mark.parametrize("name", GOLDEN_CASES)
@pytest.mark.parametrize("bs", [64, 128])
def test_masked_attention(name, bs):
    g = load_golden(name)
    o = orc.qkattn_masked(g["q"], g["k"], g["v"], g["tau"], bs)
    np.testing.assert_allclose(o.numpy(), g[f"masked_attn_{bs}"], rtol=0, atol=2e-5)


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_block_mode_is_or_of_token_mode(name):
    """64x64 block map == OR over each 64-key group of the reference's blocksz-64 token map."""
    g = load_golden(name)
    n = g["k"].shape[2]
    tok = unpack_bitmask(g["bitmask_64"], n)
    nkb = (n + 63) // 64
    pad = nkb * 64 - n
    tokp = torch.nn.functional.pad(tok, (0, pad))
    want = tokp.view(*tok.shape[:3], nkb, 64).any(dim=-1)
    pm = orc.qk_block_pmax(g["q"], g["k"], 64, 64)
    got = pm > g["tau"]
    assert torch.equal(got, want)
    idx, cnt = orc.qk_block_indexmask(g["q"], g["k"], g["tau"])
    assert torch.equal(cnt.long(), want.sum(-1))
    # block-masked attention equals the reference's masked attention when the block map is
    # expanded to tokens only where the token map says so is NOT the same thing; instead check
    # the all-kept map reproduces dense attention
    full = torch.ones_like(want)
    o = orc.block_masked_attn(g["q"], g["k"], g["v"], full)
    np.testing.assert_allclose(o.numpy(), g["sdpa"], rtol=0, atol=2e-5)


@pytest.mark.parametrize("name", GOLDEN_CASES)
def test_m_l_and_dense(name):
    g = load_golden(name)
    S = g["q"].shape[2]
    m, l = orc.maxq_denom(g["q"], g["k"])
    assert m.shape[-1] == 128 * ((S + 127) // 128)
    np.testing.assert_allclose(m[:, :, 0, :S].numpy(), g["max_q"], rtol=0, atol=1e-4)
    np.testing.assert_allclose(l[:, :, 0, :S].numpy(), g["denom"], rtol=2e-5, atol=0)
    assert torch.all(m[:, :, 0, S:] == 0) and torch.all(torch.isinf(l[:, :, 0, S:]))
    o = orc.full_attn(g["q"], g["k"], g["v"])
    np.testing.assert_allclose(o.numpy(), g["sdpa"], rtol=0, atol=2e-5)
    a = orc.attnmapor(torch.softmax((g["q"][0, 0].float() @ g["k"][0, 0].float().T) / g["q"].shape[3] ** 0.5, -1), 64)
    np.testing.assert_allclose(a.numpy(), g["attnmapor_64_float"], rtol=0, atol=1e-7)


def test_compaction_fixture():
    z = np.load(GOLDEN / "compaction_9x37.npz")
    idx, cnt = orc.boolean_to_index_mask_2d(z["mask"])
    assert np.array_equal(idx.numpy(), z["index"]) and np.array_equal(cnt.numpy(), z["count"])


def test_identity_list_equals_dense():
    """The reference's main sparse test: the identity key list reproduces dense attention
    (test/test_sparseattn_asyncgatherload_padded.cu:37-62)."""
    g = load_golden("normal_s200_d128")
    S = g["q"].shape[2]
    idx, cnt = orc.allindex_mask(1, 2, 256, S, 128)
    o = orc.sp_attn_tokens(g["q"], g["k"], g["v"], idx, cnt, 128)
    np.testing.assert_allclose(o.numpy(), g["sdpa"], rtol=0, atol=2e-5)
    nkb = (S + 63) // 64
    kb = torch.arange(nkb, dtype=torch.int32).expand(1, 2, nkb, nkb).contiguous()
    kc = torch.full((1, 2, nkb), nkb, dtype=torch.int32)
    o2 = orc.sp_attn_blocks(g["q"], g["k"], g["v"], kb, kc)
    np.testing.assert_allclose(o2.numpy(), g["sdpa"], rtol=0, atol=2e-5)


def test_packed_mask_fixture():
    """pack / unpack of the reference (python/spattn/mask_utils.py:421-440) and the lists its
    compressed cache rebuilds (:89-93)."""
    z = np.load(GOLDEN / "packed_2x3x5x136.npz")
    packed = orc.pack_mask(z["mask"])
    assert packed.dtype == np.uint8 and np.array_equal(packed, z["packed"])
    assert np.array_equal(orc.pack_mask(z["mask"].astype(np.int32) * 3), z["packed"])      # int mask, > 0 = keep
    assert np.array_equal(orc.unpack_mask(z["packed"]), z["mask"])
    idx, cnt = orc.packedmask_to_indexmask(z["packed"])
    assert np.array_equal(idx, z["index"]) and np.array_equal(cnt, z["count"])
    assert np.array_equal(orc.indexmask_to_packedmask(z["index"], z["count"], 136)[..., :17], z["packed"])
    # n_valid cuts the tail, stride / sentinel are free
    idx2, cnt2 = orc.packedmask_to_indexmask(z["packed"], n_valid=100, stride=140, sentinel=7)
    ref = z["mask"].copy()
    ref[..., 100:] = False
    assert np.array_equal(cnt2, ref.sum(-1)) and (idx2[0, 0, 0] == 7).all()


def test_topk_fixture():
    """qk_topkmask_indices of the reference (python/spattn/mask_utils.py:389-417) on a ragged shape."""
    z = np.load(GOLDEN / "topk_s300_d64_k40.npz")
    q = torch.from_numpy(z["q_bf16"]).view(torch.bfloat16).float()
    k = torch.from_numpy(z["k_bf16"]).view(torch.bfloat16).float()
    idx, cnt = orc.topk_indices(q, k, int(z["select_k"]), int(z["blocksz"]))
    assert np.array_equal(cnt.numpy(), z["count"])
    assert np.array_equal(idx.numpy(), z["index"])
