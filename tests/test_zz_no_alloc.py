"""The allocation-free entry point fgattn_block_index_lists_noalloc.

Some callers may not allocate device memory where they call the library (the enqueue hook of an
inference-engine plugin, a serving loop whose memory was partitioned once at start-up).  For them the
library lends a built-in 64 MiB scratch array.  This file checks, through the C ABI, that the variant
returns exactly what fgattn_block_index_lists returns with caller-provided scratch -- on two calls in
a row, because both share the one array and the second starts from the first one's leftovers -- and
that sizes beyond the built-in maximum are refused.  Collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _buffers(B, H, S, nkb):
    s_pad = 128 * ((S + 127) // 128)
    nqb = (S + 63) // 64
    return (torch.full((B, H, nqb, nkb), -7, dtype=torch.int32, device="cuda"),
            torch.full((B, H, nqb), -7, dtype=torch.int32, device="cuda"),
            torch.full((B, H, 1, s_pad), 3.0, device="cuda"), torch.full((B, H, 1, s_pad), 3.0, device="cuda"))


def _both(capi, w, with_output):
    from fgattn_tk_cuda_b200 import synth
    q, k, v = (t.cuda() for t in synth.make_qkv(w))
    B, H, S, D = q.shape
    nkb = (S + 63) // 64
    ref = _buffers(B, H, S, nkb)
    scratch = torch.empty(capi.block_scratch_bytes(B, H, S) // 4, device="cuda")
    o_ref = torch.empty_like(q) if with_output else None
    capi.block_index_lists(*ref, q, k, w.tau, scratch, o=o_ref, v=v if with_output else None)
    got = _buffers(B, H, S, nkb)
    o_got = torch.full_like(q, float("nan")) if with_output else None
    capi.block_index_lists_noalloc(*got, q, k, w.tau, o=o_got, v=v if with_output else None)
    capi.check()
    for a, b in zip(ref, got):
        assert torch.equal(a, b)                      # same kernels, same arithmetic: bit-identical
    if with_output:
        assert torch.equal(o_ref, o_got)
    assert 0 < got[1].sum().item() < B * H * got[0].shape[2] * nkb


def test_noalloc_matches_caller_scratch_twice_in_a_row():
    from fgattn_tk_cuda_b200 import capi, synth
    first = synth.Workload("na1", 1, 3, 1500, 128, "clustered", centroids=8, run=64, tau=1e-3, seed=77)
    second = synth.Workload("na2", 2, 2, 700, 64, "clustered", centroids=6, run=32, tau=2e-3, seed=78)
    _both(capi, first, with_output=False)
    _both(capi, second, with_output=True)             # different shape over the first call's leftovers
    _both(capi, first, with_output=True)


def test_noalloc_rejects_units_beyond_the_builtin_scratch():
    from fgattn_tk_cuda_b200 import capi
    lib = capi.lib()
    S = 40000                                          # 625 key blocks x 40064 rows x 4 B = 100 MB per unit
    assert (S + 63) // 64 * (128 * ((S + 127) // 128)) * 4 > capi.NOALLOC_SCRATCH_BYTES
    buf = ctypes.c_void_p(0x1000)                      # never dereferenced: the size check comes first
    st = lib.fgattn_block_index_lists_noalloc(buf, buf, 625, buf, buf, None, buf, buf, None, 1e-3, 1, 1, S, 128, S,
                                              0.0, None)
    assert st == 7 and b"scratch" in lib.fgattn_status_string(st)
