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


_FIRST_CALL_SCRIPT = r"""
import torch
from fgattn_tk_cuda_b200 import capi, synth
w = synth.Workload("na0", 1, 2, 900, 128, "clustered", centroids=8, run=64, tau=1e-3, seed=79)
q, k, v = (t.cuda() for t in synth.make_qkv(w))
B, H, S, D = q.shape
nqb = nkb = (S + 63) // 64
s_pad = 128 * ((S + 127) // 128)
def bufs():
    return (torch.full((B, H, nqb, nkb), -7, dtype=torch.int32, device="cuda"),
            torch.full((B, H, nqb), -7, dtype=torch.int32, device="cuda"),
            torch.full((B, H, 1, s_pad), 3.0, device="cuda"), torch.full((B, H, 1, s_pad), 3.0, device="cuda"))
got = bufs()
scratch = torch.empty(capi.block_scratch_bytes(B, H, S) // 4, device="cuda")     # allocated BEFORE, by the caller
torch.cuda.synchronize()
# the very first call into the library in this process is the allocation-free one
capi.block_index_lists_noalloc(*got, q, k, w.tau)
torch.cuda.synchronize()
free0 = torch.cuda.mem_get_info()[0]
capi.check()                                   # reads the word built into the library; allocates nothing
free1 = torch.cuda.mem_get_info()[0]
assert free0 - free1 < (1 << 20), (free0, free1)
ref = bufs()
capi.block_index_lists(*ref, q, k, w.tau, scratch)
capi.check()
for a, b in zip(ref, got):
    assert torch.equal(a, b)
print("first-call ok")
"""


def test_noalloc_as_first_call_of_a_fresh_process():
    """A process whose first and only use of the library is the allocation-free entry point: the
    results are right and fgattn_check -- which then has only the library's built-in error word to
    read -- reports a clean run without allocating anything itself."""
    import subprocess
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parents[1]
    r = subprocess.run([sys.executable, "-c", _FIRST_CALL_SCRIPT], cwd=root, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "first-call ok" in r.stdout
