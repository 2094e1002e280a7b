"""A bounded in-kernel wait that is left to run out: the kernel gives up and returns, fgattn_check
reports FGATTN_DEVICE_TIMEOUT with the id of the wait, the error word is cleared and the device keeps
working.  The probe is one warp waiting ~50 microseconds on a barrier nobody arrives at; nothing
faults, traps or spins without bound."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_runs_out_and_is_reported():
    from fgattn_tk_cuda_b200 import capi
    capi.check()                                        # clean before
    capi.selftest_bounded_wait(100000)
    with pytest.raises(capi.FgattnError) as ei:
        capi.check()
    assert ei.value.status == 6 and ei.value.code == 9001
    capi.check()                                        # the word was cleared
    # the context is intact: a real kernel runs and checks clean
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(1, 1, 256, 64, generator=g).to(torch.bfloat16).cuda() for _ in range(3))
    o = torch.empty_like(q)
    capi.full_attn(o, q, k, v)
    capi.check()
    ref = torch.softmax((q.float() @ k.float().transpose(-1, -2)) / 8.0, -1) @ v.float()
    assert (o.float() - ref).abs().max().item() < 2e-2


def test_budget_is_validated():
    from fgattn_tk_cuda_b200 import capi
    lib = capi.lib()
    assert lib.fgattn_selftest_bounded_wait(0, None) == 1
    assert lib.fgattn_selftest_bounded_wait(10 ** 10, None) == 1
