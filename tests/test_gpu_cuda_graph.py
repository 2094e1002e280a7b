"""The sparse step can be captured in a CUDA graph and replayed: no entry point synchronises,
allocates with the CUDA allocator or touches the legacy default stream once it has been called once."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_block_sparse_step_replays_from_a_cuda_graph():
    import fgattn_tk_cuda_b200.spattn as spattn  # noqa: F401  registers torch.ops.cuda_attn
    from fgattn_tk_cuda_b200 import capi
    mu = spattn.mask_utils
    import dataclasses
    from fgattn_tk_cuda_b200 import synth
    w = dataclasses.replace(synth.WORKLOADS["c3"], H=4, S=4096)      # clustered: a mix of kept / dropped blocks
    q, k, v = synth.make_qkv(w, device="cuda")
    idx, cnt, max_q, denom = mu.qk_block_indexmask_cuda(q, k, w.tau)
    assert 0 < int(cnt.sum()) < idx.numel()
    eager = torch.empty_like(q)
    torch.ops.cuda_attn.sp_attn_blocks_ml(eager, q, k, v, idx, cnt, max_q, denom)      # also the warm-up call
    eager_rn = torch.empty_like(q)
    torch.ops.cuda_attn.sp_attn_blocks(eager_rn, q, k, v, idx, cnt)
    capi.check()

    out = torch.zeros_like(q)
    out_rn = torch.zeros_like(q)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            torch.ops.cuda_attn.sp_attn_blocks_ml(out, q, k, v, idx, cnt, max_q, denom)
            torch.ops.cuda_attn.sp_attn_blocks(out_rn, q, k, v, idx, cnt)
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(3):
        out.zero_()
        out_rn.zero_()
        graph.replay()
    torch.cuda.synchronize()
    capi.check()
    assert torch.equal(out, eager)
    assert torch.equal(out_rn, eager_rn)
