"""Generate the golden fixtures in this folder from the UNMODIFIED reference.

Run in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports python/spattn/mask_utils.py and python/test_mask.py from the reference (CPU only; the
compiled module `spattn.cuda_attn` is stubbed because test_mask.py imports it at module scope),
runs the reference functions on small seeded inputs and stores inputs + outputs as .npz.
The fixtures travel with the repository; the reference does not.
"""
import sys
import types
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def load_reference(ref_root: Path):
    sys.path.insert(0, str(ref_root / "python"))
    sys.modules.setdefault("spattn.cuda_attn", types.ModuleType("spattn.cuda_attn"))
    import spattn.mask_utils as mu           # noqa: E402
    import spattn
    spattn.cuda_attn = sys.modules["spattn.cuda_attn"]
    import test_mask as tm                   # noqa: E402
    return mu, tm


def clustered(S, D, n_cent, run, seed):
    g = torch.Generator().manual_seed(seed)
    cent = torch.randn(n_cent, D, generator=g) * 2.0
    def draw():
        pick = torch.randint(0, n_cent, ((S + run - 1) // run,), generator=g)
        return cent[pick].repeat_interleave(run, dim=0)[:S] + 0.5 * torch.randn(S, D, generator=g)
    return draw(), draw(), torch.randn(S, D, generator=g)


def bf16_round(x):
    return x.to(torch.bfloat16).to(torch.float32)


def main(ref_root: str):
    mu, tm = load_reference(Path(ref_root))
    torch.manual_seed(0)
    cases = {
        # name: (B, H, S, D, kind, tau, blocksz list)
        "normal_s256_d64": (1, 2, 256, 64, "normal", 1e-3),
        "normal_s200_d128": (1, 2, 200, 128, "normal", 4e-3),          # ragged last block
        "clustered_s512_d128": (1, 2, 512, 128, "clustered", 1e-4),
        "clustered_s389_d64": (2, 1, 389, 64, "clustered", 1e-3),      # ragged, D=64
    }
    for name, (B, H, S, D, kind, tau) in cases.items():
        q = torch.empty(B, H, S, D); k = torch.empty_like(q); v = torch.empty_like(q)
        for i in range(B * H):
            if kind == "normal":
                g = torch.Generator().manual_seed(100 + i)
                qh, kh, vh = (torch.randn(S, D, generator=g) for _ in range(3))
            else:
                qh, kh, vh = clustered(S, D, 8, 64, 200 + i)
            q.view(-1, S, D)[i], k.view(-1, S, D)[i], v.view(-1, S, D)[i] = qh, kh, vh
        q, k, v = bf16_round(q), bf16_round(k), bf16_round(v)           # exactly representable in bf16
        bits = lambda t: t.to(torch.bfloat16).view(torch.int16).numpy()      # stored as bf16 bit patterns
        out = {"q_bf16": bits(q), "k_bf16": bits(k), "v_bf16": bits(v), "tau": np.float64(tau)}
        for bs in (64, 128):
            bit = mu.qk_bitmask(q, k, thresh=tau, blocksz=bs)            # mask_utils.py:206-222
            idx, cnt = mu.qk_indexmask(q, k, thresh=tau, blocksz=bs)     # mask_utils.py:225-245
            idx2, cnt2 = mu.bitmask_to_indexmask(bit)                    # mask_utils.py:272-289
            assert torch.equal(idx, idx2) and torch.equal(cnt, cnt2)
            out[f"bitmask_{bs}"] = np.packbits(bit.numpy(), axis=-1)
            out[f"index_{bs}"] = idx.numpy().astype(np.int32)
            out[f"count_{bs}"] = cnt.numpy().astype(np.int32)
            # masked attention of python/test_mask.py:37-54; its qdotk hard-codes D=128, so for
            # D=64 the inputs are pre-scaled so that the effective scale is 1/sqrt(D).
            qs = q * ((128.0 / D) ** 0.5)
            out[f"masked_attn_{bs}"] = tm.qkattn_masked(qs, k, v, thresh=tau, blocksz=bs).numpy()
        # attnmapor on a float map with a ragged tail (mask_utils.py:126-142)
        amap = torch.softmax((q[0, 0] @ k[0, 0].T) / D ** 0.5, dim=-1)
        out["attnmapor_64_float"] = mu.attnmapor(amap, 64).numpy()
        # m, l definitions of python/test/spattn/test_mask_utils.py:42-52
        qk = torch.einsum("bhmd,bhnd->bhmn", q, k)
        mx = qk.max(dim=-1).values
        out["max_q"] = mx.numpy()
        out["denom"] = torch.exp((qk - mx[..., None]) / D ** 0.5).sum(dim=-1).numpy()
        out["sdpa"] = torch.nn.functional.scaled_dot_product_attention(q, k, v).numpy()  # test_extension.py:15-20
        np.savez_compressed(HERE / f"{name}.npz", **out)
        print(name, {k_: v_.shape for k_, v_ in out.items() if hasattr(v_, "shape")})

    # boolean_to_index_mask_2d on random maps incl. empty and full rows (mask_utils.py:152-167)
    g = torch.Generator().manual_seed(7)
    bm = torch.rand(9, 37, generator=g) < 0.3
    bm[2] = False
    bm[5] = True
    idx, cnt = mu.boolean_to_index_mask_2d(bm)
    np.savez_compressed(HERE / "compaction_9x37.npz", mask=bm.numpy(), index=idx.numpy(), count=cnt.numpy())

    # pack / unpack (mask_utils.py:421-440).  Both create their bit weights with device='cuda'; there
    # is no GPU where the fixtures are made, so torch.tensor is wrapped to drop the device argument
    # while the (unmodified) reference functions run.
    real_tensor = torch.tensor
    torch.tensor = lambda *a, **kw: real_tensor(*a, **{k_: v_ for k_, v_ in kw.items() if k_ != "device"})
    try:
        g = torch.Generator().manual_seed(11)
        pm = torch.rand(2, 3, 5, 136, generator=g) < 0.2
        pm[0, 0, 0] = False
        pm[1, 2, 4] = True
        packed = mu.pack(pm)
        back = mu.unpack(packed)
    finally:
        torch.tensor = real_tensor
    assert torch.equal(back, pm)
    pidx, pcnt = mu.bitmask_to_indexmask(pm)                              # what the compressed cache returns
    np.savez_compressed(HERE / "packed_2x3x5x136.npz", mask=pm.numpy(), packed=packed.numpy(),
                        index=pidx.numpy().astype(np.int32), count=pcnt.numpy().astype(np.int32))

    # top-k selector (mask_utils.py:389-417) on fp32 copies of bf16-representable inputs; ragged last
    # query block (300 = 2 * 128 + 44).  The function prints its result; that output is discarded.
    import contextlib, io
    g = torch.Generator().manual_seed(21)
    B, H, S, D, K = 1, 2, 300, 64, 40
    tq = bf16_round(torch.randn(B, H, S, D, generator=g))
    tk = bf16_round(torch.randn(B, H, S, D, generator=g))
    with contextlib.redirect_stdout(io.StringIO()):
        tidx, tcnt = mu.qk_topkmask_indices(tq, tk, K, B, H, S, D, 128)
    np.savez_compressed(HERE / "topk_s300_d64_k40.npz", q_bf16=tq.to(torch.bfloat16).view(torch.int16).numpy(),
                        k_bf16=tk.to(torch.bfloat16).view(torch.int16).numpy(), index=tidx.numpy().astype(np.int32),
                        count=tcnt.numpy().astype(np.int32), select_k=np.int64(K), blocksz=np.int64(128))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/make_golden.py <checkout of sankeerth95/fgattn_tk_cuda>")
    main(sys.argv[1])
