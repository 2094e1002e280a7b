"""Stage timings at the shapes the reference's own benchmark scripts use.

Two tables, one JSON line per measurement on stdout:

* ``stages``: the stages of python/benchmark.py:6-127 of the reference (fused attention + max_q/denom,
  the token-list sparse kernel swept over list lengths, the index-mask build, pack / unpack, mask ->
  list compaction) at batch 1, heads {12, 40}, seq {32760, 75600}, D 128, block size 128
  (python/benchmark.py:113-126).
* ``model``: the attention calls of microbench.py:5-73 of the reference (heads 40, D 128, self
  attention at seq {20280, 32768, 45832, 74056} and cross attention against 512 keys).  Its linear
  layers are library GEMMs and are not part of this package.

The reference loads tensors captured from a diffusion model that it does not ship; the inputs here are
the seeded clustered construction of `synth` (64 centroids, runs of 256 tokens).  Every time is taken
with CUDA events around `reps` back-to-back calls after `warmup` calls.

    python -m fgattn_tk_cuda_b200.microbench --table stages --heads 12 --seq 32760
    python -m fgattn_tk_cuda_b200.microbench --table model
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import sys

import torch

STAGE_HEADS = (12, 40)               # python/benchmark.py:117
STAGE_SEQS = (32760, 75600)          # python/benchmark.py:118
MODEL_SEQS = {"480p, 49": 20280, "480p, 81": 32768, "720p, 49": 45832, "720p, 81": 74056}   # microbench.py:6-7
MODEL_HEADS = 5120 // 128            # microbench.py:9-12
CROSS_KEYS = 512                     # microbench.py:62-63
SWEEP_POINTS = 16                    # python/benchmark.py:31-33: lists of i * 4 * (seq // 64) tokens, i < 16


def sweep_lengths(seq: int):
    """Token-list lengths of the sparse-kernel sweep (python/benchmark.py:31-33)."""
    return [i * 4 * (seq // 64) for i in range(SWEEP_POINTS)]


def _time(fn, reps: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def _emit(**kw):
    print(json.dumps(kw), flush=True)


def _qkv(heads: int, seq: int, kv: int | None = None):
    from . import synth
    w = dataclasses.replace(synth.WORKLOADS["c3"], B=1, H=heads, S=seq)
    q, k, v = synth.make_qkv(w, device="cuda")
    if kv is not None:
        wk = dataclasses.replace(w, S=kv, seed=w.seed + 7)
        _, k, v = synth.make_qkv(wk, device="cuda")
    return q, k, v


def stage_table(heads: int, seq: int, reps: int, warmup: int, sweep=None):
    from . import capi
    from .spattn import mask_utils as mu, sparseattn_functionals as sf
    q, k, v = _qkv(heads, seq)
    B, H, S, D = q.shape
    shape = [B, H, S, D]
    thresh = 0.5 / 32760                                     # python/benchmark.py:9
    dense_flops = 4.0 * B * H * S * S * D
    nb, s_pad = (S + 127) // 128, 128 * ((S + 127) // 128)

    ms = _time(lambda: sf.baseline_attn_maxq_denom(q, k, v), reps, warmup)
    _emit(table="stages", stage="fullattn_maxq_denom", shape=shape, ms=ms, tflops=dense_flops / ms / 1e9)
    ms = _time(lambda: sf.baseline_attn(q, k, v), reps, warmup)
    _emit(table="stages", stage="full_attn", shape=shape, ms=ms, tflops=dense_flops / ms / 1e9)

    # sparse kernel over random token lists of growing length; every query block lists the same
    # `n` distinct random tokens
    out = torch.empty_like(q)
    perm = torch.randperm(S, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1)).to(torch.int32)
    for n in (sweep_lengths(S) if sweep is None else sweep):
        stride = max(128, 128 * ((n + 127) // 128))
        row = torch.full((stride,), stride, dtype=torch.int32, device="cuda")
        row[:n] = perm[:n]
        idx = row.expand(B, H, nb, stride).contiguous()
        cnt = torch.full((B, H, nb), n, dtype=torch.int32, device="cuda")
        ms = _time(lambda: torch.ops.cuda_attn.sp_attn(out, q, k, v, idx, cnt), reps, warmup)
        _emit(table="stages", stage="sp_attn", shape=shape, listed_tokens=n, ms=ms,
              tflops=4.0 * B * H * S * n * D / ms / 1e9)
        del idx, cnt

    ms = _time(lambda: mu.qk_indexmask_cuda(q, k, thresh, blocksz=128), reps, warmup)
    idx, cnt = mu.qk_indexmask_cuda(q, k, thresh, blocksz=128)
    _emit(table="stages", stage="qk_indexmask_cuda", shape=shape, ms=ms,
          token_density=float(cnt.float().mean().item()) / S)
    ms = _time(lambda: torch.ops.cuda_attn.sp_attn(out, q, k, v, idx, cnt), reps, warmup)
    _emit(table="stages", stage="sp_attn_threshold_lists", shape=shape, ms=ms,
          tflops=4.0 * 128 * D * float(cnt.sum().item()) / ms / 1e9)
    del idx, cnt

    mask = mu.qk_token_mask_cuda(q, k, thresh)[0]
    n_entries = mask.numel()
    ms = _time(lambda: mu.bitmask_to_indexmask_cuda(mask, S), reps, warmup)       # python/benchmark.py:94-109
    _emit(table="stages", stage="bitmask_to_indexmask_cuda", shape=shape, ms=ms, gbs=8.0 * n_entries / ms / 1e6)
    ms = _time(lambda: mu.pack(mask), reps, warmup)                                # python/benchmark.py:67-90
    _emit(table="stages", stage="pack", shape=shape, ms=ms, gbs=(4 + 1 / 8) * n_entries / ms / 1e6)
    packed = mu.pack(mask)
    ms = _time(lambda: mu.unpack(packed, dtype=torch.int32), reps, warmup)
    _emit(table="stages", stage="unpack", shape=shape, ms=ms, gbs=(4 + 1 / 8) * n_entries / ms / 1e6)
    ms = _time(lambda: mu.packedmask_to_indexmask_cuda(packed, seq=S), reps, warmup)
    _emit(table="stages", stage="packedmask_to_indexmask_cuda", shape=shape, ms=ms,
          gbs=(4 + 1 / 8) * n_entries / ms / 1e6)
    capi.check()


def model_table(reps: int, warmup: int, heads: int = MODEL_HEADS, sdpa: bool = False):
    from . import capi
    from .spattn import sparseattn_functionals as sf
    for label, seq in MODEL_SEQS.items():
        for kind, kv in (("self", None), ("cross", CROSS_KEYS)):
            q, k, v = _qkv(heads, seq, kv)
            flops = 4.0 * heads * seq * k.shape[2] * 128
            ms = _time(lambda: sf.baseline_attn(q, k, v), reps, warmup)
            rec = dict(table="model", label=label, attention=kind, shape=list(q.shape), keys=k.shape[2], ms=ms,
                       tflops=flops / ms / 1e9)
            if sdpa:    # the library call the reference's script times, for context
                ms_lib = _time(lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v), reps, warmup)
                rec["sdpa_ms"] = ms_lib
            _emit(**rec)
            del q, k, v
    capi.check()


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--table", choices=("stages", "model", "all"), default="all")
    ap.add_argument("--heads", type=int, nargs="*", default=None, help="stages: head counts (default 12 40)")
    ap.add_argument("--seq", type=int, nargs="*", default=None, help="stages: sequence lengths (default 32760 75600)")
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--model-heads", type=int, default=MODEL_HEADS, help="model: heads (default 40)")
    ap.add_argument("--sdpa", action="store_true", help="model: also time torch's scaled_dot_product_attention")
    a = ap.parse_args(argv)
    if not torch.cuda.is_available():
        sys.exit("microbench needs a CUDA device")
    if a.table in ("stages", "all"):
        for h in (a.heads or STAGE_HEADS):
            for s in (a.seq or STAGE_SEQS):
                stage_table(h, s, a.reps, a.warmup)
    if a.table in ("model", "all"):
        model_table(a.reps, a.warmup, heads=a.model_heads, sdpa=a.sdpa)


if __name__ == "__main__":
    main()
