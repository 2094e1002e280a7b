#!/usr/bin/env python
"""Benchmark of the threshold block-sparse attention forward path on B200.

One "step" = one block-sparse forward pass (sp_attn_blocks_ml: gather of the listed K/V tiles +
softmax with the precomputed max_q / denom + P*V) over one batch of the workload, with the key-block
lists and (max_q, denom) built once, untimed, by the library's own one-pass mask pipeline.
Metric: TFLOP/s on kept 64x64 blocks (4*64*64*D flops per kept block).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c3] [--impl reference]

For N > 1 launch under `python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N`;
every rank runs the full workload on its own heads (weak scaling, no collective on the data path).
Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

METRIC = "sparse_fwd_tflops_on_kept_blocks"
UNIT = "TFLOP/s"


def read_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"bf16_tflops": float(d["bf16_tflops"]), "bf16_tflops_sustained": float(d["bf16_tflops_sustained"]),
                "hbm_gbs": float(d["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.004):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.nv = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        names = {
            nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
            nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
            nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
            nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake",
        }
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(s)}


def physical_gpu_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


# --------------------------------------------------------------------------------------------------
# reference arm / cpu baseline: the CPU port of the reference's PyTorch path on a bounded sample
# --------------------------------------------------------------------------------------------------
def cpu_sample(workload, rows: int):
    """One head of the workload, the first `rows` query rows against all keys."""
    from fgattn_tk_cuda_b200 import synth
    q, k, v = synth.make_qkv(workload, device="cpu", heads=range(1))
    q, k, v = q.float(), k.float(), v.float()
    return q[:, :, :rows].contiguous(), k, v


def cpu_step(q_rows, k, v, tau):
    """The reference's CPU path for the sparse step on the sample: softmax over all keys, 64x64
    threshold block map, masked P*V without renormalisation (python/spattn/mask_utils.py:206-245,
    python/test_mask.py:37-54), through the oracle port.  Returns kept blocks."""
    from oracle import fgattn_oracle as orc
    S_kv = k.shape[2]
    kk = k
    # the oracle functions take q and k of equal length only for shape bookkeeping of m/l; the
    # block map and the masked attention work on any number of query rows
    bm = orc.qk_block_bitmask(q_rows, kk, tau, 64, 64, kv_seq_len=S_kv)
    orc.block_masked_attn(q_rows, kk, v, bm, 64, 64, kv_seq_len=S_kv)
    return int(bm.sum())


def run_cpu(workload, steps: int, warmup: int, budget_s: float):
    torch.set_num_threads(os.cpu_count() or 1)
    cores = torch.get_num_threads()
    D = workload.D
    # calibrate the sample size (query rows) against the time budget
    q, k, v = cpu_sample(workload, 256)
    t0 = time.perf_counter()
    cpu_step(q, k, v, workload.tau)
    t256 = time.perf_counter() - t0
    per_step = budget_s / max(1, steps + warmup)
    rows = int(max(64, min(workload.S, (per_step / max(t256, 1e-6)) * 256)) // 64 * 64)
    q, k, v = cpu_sample(workload, rows)
    for _ in range(warmup):
        cpu_step(q, k, v, workload.tau)
    times, kept = [], 0
    for _ in range(steps):
        t0 = time.perf_counter()
        kept = cpu_step(q, k, v, workload.tau)
        times.append(time.perf_counter() - t0)
    mean_s = sum(times) / len(times)
    flops = 4.0 * 64 * 64 * D * kept
    return {"value": flops / mean_s / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
            "sample": f"head 0 of {workload.name}, first {rows} query rows x all {workload.S} keys, fp32 torch CPU: "
                      f"threshold block map + masked attention; {mean_s:.2f} s per step, {kept} kept blocks",
            "ms_per_step": mean_s * 1e3}


# --------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c3")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--heads", type=int, default=0, help="profile-sized run: only the first N heads (B=1)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    from fgattn_tk_cuda_b200 import synth
    w = synth.WORKLOADS[args.workload]
    if args.heads > 0:
        import dataclasses
        w = dataclasses.replace(w, name=f"{w.name}_first{args.heads}heads", B=1, H=args.heads)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    config = {"workload": w.name, "B": w.B, "H": w.H, "S": w.S, "D": w.D, "block": "64x64", "tau": w.tau,
              "units_per_gpu": f"{w.B * w.H} (batch x head) units", "partition": f"replicated workload x{world}, "
              "disjoint head seeds per rank, no collective", "l2": f"inputs ({4 * w.B * w.H * w.S * w.D * 2 >> 20} MiB of q,k,v,o) larger than L2, no flush"}

    if args.impl == "reference":
        if rank != 0:
            return
        steps = min(args.steps, 20)
        r = run_cpu(w, steps, min(args.warmup, 3), budget_s=150.0)
        line = {"impl": "reference", "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus,
                "steps": steps, "warmup": min(args.warmup, 3), "ms_per_step": r["ms_per_step"],
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": config,
                "cpu_baseline": {k_: r[k_] for k_ in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    from fgattn_tk_cuda_b200 import capi
    import fgattn_tk_cuda_b200.spattn as spattn            # registers torch.ops.cuda_attn (the plugin boundary)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)

    peaks = read_peaks()
    n_heads = w.B * w.H
    heads = range(rank * n_heads, (rank + 1) * n_heads)    # disjoint seeds per rank, same shapes
    q, k, v = synth.make_qkv(w, device=dev, heads=heads)
    q, k, v = (t.view(w.B, w.H, w.S, w.D) for t in (q, k, v))
    B, H, S, D = q.shape
    nqb = nkb = (S + 63) // 64

    # ---- untimed set-up: one-pass m/l + lists (+ dense output), timed separately for the report
    def ev_time(fn, n, warm):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    o = torch.empty_like(q)
    idx, cnt, max_q, denom = spattn.mask_utils.qk_block_indexmask_cuda(q, k, w.tau)
    capi.check()
    nnz = int(cnt.sum().item())
    density = nnz / (B * H * nqb * nkb)
    F_sparse = 4.0 * 64 * 64 * D * nnz
    F_full = 4.0 * B * H * S * S * D
    scratch = spattn.mask_utils._block_scratch(q)
    ms_full = ev_time(lambda: capi.full_attn(o, q, k, v), 5, 2)
    ms_lists = ev_time(lambda: capi.block_index_lists(idx, cnt, max_q, denom, q, k, w.tau, scratch), 5, 2)
    ms_maxq = ev_time(lambda: capi.maxq_denom(max_q, denom, q, k), 5, 2)
    s_pad = 128 * ((S + 127) // 128)
    mask_bytes = B * H * (4.0 * s_pad * nkb * 2 + 8.0 * S + 4.0 * nqb * nkb + 4.0 * nqb)
    ms_build = ev_time(lambda: capi.block_index_lists(idx, cnt, max_q, denom, q, k, w.tau, scratch, o=o, v=v), 5, 2)
    # one-bit-per-entry mask kernels on a token mask of the reference granularity (int32 [B,H,S/128,S_pad],
    # 8 % kept): pack = 4 B read + 1/8 B written per entry; packed -> lists = 1/8 B read + 4 B written
    tmask = (torch.rand(B, H, (S + 127) // 128, s_pad, device=dev) < 0.08).to(torch.int32)
    # threshold token mask (reference granularity): the full second Q K^T pass against the pass that only
    # visits the kept 64x64 blocks
    ms_tokmask = ev_time(lambda: capi.booleanmask_128(tmask, max_q, denom, q, k, w.tau), 3, 1)
    ms_tokmask_listed = ev_time(lambda: capi.booleanmask_128_listed(tmask, max_q, denom, q, k, w.tau, idx, cnt), 5, 2)
    # the reference's sparse operator on the threshold token lists of that mask (lists of very different lengths)
    thr_idx = torch.empty_like(tmask)
    thr_cnt = torch.empty(tmask.shape[:3], dtype=torch.int32, device=dev)
    capi.booleanmask_to_indexmask(thr_idx, thr_cnt, tmask, S)
    ms_tok_thr = ev_time(lambda: capi.sp_attn(o, q, k, v, thr_idx, thr_cnt), 5, 2)
    F_tok_thr = 4.0 * 128 * D * float(thr_cnt.sum().item())
    del thr_idx, thr_cnt
    tmask = (torch.rand(B, H, (S + 127) // 128, s_pad, device=dev) < 0.08).to(torch.int32)
    tpacked = torch.empty(B, H, tmask.shape[2], s_pad // 8, dtype=torch.uint8, device=dev)
    tidx = torch.empty_like(tmask)
    tcnt = torch.empty(tmask.shape[:3], dtype=torch.int32, device=dev)
    pack_bytes = tmask.numel() * (4.0 + 0.125)
    ms_pack = ev_time(lambda: capi.pack_mask(tpacked, tmask), 10, 3)
    ms_p2i = ev_time(lambda: capi.packedmask_to_indexmask(tidx, tcnt, tpacked, S), 10, 3)
    ms_m2i = ev_time(lambda: capi.booleanmask_to_indexmask(tidx, tcnt, tmask, S), 10, 3)
    del tmask, tidx
    # top-k selector at the reference granularity: 128-row query blocks, 10 % of the keys
    sel_k = max(1, S // 10)
    kstride = 128 * ((sel_k + 127) // 128)
    kidx = torch.empty(B, H, (S + 127) // 128, kstride, dtype=torch.int32, device=dev)
    tk_scratch = torch.empty(capi.topk_scratch_bytes(B, H, S, D, 128), dtype=torch.uint8, device=dev)
    ms_topk = ev_time(lambda: capi.topk_indices(kidx, tcnt, q, k, sel_k, blocksz=128, scratch=tk_scratch), 5, 2)
    # the reference's own sparse operator (128-row query blocks, key-token lists, renormalising) on those lists
    ms_tok = ev_time(lambda: capi.sp_attn(o, q, k, v, kidx, tcnt), 5, 2)
    F_tok = 4.0 * B * H * S * sel_k * D
    del kidx, tk_scratch
    # replay of a cached mask: the renormalising block kernel on the same key-block lists
    ms_renorm = ev_time(lambda: torch.ops.cuda_attn.sp_attn_blocks(o, q, k, v, idx, cnt), 10, 3)

    step = lambda: torch.ops.cuda_attn.sp_attn_blocks_ml(o, q, k, v, idx, cnt, max_q, denom)  # noqa: E731

    def barrier():
        if world > 1:
            torch.distributed.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    clocks = sampler.stop()
    capi.check()
    ms_step = e0.elapsed_time(e1) / args.steps

    # ---- end to end through the operator boundary with host buffers
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty(o.shape, dtype=o.dtype).pin_memory()
    # Every step copies its own q, k, v from pinned host memory, runs the operator and reads o back.
    # Steps are independent, so they are double-buffered over three streams: the copies of step i+1
    # and the read-back of step i-1 overlap the kernel of step i (H2D and D2H use different engines).
    cur = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    dbuf = [tuple(torch.empty_like(t) for t in (q, k, v, o)) for _ in range(2)]
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_comp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def e2e_step(i):
        b = i & 1
        bq, bk, bv, bo = dbuf[b]
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_comp[b])                 # the kernel of step i-2 has read this buffer
            bq.copy_(hq, non_blocking=True)
            bk.copy_(hk, non_blocking=True)
            bv.copy_(hv, non_blocking=True)
            ev_in[b].record(s_in)
        cur.wait_event(ev_in[b])
        cur.wait_event(ev_out[b])                       # o of step i-2 has been read back
        torch.ops.cuda_attn.sp_attn_blocks_ml(bo, bq, bk, bv, idx, cnt, max_q, denom)
        ev_comp[b].record(cur)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[b])
            ho.copy_(bo, non_blocking=True)
            ev_out[b].record(s_out)

    def e2e_run(n):
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(cur)
        for i in range(n):
            e2e_step(i)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
        e1.record(cur)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    e2e_steps = max(4, min(args.steps, 10))
    e2e_run(2)
    ms_e2e = e2e_run(e2e_steps)
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv))
    d2h = ho.numel() * ho.element_size()

    # ---- max over ranks
    ms_all, ms_e2e_all, F_total = ms_step, ms_e2e, F_sparse
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms_step, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        f = torch.tensor([F_sparse], device=dev, dtype=torch.float64)
        dist.all_reduce(f, op=dist.ReduceOp.SUM)
        ms_all, ms_e2e_all, F_total = t[0].item(), t[1].item(), f[0].item()

    if rank == 0:
        achieved = F_sparse / ms_step / 1e9                 # this rank's kernel, TFLOP/s
        peak = peaks["bf16_tflops"]
        line = {
            "metric": METRIC, "value": F_total / ms_all / 1e9, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_all, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
            "density": density, "kept_blocks_per_gpu": nnz,
            "e2e": {"value": F_total / ms_e2e_all / 1e9, "unit": UNIT, "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e_all,
                    "api": "torch.ops.cuda_attn.sp_attn_blocks_ml on q, k, v copied from pinned host memory each step, "
                           "o read back each step; steps double-buffered over copy-in / compute / copy-out streams"},
            "gpu_launches": 2 * args.steps,          # per step: sparse_order_kernel + sparse_ml_persistent_kernel
            "clocks": clocks,
            "roofline": {"bound": "tensor", "kernel": "sparse_ml_persistent_kernel<128>", "achieved": achieved,
                         "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
                         "peak_source": f"{peaks['source']} bf16_tflops (burst: kernel timed alone)",
                         "frac_of_sustained": achieved / peaks["bf16_tflops_sustained"], "traffic": None},
            "stages": {
                "full_attn_ms": ms_full, "full_attn_tflops": F_full / ms_full / 1e9,
                "full_attn_frac_of_peak": F_full / ms_full / 1e9 / peak,
                "block_lists_ms": ms_lists, "block_lists_qk_tflops": F_full / 2 / ms_lists / 1e9,
                "maxq_denom_ms": ms_maxq, "maxq_denom_qk_tflops": F_full / 2 / ms_maxq / 1e9,
                "mask_epilogue_note": "block_lists_ms - maxq_denom_ms (difference of two timings; the compaction "
                                      "kernel alone is profiled in profiles/block_threshold_compact_c3_16heads.md)",
                "mask_epilogue_ms": ms_lists - ms_maxq,
                "mask_epilogue_gbs": mask_bytes / max(ms_lists - ms_maxq, 1e-6) / 1e6,
                "mask_epilogue_frac_of_hbm_peak": mask_bytes / max(ms_lists - ms_maxq, 1e-6) / 1e6 / peaks["hbm_gbs"],
                "booleanmask_128_ms": ms_tokmask, "booleanmask_128_listed_ms": ms_tokmask_listed,
                "pack_mask_ms": ms_pack, "pack_mask_gbs": pack_bytes / ms_pack / 1e6,
                "pack_mask_frac_of_hbm_peak": pack_bytes / ms_pack / 1e6 / peaks["hbm_gbs"],
                "packedmask_to_indexmask_ms": ms_p2i, "packedmask_to_indexmask_gbs": pack_bytes / ms_p2i / 1e6,
                "packedmask_to_indexmask_frac_of_hbm_peak": pack_bytes / ms_p2i / 1e6 / peaks["hbm_gbs"],
                "booleanmask_to_indexmask_ms": ms_m2i, "booleanmask_to_indexmask_gbs": pack_bytes / 4.125 * 8 / ms_m2i / 1e6,
                "topk_indices_ms": ms_topk, "topk_select_k": sel_k,
                "sp_attn_threshold_tokens_ms": ms_tok_thr,
                "sp_attn_threshold_tokens_tflops_on_listed_tokens": F_tok_thr / ms_tok_thr / 1e9,
                "sp_attn_tokens_ms": ms_tok, "sp_attn_tokens_tflops_on_listed_tokens": F_tok / ms_tok / 1e9,
                "sp_attn_blocks_renorm_ms": ms_renorm,
                "sp_attn_blocks_renorm_tflops_on_kept_blocks": F_sparse / ms_renorm / 1e9,
                "dense_plus_lists_ms": ms_build, "dense_plus_lists_tflops": F_full / ms_build / 1e9,
                "sparse_ms": ms_step, "sparse_speedup_over_full": ms_full / ms_step,
                "ideal_speedup_1_over_density": 1.0 / density,
                "speedup_gap": (1.0 / density) / (ms_full / ms_step)},
        }
        # dram__bytes_read + dram__bytes_write of one launch, from the ncu capture summarised in
        # profiles/sparse_ml_persistent_c3_16heads.md (16 heads: 312 MB), scaled by heads
        if args.workload == "c3":
            line["roofline"]["traffic"] = 312.0e6 * (w.B * w.H) / 16.0
        if world == 1 and not args.no_cpu_baseline:
            r = run_cpu(w, steps=2, warmup=1, budget_s=25.0)
            line["cpu_baseline"] = {k_: r[k_] for k_ in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line))
    if world > 1:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
