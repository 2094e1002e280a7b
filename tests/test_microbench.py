"""The stage-timing script that mirrors the reference's benchmark scripts (python/benchmark.py,
microbench.py): shape tables on the CPU, one small run of every stage on the GPU."""
import json

import pytest


def test_shape_tables_follow_the_reference_scripts():
    from fgattn_tk_cuda_b200 import microbench as mb
    assert mb.STAGE_HEADS == (12, 40) and mb.STAGE_SEQS == (32760, 75600)          # python/benchmark.py:117-118
    assert list(mb.MODEL_SEQS.values()) == [20280, 32768, 45832, 74056] and mb.MODEL_HEADS == 40
    lens = mb.sweep_lengths(32760)
    assert len(lens) == 16 and lens[0] == 0 and lens[1] == 4 * (32760 // 64) and lens[-1] < 32760


@pytest.mark.gpu
def test_every_stage_runs_on_a_small_shape(capsys):
    from fgattn_tk_cuda_b200 import microbench as mb
    mb.stage_table(2, 1000, reps=1, warmup=1, sweep=[0, 100, 1000])
    mb.model_table(reps=1, warmup=1, heads=1, sdpa=False)
    recs = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    stages = [r["stage"] for r in recs if r["table"] == "stages"]
    for name in ("fullattn_maxq_denom", "full_attn", "sp_attn", "qk_indexmask_cuda", "sp_attn_threshold_lists",
                 "bitmask_to_indexmask_cuda", "pack", "unpack", "packedmask_to_indexmask_cuda"):
        assert name in stages
    model = [r for r in recs if r["table"] == "model"]
    assert len(model) == 8 and {r["keys"] for r in model if r["attention"] == "cross"} == {512}
    assert all(r["ms"] > 0 for r in recs)
