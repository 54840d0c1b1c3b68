"""The comparison harness writes the reference's result layout (test/test_speedup.py:208-238) and skips configurations
that are already in the file (test/test_speedup.py:53-69)."""
import json

import pytest
import torch

KEYS = {"flash_attn_base_result", "hbsattn(our fix)", "hbsattn(our auto)", "hanlab_block-sparse-attn", "flexattention",
        "unit_seqlen", "headdim", "nhead_q", "causal", "sparse_ratio"}


def test_resume_skip_and_append(tmp_path):
    from hbsattn_b200 import speed_sweep
    path = str(tmp_path / "res.json")
    cfg = {"unit_seqlen": 256, "headdim": 128, "nhead_q": 4, "causal": True, "sparse_ratio": 0.9}
    assert not speed_sweep.already_there(path, cfg)
    assert speed_sweep.append_result(path, dict(cfg, **{"hbsattn(our fix)": {"runtime_mean": 1.0}})) == 1
    assert speed_sweep.already_there(path, cfg)
    assert not speed_sweep.already_there(path, dict(cfg, unit_seqlen=512))
    assert speed_sweep.append_result(path, dict(cfg, unit_seqlen=512)) == 2
    # a second run of an existing configuration leaves the file alone and needs no GPU
    assert speed_sweep.main(["--causal", "--unit_seqlen", "256", "--nheads", "4", "--sparse_ratio", "0.9", "--save_benchmark_to_file", path]) == 0
    assert len(json.load(open(path))) == 2


@pytest.mark.gpu
def test_sweep_entry_layout(tmp_path):
    from hbsattn_b200 import speed_sweep
    path = str(tmp_path / "res.json")
    argv = ["--causal", "--unit_seqlen", "512", "--nheads", "2", "--batch_size", "2", "--sparse_ratio", "0.5", "--nruns", "3",
            "--nwarmup", "1", "--no_flex", "--save_benchmark_to_file", path]
    assert speed_sweep.main(argv) == 0
    (entry,) = json.load(open(path))
    assert KEYS <= set(entry)
    for col in ("hbsattn(our fix)", "hbsattn(our auto)"):
        r = entry[col]
        assert set(r) == {"runtime_mean", "runtime_std", "runtime_min", "runtime_max", "all_times", "error"}
        assert len(r["all_times"]) == 2 and r["runtime_min"] > 0
    assert entry["hanlab_block-sparse-attn"] == {}
    assert torch.cuda.is_available()
