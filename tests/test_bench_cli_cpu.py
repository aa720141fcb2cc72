"""CPU checks of the command-line contracts around the benchmarks (no GPU needed)."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_arm_reports_unavailable():
    """`bench.py --impl reference` must exit 0 with one JSON line that says why the reference cannot run."""
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "1",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr[-2000:]
    line = [ln for ln in out.stdout.splitlines() if ln.startswith("{")][-1]
    d = json.loads(line)
    assert d["impl"] == "reference" and isinstance(d.get("unavailable"), str) and d["unavailable"]


def test_bench_configs_cover_the_named_shapes():
    sys.path.insert(0, ROOT)
    import bench
    full = bench.CONFIGS["full"]
    assert (full["tokens"], full["hidden"], full["experts_per_rank"], full["topk"], full["ffn"]) == (8192, 2048, 8, 6, 1408)
    scaling = bench.CONFIGS["scaling"]
    assert (scaling["tokens"], scaling["hidden"], scaling["experts_total"], scaling["topk"], scaling["ffn"],
            scaling["layers"]) == (16384, 4096, 8, 2, 14336, 3)
    skewed = bench.CONFIGS["skewed"]
    assert skewed["tokens"] == (2048, 6144) and skewed["routing"] == "zipf" and skewed["ckpt_level"] == 1
    assert (skewed["hidden"], skewed["experts_per_rank"], skewed["topk"], skewed["ffn"]) == (7168, 32, 8, 2048)


def test_comm_bench_routing_is_distinct_and_normalised():
    from streamep_b200.comm_bench import make_uniform_routing
    idx, w = make_uniform_routing(257, 8, 64, seed=3, dev="cpu")
    assert idx.shape == (257, 8) and idx.dtype == torch.int64
    assert int(idx.min()) >= 0 and int(idx.max()) < 64
    assert all(len(set(row.tolist())) == 8 for row in idx)
    assert torch.allclose(w.sum(-1), torch.ones(257))
