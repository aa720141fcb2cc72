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


def test_kernel_timing_summary_reads_every_stamp_column():
    """The per-CTA stamp rows ([SMs, 12] int64) are turned into the figures the timing harness prints."""
    from streamep_b200.stream_moe.kernel_timing import summarise
    t = torch.zeros(4, 12, dtype=torch.int64)
    assert summarise(t) == {}                                  # no CTA left a start stamp: that kind was not launched
    #           start  gate_ns first  tiles@push push0 push1  end    tiles  mma_total mma_ops mma_acc spare
    t[0] = torch.tensor([1000, 2000, 3000, 2, 1500, 9000, 11000, 7, 10000, 2500, 100, 0])
    t[1] = torch.tensor([1400, 4000, 5000, 4, 1600, 7000, 21000, 9, 20000, 5000, 200, 0])
    t[2] = torch.tensor([1200, 0, 0, 0, 0, 0, 15000, 0, 0, 0, 0, 0])   # a push-only CTA without gates or MMAs
    s = summarise(t)
    assert s["ctas"] == 3 and abs(s["kernel_us"] - 20.0) < 1e-9 and abs(s["start_skew_us"] - 0.4) < 1e-9
    assert abs(s["gate_wait_us_mean"] - 2.0) < 1e-9 and abs(s["gate_wait_us_max"] - 4.0) < 1e-9
    assert abs(s["first_tile_ready_us_mean"] - 3.0) < 1e-9      # (2.0 + 4.0) / 2 us after the earliest start
    assert abs(s["push_end_us_max"] - 8.0) < 1e-9 and abs(s["tiles_done_at_push_end"] - 3.0) < 1e-9
    assert abs(s["mma_wait_operands_frac"] - 0.25) < 1e-9 and abs(s["mma_wait_accumulator_frac"] - 0.01) < 1e-9
