"""Launches the multi-process NVLink checks when the box has at least two GPUs."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least 2 GPUs")
def test_multiprocess_nvlink_paths():
    n = 8 if torch.cuda.device_count() >= 8 else (4 if torch.cuda.device_count() >= 4 else 2)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29533",
           os.path.join(ROOT, "tests", "multigpu", "layer_check.py")]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    sys.stdout.write(out.stdout[-6000:])
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "ALL PASS" in out.stdout
    # the same layer and capacity-mode checks with the arena on the VMM allocator (descriptors over Unix sockets)
    out = subprocess.run(cmd + ["--allocator", "vmm", "--scenario", "capacity"], capture_output=True, text=True,
                         timeout=900, env=env)
    sys.stdout.write(out.stdout[-3000:])
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "ALL PASS" in out.stdout and "arena allocator: vmm" in out.stdout
