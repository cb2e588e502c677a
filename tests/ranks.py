"""Helpers of the tests that start one process per GPU."""
import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def run_ranks(child: str, world: int, port: int, expect: str):
    """Run tests/<child> as `world` torchrun ranks on this machine's GPUs (NVLS off: a rank that dies
    while bound to a multicast object can fault its peers) and require its closing line."""
    import subprocess
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", str(port), str(ROOT / "tests" / child)]
    out = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert expect in out.stdout


def gpu_count() -> int:
    try:
        import torch
        return torch.cuda.device_count()
    except Exception:
        return 0
