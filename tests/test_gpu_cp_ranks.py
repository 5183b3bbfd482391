"""Context parallelism ACROSS GPUs: two ranks (one process per GPU, NCCL) each own a token shard of one sequence; the
per-rank affine state maps are all-gathered, scanned and the outputs fixed up.  Compared on every rank with the fp64
recurrence (equal and cost-balanced shards, slow gates included).  Skipped when fewer than two GPUs are visible."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_two_rank_context_parallel_matches_the_recurrence():
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    worker = Path(__file__).resolve().parent / "cp_ranks_worker.py"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    res = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29517", str(worker)],
                         capture_output=True, text=True, timeout=600, env=env)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert res.stdout.count("context-parallel parity ok") == 2
