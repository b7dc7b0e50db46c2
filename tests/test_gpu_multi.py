"""Feature-sharded step on 2 GPUs against the unsharded CPU oracle (skipped with fewer than 2 GPUs)."""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


CASES = [(k, p, "nccl") for k in ("jumprelu", "topk", "batchtopk") for p in ("fp32", "bf16")]
# exchange fused into the kernels over peer memory
CASES += [(k, p, "fused") for k in ("jumprelu", "topk", "batchtopk") for p in ("fp32", "bf16")]


@pytest.mark.parametrize("kind,prec,mode", CASES)
def test_two_shards_match_unsharded_oracle(kind, prec, mode):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29533", str(ROOT / "tests" / "mp_worker.py"), kind, prec, mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.parametrize("join", ["early", "late"])
@pytest.mark.parametrize("kind", ["topk", "batchtopk"])
def test_sharded_batch_uploader_feeds_the_same_steps(kind, join):
    """parallel.ShardedBatchUploader (each rank uploads its token rows, peers receive the input halves) against
    whole device batches: identical losses and parameters over three optimizer steps, with both ways of ordering
    the peer copies."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29534", str(ROOT / "tests" / "mp_worker.py"), kind, "bf16", "fused", join]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
