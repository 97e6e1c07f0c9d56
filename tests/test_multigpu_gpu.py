"""Multi-GPU tests (need >= 2 GPUs): fused peer-memory all-reduce vs NCCL, and dp / tp / pp plans on real GPUs.
Each test launches child ranks with torch.distributed.run on 127.0.0.1."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _launch(mode: str, n: int = 2, **extra_env):
    env = dict(os.environ, NCCL_NVLS_ENABLE=os.environ.get("NCCL_NVLS_ENABLE", "1"), **extra_env)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", "29731", os.path.join(HERE, "multigpu_worker.py"), mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=420, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_allreduce_matches_nccl():
    assert "ALLREDUCE_OK" in _launch("allreduce")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_dp_tp_pp_training_on_two_gpus():
    assert "TRAIN_OK" in _launch("train")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_gemm_allreduce_matches_gemm_plus_nccl():
    assert "GEMM_AR_OK" in _launch("gemm_ar")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_allgather_gemm_matches_allgather_plus_gemm():
    assert "AG_GEMM_OK" in _launch("ag_gemm")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_gemm_reduce_scatter_matches_gemm_plus_nccl():
    assert "GEMM_RS_OK" in _launch("gemm_rs")


@pytest.mark.parametrize("mode,ok", [("allreduce", "ALLREDUCE_OK"), ("gemm_ar", "GEMM_AR_OK"), ("ag_gemm", "AG_GEMM_OK"),
                                     ("gemm_rs", "GEMM_RS_OK")])
def test_fused_collective_kernels_on_four_gpus(mode, ok):
    """The same checks at tensor-parallel degree 4: three peers per rank, four owners of output slices."""
    if torch.cuda.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    assert ok in _launch(mode, n=4)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_guard_words_around_symmetric_buffers_survive_the_collectives():
    """With SSB_CANARIES=1 the symmetric buffers sit 256 bytes into guarded allocations: the all-reduce, the
    reduce-scatter / all-gather of the sharded update and a whole data-parallel training run must give the same
    results through the shifted peer and multicast addresses and leave every guard word as it was."""
    out = _launch("allreduce", SSB_CANARIES="1")
    assert "ALLREDUCE_OK" in out and "GUARDS_OK" in out
    out = _launch("train", SSB_CANARIES="1")
    assert "TRAIN_OK" in out and "GUARDS_OK" in out
