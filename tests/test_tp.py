"""Tensor-parallel path: world-size-2 gloo ranks on CPU (sharded oracle + collectives), and
NCCL ranks on 2 GPUs when the box has them."""
import os
import socket
import subprocess
import sys

import pytest

from conftest import ROOT


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_ranks(world: int, *worker_args: str, timeout: int = 600, handover: str = ""):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()),
           os.path.join(ROOT, "tests", "tp_worker.py"), *worker_args]
    env = dict(os.environ, OMP_NUM_THREADS="1", NCCL_NVLS_ENABLE="0")
    # "fused" = peer-memory all-reduce + residual + norm kernel (one-shot at 2 ranks, two-shot beyond),
    # "twoshot" = the same with the two-shot kernel at any rank count, "nccl" = library all-reduce
    if handover:
        env["ORION_TP_ALLREDUCE"] = handover
    return subprocess.run(cmd, cwd=ROOT, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                          timeout=timeout)


def test_two_gloo_ranks_reproduce_the_unsharded_forward():
    r = _run_ranks(2, "--mode", "cpu")
    assert r.returncode == 0, r.stdout[-3000:]


def test_four_gloo_ranks_reproduce_the_unsharded_forward():
    r = _run_ranks(4, "--mode", "cpu")
    assert r.returncode == 0, r.stdout[-3000:]


@pytest.mark.gpu
@pytest.mark.parametrize("handover", ["fused", "twoshot", "nccl"])  # twoshot: the kernel of 3+ ranks, forced
@pytest.mark.parametrize("dtype", ["F32", "BF16"])
def test_two_gpu_ranks_match_the_oracle(pkg, dtype, handover):
    if pkg.device_count() < 2:
        pytest.skip("needs two GPUs on the box")
    r = _run_ranks(2, "--mode", "gpu", "--dtype", dtype, handover=handover)
    assert r.returncode == 0, r.stdout[-3000:]


@pytest.mark.gpu
@pytest.mark.parametrize("handover", ["fused", "nccl"])
@pytest.mark.parametrize("dtype", ["F32", "BF16"])
def test_four_gpu_ranks_match_the_oracle(pkg, dtype, handover):
    """One KV head per rank: the widest split the test model allows, and three peers per inbox in
    the fused hand-over."""
    if pkg.device_count() < 4:
        pytest.skip("needs four GPUs on the box")
    r = _run_ranks(4, "--mode", "gpu", "--dtype", dtype, handover=handover)
    assert r.returncode == 0, r.stdout[-3000:]


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("handover", ["fused", "nccl"])
@pytest.mark.parametrize("dtype", ["F32", "BF16"])
def test_ranks_match_the_oracle_on_the_eight_kv_head_model(pkg, dtype, handover, world):
    """The benchmark's own parity model (8 kv heads: whole heads at 2, 4 and 8 ranks): a ragged prefill, a
    mixed batch, a 48-row and a 160-row decode batch; logits of rank 0 and the arena of every rank."""
    if pkg.device_count() < world:
        pytest.skip(f"needs {world} GPUs on the box")
    r = _run_ranks(world, "--mode", "gpu", "--dtype", dtype, "--model", "kv8", handover=handover)
    assert r.returncode == 0, r.stdout[-3000:]


@pytest.mark.gpu
@pytest.mark.parametrize("handover", ["fused", "twoshot"])
def test_two_gpu_ranks_at_one_mi_elements_per_handover(pkg, handover):
    """256 rows x hidden 4096: the size from which the bf16 build hands over in two shots at 2 ranks."""
    if pkg.device_count() < 2:
        pytest.skip("needs two GPUs on the box")
    r = _run_ranks(2, "--mode", "gpu", "--dtype", "BF16", "--model", "wide", handover=handover)
    assert r.returncode == 0, r.stdout[-3000:]


@pytest.mark.gpu
def test_collective_trait_over_nccl_on_two_gpus(pkg):
    """all_reduce_sum / all_gather / reduce_scatter_sum / barrier of the Collective trait through the C boundary."""
    if pkg.device_count() < 2:
        pytest.skip("needs two GPUs on the box")
    r = _run_ranks(2, "--mode", "gpu", "--model", "collective")
    assert r.returncode == 0, r.stdout[-3000:]


@pytest.mark.gpu
def test_collective_of_one_rank_behaves_like_single_rank(pkg):
    """world 1 at the C boundary = SingleRank (lib.rs:257-292): every operation is a copy, no NCCL involved."""
    import numpy as np

    coll = pkg.NcclCollective(pkg.CudaBackend(0), b"", pkg.Rank.single())
    buf = np.arange(7, dtype=np.float32)
    coll.all_reduce_sum(buf)
    assert buf.tolist() == list(range(7))
    out = np.zeros(4, np.float32)
    coll.all_gather(np.array([1, 2, 3, 4], np.float32), out)
    assert out.tolist() == [1, 2, 3, 4]
    coll.reduce_scatter_sum(np.array([5, 6], np.float32), out[:2])
    assert out[:2].tolist() == [5, 6]
    coll.barrier()
    with pytest.raises(pkg.InternalError):
        coll.all_gather(np.zeros(3, np.float32), np.zeros(4, np.float32))
