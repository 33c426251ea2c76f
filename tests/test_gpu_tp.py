"""Tensor-parallel linears over NCCL on real GPUs (skipped on a one-GPU box): column- and
row-parallel forms are bit-identical to one GPU."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_tp_linears_bit_identical_over_nccl():
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29511", os.path.join(here, "tp_nccl_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "tp_nccl_worker: OK" in p.stdout


def test_tp_decoder_bit_identical_over_nccl():
    """The sharded decoder stack (column-parallel q/k/v and gate/up, row-parallel o/down with an int32
    all-reduce, per-rank KV cache) gives the logits of the one-GPU stack, eagerly and from a CUDA graph."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29512", os.path.join(here, "tp_decoder_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "tp_decoder_worker: OK" in p.stdout


def test_expert_parallel_moe_bit_identical_over_nccl():
    """Experts split over two ranks, tokens and router replicated, fp32 all-reduce of the weighted partial sums:
    the output of the one-GPU block, bit for bit (top-2)."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs")
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29514", os.path.join(here, "ep_moe_worker.py")]
    p = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "ep_moe_worker: OK" in p.stdout
