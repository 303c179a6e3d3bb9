"""Tensor/expert-parallel engine on 2 GPUs (one process per GPU, NCCL bootstrap, peer-memory partial sums)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_tp2_engine_matches_oracle():
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29517", os.path.join(here, "multi", "tp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    sys.stdout.write(r.stdout[-3000:])
    sys.stderr.write(r.stderr[-3000:])
    assert r.returncode == 0
    assert "TP_WORKER_OK" in r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_allgather_gemm_and_gemm_reducescatter():
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", TP_ROWS="512", TP_K="1024", TP_N="1024", TP_REPS="3")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29519", os.path.join(here, "multi", "tp_linear_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    sys.stdout.write(r.stdout[-3000:])
    sys.stderr.write(r.stderr[-3000:])
    assert r.returncode == 0 and "TP_LINEAR_OK" in r.stdout


def _run_ep(nproc: int, port: int, **env_extra):
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **env_extra)
    worker = os.path.join(here, "multi", "ep_worker.py")
    if nproc == 1:
        cmd = [sys.executable, worker]
    else:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
               "--master-addr", "127.0.0.1", "--master-port", str(port), worker]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    sys.stdout.write(r.stdout[-3000:])
    sys.stderr.write(r.stderr[-3000:])
    assert r.returncode == 0 and "EP_OK" in r.stdout


@pytest.mark.parametrize("mx", ["0", "1"])
def test_grouped_experts_one_rank(mx):
    """Tile-table grouped GEMMs and the scatter epilogue with every expert local (no peers)."""
    _run_ep(1, 0, EP_TOKENS="384", EP_H="512", EP_I="256", EP_E="8", EP_TOPK="4", EP_REPS="2", EP_MX=mx)
    if mx == "1":
        _run_ep(1, 0, EP_TOKENS="384", EP_H="512", EP_I="256", EP_E="8", EP_TOPK="4", EP_REPS="2", EP_MX=mx,
                EP_WIRE="bf16")
        # 192-token expert tiles: block-scaled MMAs of N = 192 (and narrower ones for partly filled tiles) whose token
        # scales span two scale atoms
        _run_ep(1, 0, EP_TOKENS="1000", EP_H="1024", EP_I="512", EP_E="16", EP_TOPK="6", EP_REPS="2", EP_MX=mx,
                EP_TILE="192")


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("mx,wire", [("0", "auto"), ("1", "fp8"), ("1", "bf16")])
def test_expert_parallel_dispatch_gemm_combine(mx, wire):
    """wire "fp8": the sender quantises each row inside the dispatch kernel and stores it into the owner's FC1 operand
    buffers; "bf16": bf16 rows travel and the owner quantises what it received."""
    _run_ep(2, 29521, EP_TOKENS="384", EP_H="512", EP_I="256", EP_E="8", EP_TOPK="4", EP_REPS="2", EP_MX=mx,
            EP_WIRE=wire)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_serving_backend_with_mirrored_ranks():
    """Rank 0 schedules and samples; rank 1 mirrors every engine call (set_rows / forward / logits gather / pages)."""
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29523", os.path.join(here, "multi", "serve_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    sys.stdout.write(r.stdout[-3000:])
    sys.stderr.write(r.stderr[-3000:])
    assert r.returncode == 0 and "SERVE_WORKER_OK" in r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_stage_pipeline_over_peer_memory():
    here = os.path.dirname(os.path.abspath(__file__))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29531", os.path.join(here, "multi", "pp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    sys.stdout.write(r.stdout[-3000:])
    sys.stderr.write(r.stderr[-3000:])
    assert r.returncode == 0 and "PP_WORKER_OK" in r.stdout
