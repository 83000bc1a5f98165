"""The fused peer exchange on 2 GPUs (skipped on machines with fewer): launches tests/exchange_check.py
the way multi-GPU jobs are launched, one process per GPU under torch.distributed.run."""
import os
import socket
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu


def _run_on_two_gpus(script_name):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    script = os.path.join(os.path.dirname(os.path.abspath(__file__)), script_name)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(port), script]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=170)
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-2000:]
    assert "rank 0: OK" in out and "rank 1: OK" in out, out[-2000:]


def test_peer_exchange_matches_nccl_all_gather():
    _run_on_two_gpus("exchange_check.py")


def test_sharded_decode_session_matches_the_unsharded_model():
    _run_on_two_gpus("sharded_decode_check.py")
