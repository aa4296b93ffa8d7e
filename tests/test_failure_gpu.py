"""Failure detection without faulting a GPU: waits that run out return an error
status and leave the context usable; a rank that launches late makes its peer's
short deadline expire, and a collective reset brings both back."""
import os
import subprocess
import sys

import pytest
import torch

import flashoverlap_b200  # noqa: F401

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def test_wait_that_nothing_satisfies_times_out_with_status():
    impl = torch.classes.flashoverlap_class.OverlapImpl()
    impl.nccl_init(0, 1, [0] * 16)
    impl.cutlass_init()
    impl.wait_on_unset_counter(200)
    torch.cuda.synchronize()
    st = impl.status()
    assert st[0] == 2 and st[4] == 1, impl.status_string()  # ST_TIMEOUT_FLAG, wanted 1
    with pytest.raises(RuntimeError, match="did not arrive"):
        impl.check_status()
    # the next operation refuses to run on top of a reported failure, without anybody asking for the status
    A = torch.randn(256, 128, device="cuda", dtype=torch.float16)
    B = torch.randn(256, 128, device="cuda", dtype=torch.float16)
    C = torch.empty(256, 256, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError, match="earlier flashoverlap kernel reported a failure"):
        impl.cutlass_gemm(A, B, C, 0)
    impl.reset()
    assert impl.status()[0] == 0
    # the context is still usable
    impl.cutlass_gemm(A, B, C, 0)
    torch.cuda.synchronize()
    impl.check_status()
    assert (C.float() - A.float() @ B.float().t()).abs().max().item() < 0.1


@pytest.mark.timeout(300)
def test_late_rank_trips_short_deadline_and_reset_recovers():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0", FLASHOVERLAP_NVLS="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr",
           "127.0.0.1", "--master-port", "29544", os.path.join(HERE, "failure_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=280)
    tail = "\n".join((res.stdout + "\n" + res.stderr).splitlines()[-40:])
    assert res.returncode == 0, tail
    assert "rank 0 timed out as expected" in res.stdout, tail
    assert "recovered" in res.stdout, tail
