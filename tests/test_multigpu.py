"""Runs the multi-GPU correctness worker under torchrun on every GPU of the
node (2, 4 or 8); skipped on a single-GPU machine."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _world():
    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    for w in (8, 4, 2):
        if n >= w:
            return w
    return 0


@pytest.mark.timeout(900)
@pytest.mark.parametrize("nvls", ["1", "0"], ids=["nvls", "p2p"])
def test_fused_ops_match_torch_semantics_on_all_gpus(nvls):
    world = _world()
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    env = dict(os.environ)
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    env["FLASHOVERLAP_NVLS"] = nvls
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29533", os.path.join(HERE, "mgpu_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=850)
    tail = "\n".join((res.stdout + "\n" + res.stderr).splitlines()[-60:])
    assert res.returncode == 0, tail
    assert "DONE failures=0" in res.stdout, tail
    if nvls == "0":
        assert "mode: P2P stores" in res.stdout, tail


@pytest.mark.timeout(600)
def test_hierarchical_path_with_pretend_nodes():
    """Fused kernel inside a node, NCCL across nodes: the GPUs of this machine
    are cut into two pretend nodes."""
    world = _world()
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    env = dict(os.environ)
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    env["FLASHOVERLAP_FAKE_NODES"] = "2"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", "29535", os.path.join(HERE, "hier_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=550)
    tail = "\n".join((res.stdout + "\n" + res.stderr).splitlines()[-40:])
    assert res.returncode == 0, tail
    assert "DONE failures=0" in res.stdout, tail
