"""Multi-process CPU tests on the gloo backend: the plumbing config of the
headline benchmark (world size 2 and 3) and a host-side failure injection (a
rank that never joins the collective)."""
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def run(world, mode, port, timeout_s="60"):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", FO_TEST_TIMEOUT=timeout_s, CUDA_VISIBLE_DEVICES="")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "gloo_worker.py"), mode]
    return subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)


@pytest.mark.parametrize("world", [2, 4])
def test_fused_semantics_on_gloo(world):
    res = run(world, "golden", 29610 + world)
    tail = "\n".join((res.stdout + res.stderr).splitlines()[-40:])
    assert res.returncode == 0, tail
    assert "FAIL" not in res.stdout, tail
    assert res.stdout.count("PASS") == 9 * world, tail


def test_rank_that_never_joins_is_an_error_not_a_hang():
    res = run(2, "never_joins", 29620, timeout_s="8")
    tail = "\n".join((res.stdout + res.stderr).splitlines()[-40:])
    assert "collective failed as expected" in res.stdout, tail
    assert "unexpectedly succeeded" not in res.stdout, tail
