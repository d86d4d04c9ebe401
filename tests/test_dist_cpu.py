"""Multi-process host-side logic on CPU (gloo, world 2): tensor parallelism, expert parallelism
with replicated and with data-parallel attention, and the collective wrappers. Real processes and
a real process group, as the reference's collective tests use (torchrun + init_process_group,
xlite/tests/kernels/all_reduce.py:8-63) — no mocks."""
import os
import socket
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def run_workers(mode, world=2, timeout=600, extra_env=None):
    env = dict(os.environ)
    env["OMP_NUM_THREADS"] = "2"
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "dist_worker.py"), "--mode", mode]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)
    assert r.returncode == 0 and "WORKER_OK" in r.stdout, f"{mode} failed:\n{r.stdout[-3000:]}\n{r.stderr[-3000:]}"
    return r.stdout


@pytest.mark.parametrize("mode", ["collectives_cpu", "tp_cpu", "sp_cpu", "moe_ep_cpu", "moe_ep_slice_cpu", "vocab_greedy_cpu", "dp_ep_cpu", "kv_transfer_cpu",
                                  "dual_stream_cpu", "spec_tp_cpu", "serve_tp_cpu", "serve_dp_cpu", "serve_fail_cpu"])
def test_two_ranks(mode):
    run_workers(mode, 2)
