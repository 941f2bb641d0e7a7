"""dim_in sharding across real ranks: one process per GPU, the library's communicator (NCCL bound at run time) and
its one-shot all-reduce over NVLink.  Needs at least two GPUs in one machine; skipped otherwise.  The ranks run
tests/multi_gpu_worker.py; NVLS is switched off for these runs (plain peer loads and stores only)."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _gpus():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _run(case, world, port):
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "multi_gpu_worker.py"), str(r), str(world), str(port), case],
                              env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n[timed out]"
        outs.append((p.returncode, out))
    for r, (rc, out) in enumerate(outs):
        assert rc == 0 and "RANK %d OK" % r in out, "rank %d:\n%s" % (r, out[-3000:])


@pytest.mark.skipif(_gpus() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("case,port", [("allreduce", 29711), ("relu", 29712), ("cnn", 29713), ("timeout", 29714)])
def test_two_ranks(case, port):
    _run(case, 2, port)


@pytest.mark.skipif(_gpus() < 4, reason="needs four GPUs")
@pytest.mark.parametrize("case,port", [("allreduce", 29721), ("cnn", 29723)])
def test_all_ranks_of_the_box(case, port):
    _run(case, min(_gpus(), 8), port)
