"""Data-parallel training over NCCL against a single-device CPU run of the whole batch. Needs at
least two GPUs; on a one-GPU box it is skipped."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def gpu_count():
    try:
        out = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30).stdout
        return sum(1 for line in out.splitlines() if line.startswith("GPU "))
    except (OSError, subprocess.TimeoutExpired):
        return 0


@pytest.mark.parametrize("world,exchange", [(2, "peer"), (2, "nccl")])
def test_shards_train_like_one_device_on_the_whole_batch(world, exchange):
    """Gradients summed by the backend's own kernel over peer memory (the default between the
    GPUs of one machine), and by the NCCL all-reduce (MSX_PEER_REDUCE=0)."""
    if gpu_count() < world:
        pytest.skip("needs %d GPUs" % world)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MSX_PEER_REDUCE="1" if exchange == "peer" else "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(world),
           "--master-addr", "127.0.0.1", "--master-port", "29731", os.path.join(HERE, "dp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "DP_PARITY_OK" in r.stdout, r.stdout[-3000:] + r.stderr[-3000:]
    assert "exchange=%s" % exchange in r.stdout, r.stdout[-3000:]
