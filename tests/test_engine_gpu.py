"""launch_engine with a GPU worker: generation requests through the RPC pipes return the tokens
the model produces when called directly (tests/engine_check_gpu.py; its own
process because torch RPC cannot be re-initialised inside one)."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_engine_generation_on_gpu():
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "engine_check_gpu.py")], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "engine gpu ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_engine_generation_on_two_gpus():
    """launch_engine(tp_world_size=2): two workers, each with its shard and the library's own
    exchange context (enabled by the worker), the same batch sent to both, rank 0's answer
    returned (energonai/engine.py:79-80, 94-97; the reference's tests/test_engine/test_tp.py)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, PYTHONPATH=ROOT, MASTER_ADDR="127.0.0.1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "engine_check_gpu.py"), "2"], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "engine gpu ok 2" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
