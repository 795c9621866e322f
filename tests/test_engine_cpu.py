"""launch_engine / AsyncEngine / Worker over torch RPC with CPU (gloo) workers, mirroring the
reference's engine tests (tests/test_engine/test_single_device.py, test_tp.py): BoringModel maps
x to 4x + 1 for any tensor-parallel size; results come back by request id.  Each life cycle runs
in its own process (tests/engine_check.py)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("tp_world_size", [1, 2])
def test_engine_life_cycle(tp_world_size):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "engine_check.py"), str(tp_world_size)], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=180)
    assert r.returncode == 0 and f"engine ok {tp_world_size}" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_engine_with_the_generation_batch_manager():
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "engine_check.py"), "1", "generation"], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=180)
    assert r.returncode == 0 and "engine generation ok 1" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_engine_reports_rejected_requests_and_dead_workers():
    """Failures are made on the host: a model call that raises, and a worker process that exits."""
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "engine_check.py"), "1", "failure"], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=180)
    assert r.returncode == 0 and "engine failure ok" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


@pytest.mark.parametrize("mode,marker", [("unhealthy", "engine unhealthy ok"), ("startup", "engine startup ok")])
def test_engine_faulted_worker_and_failed_start(mode, marker):
    """unhealthy: a worker whose health check reports a fault (what a timed-out device-side wait
    becomes) stops returning results.  startup: a model_fn that raises ends launch_engine with
    WorkerFailedError.  Both failures are made on the host."""
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="", PYTHONPATH=ROOT)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "engine_check.py"), "1", mode], cwd=ROOT, env=env,
                       capture_output=True, text=True, timeout=180)
    assert r.returncode == 0 and marker in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]


def test_launch_engine_size_aliases_are_checked_before_anything_starts():
    from energonai_b200.engine import launch_engine
    with pytest.raises(ValueError, match="disagree"):
        launch_engine(2, 1, "127.0.0.1", 1, 1, lambda: None, tp_init_size=4)
    with pytest.raises(TypeError, match="model_fn"):
        launch_engine(tp_init_size=1)


def test_pipeline_parallelism_is_rejected():
    from energonai_b200.engine import AsyncEngine
    with pytest.raises(RuntimeError, match="pp_world_size"):
        AsyncEngine(1, 2, "127.0.0.1", 1, 1)
