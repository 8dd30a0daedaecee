"""Host-side tests of ``measure.GpuPoolMeasurer``: a candidate that hangs, one that raises and a
worker that dies each score ``inf``; the worker is replaced and the next job is served
(flextensor/scheduler.py:710-712,742-752: failure -> inf, broken pool rebuilt).  The workers run
stub evaluators (``tests/pool_stubs.py``): no GPU is used, none is faulted or hung."""
import math
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import pool_stubs as P  # noqa: E402

from flextensor_b200.measure import GpuPoolMeasurer, Job, make_job, task_spec  # noqa: E402
from flextensor_b200.task import TASK_TABLE, Task, gemm, register_task  # noqa: E402
from flextensor_b200.utils import Config  # noqa: E402

KEY = "gemm_gemm_(256, 128, 128)_cuda(0)"


@pytest.fixture()
def pool():
    m = GpuPoolMeasurer(devices=[0], startup_timeout=60.0, evaluate="pool_stubs:evaluate")
    yield m
    m.close()


def test_hung_candidate_scores_inf_and_the_worker_is_replaced(pool):
    cfg = Config([{}], None)
    assert pool([(KEY, cfg, 0)], timeout=5.0)[0] < math.inf          # starts the worker
    first = pool.workers[0].proc.pid
    out = pool([(KEY, cfg, P.SLEEP_FOREVER), (KEY, cfg, 0)], timeout=0.5)
    assert out[0] == math.inf and out[1] < math.inf                  # the next job is served
    assert pool.replaced == 1
    assert pool.workers[0].proc.pid != first and pool.workers[0].proc.is_alive()


def test_dead_worker_scores_inf_and_is_replaced(pool):
    cfg = Config([{}], None)
    out = pool([(KEY, cfg, P.EXIT_NONZERO), (KEY, cfg, 0), (KEY, cfg, P.RAISE), (KEY, cfg, 0)], timeout=5.0)
    assert out[0] == math.inf and out[2] == math.inf
    assert out[1] < math.inf and out[3] < math.inf
    assert pool.replaced == 1                                        # raising does not cost the worker


def test_runtime_registered_task_resolves_in_a_spawned_worker(pool):
    """A task registered after import is unknown to a spawned worker's table; the job carries what
    rebuilds it (the reference's forked children inherit the table instead)."""
    task = Task("gemm", "fresh", gemm, (96, 160, 224), "cuda", 0)
    register_task(task)
    assert task.key not in ("", KEY) and task_spec(task) == ("gemm", "fresh", "flextensor_b200.task", "gemm",
                                                             (96, 160, 224), "cuda", 0)
    job = make_job(task.key, Config([{}], None), P.RESOLVE, precision="tf32")
    assert isinstance(job, Job) and tuple(job) == (task.key, Config([{}], None), P.RESOLVE)
    assert pool([job], timeout=30.0) == [3.5]                        # 3 buffers, precision travelled
    other = Task("gemm", "fresh", gemm, (96, 160, 32), "cuda", 0)
    register_task(other)
    bare = (other.key, Config([{}], None), P.RESOLVE)                # without the spec: KeyError -> inf
    assert pool([bare], timeout=30.0) == [math.inf]
    del TASK_TABLE[task.key], TASK_TABLE[other.key]


def test_a_lambda_builder_cannot_travel():
    task = Task("gemm", "anon", lambda n, k, m: gemm(n, k, m), (32, 32, 32), "cuda", 0)
    assert task_spec(task) is None
