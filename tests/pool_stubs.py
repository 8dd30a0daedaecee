"""Evaluators for host-side tests of the measurement pool: they stand where a worker would plan,
build and time a candidate on its GPU, and touch no GPU at all.  A job's ``op_pos`` field selects
the behaviour, so one pool can be driven through every failure the pool has to survive."""
import os
import time

SLEEP_FOREVER, RAISE, EXIT_NONZERO, RESOLVE = 101, 102, 103, 104


def evaluate(job, number, dev_id):
    task_key, config, op_pos = job
    if op_pos == SLEEP_FOREVER:      # a candidate that hangs: sleeps on the host past any timeout
        time.sleep(3600)
    if op_pos == RAISE:              # a candidate whose build fails
        raise ValueError("this candidate does not build")
    if op_pos == EXIT_NONZERO:       # a worker that dies under a candidate
        os._exit(7)
    if op_pos == RESOLVE:            # resolve the job's task in this (spawned) process, no CUDA needed
        from flextensor_b200.measure import resolve_task
        task = resolve_task(job)
        ops, bufs = task.func(*task.args)
        return float(len(bufs)) + (0.5 if getattr(job, "precision", None) == "tf32" else 0.0)
    return 1.0 + 0.001 * os.getpid() / 1e6 + float(dev_id)
