"""Measurement of candidate configurations.

The reference measures a candidate by compiling it with TVM, loading the library and
timing it inside a killable child process (flextensor/measure.py:63-115,
flextensor/scheduler.py:682-761): ``master_routine(timeout, func, *args)`` forks a
servant, waits ``timeout`` seconds on a queue, terminates it, and any failure becomes
``inf``.  Here the kernels are pre-compiled, so a candidate costs one launch series and
no compile; what remains is the isolation: candidates run in worker processes pinned
one per GPU (``GpuPoolMeasurer``), a worker that exceeds the timeout is killed and
replaced, and its candidate scores ``inf``.  ``build_and_eval`` and ``master_routine``
keep their reference signatures.
"""
import importlib
import multiprocessing as _mp
import os
import queue as _queue
import sys
import time

mp = _mp.get_context("spawn")

_DEFAULT = {"measurer": None}


def servant_routine(func, que, *args, **kwargs):
    try:
        ret = func(*args, **kwargs)
    except Exception as exc:  # reported to the master as a value
        ret = exc
    que.put(ret)


def master_routine(timeout, func, *args, **kwargs):
    """Run ``func`` in a child process; its result, or an Exception on failure/timeout."""
    que = mp.Queue()
    servant = mp.Process(target=servant_routine, args=(func, que, *args), kwargs=kwargs)
    servant.start()
    try:
        ret = que.get(block=True, timeout=timeout)
    except Exception as exc:
        ret = exc if str(exc) else RuntimeError("timeout after %s s" % timeout)
    servant.terminate()
    servant.join()
    return ret


_INPUT_CACHE = {}


def make_inputs(bufs, device, low=0.0, high=1.0, seed=None, cache=True):
    """Random arrays for the buffers of a task (uniform(low, high) floats as measure.py:98; integers in
    [-127, 127] for int8), output buffer included, as CUDA tensors drawn on the device.

    Candidates of one task differ only in their knobs, so the arrays of the last task are kept and
    handed out again (``cache``): a worker does not redraw gigabytes per candidate.
    """
    import torch
    from .runtime import torch_dtype
    key = (str(device), float(low), float(high), seed,
           tuple((tuple(int(s) for s in buf.shape), buf.dtype) for buf in bufs))
    if cache and key in _INPUT_CACHE:
        return _INPUT_CACHE[key]
    gen = torch.Generator(device=device)
    gen.manual_seed(0 if seed is None else int(seed))
    arrays = []
    for buf in bufs:
        shape = tuple(int(s) for s in buf.shape)
        if buf.dtype == "int8":
            arrays.append(torch.randint(-127, 128, shape, device=device, dtype=torch.int8, generator=gen))
        elif buf.dtype == "int32":
            arrays.append(torch.zeros(shape, dtype=torch.int32, device=device))
        else:
            t = torch.rand(shape, device=device, generator=gen, dtype=torch.float32) * (high - low) + low
            arrays.append(t.to(torch_dtype(buf.dtype)))
    if cache:
        _INPUT_CACHE.clear()  # keep one task's arrays only
        _INPUT_CACHE[key] = arrays
    return arrays


def build_and_eval(lib, s, bufs, target, dev_id, rpc_info=None, number=1):
    """Build the plan, run it on random inputs on GPU ``dev_id``; mean milliseconds per call.

    ``lib`` (a path in the reference, where the compiled module was exported) is unused.
    """
    import torch
    from .runtime import build
    if target != "cuda":
        raise RuntimeError("only target 'cuda' is measured on this backend")
    device = torch.device("cuda", dev_id)
    with torch.cuda.device(device):
        func = build(s, bufs, target)
        arrays = make_inputs(bufs, device)
        evaluator = func.time_evaluator(func.entry_name, None, number=max(int(number), 1))
        return evaluator(*arrays).mean * 1e3


def _evaluate(s, bufs, target, dev_id, number=1, q=None):
    """In-process timing of a plan with uniform(-10, 10) inputs (flextensor/measure.py:29-52);
    milliseconds, also put on ``q`` when a queue is given."""
    import torch
    from .runtime import build
    device = torch.device("cuda", dev_id)
    with torch.cuda.device(device):
        func = build(s, bufs, target)
        arrays = make_inputs(bufs, device, low=-10.0, high=10.0)
        func(*arrays)
        func.check()
        cost = func.time_evaluator(func.entry_name, None, number=max(int(number), 1))(*arrays).mean * 1e3
    if q is not None:
        q.put(cost)
    return cost


class Job(tuple):
    """One candidate, ``(task_key, Config, op_pos)`` when unpacked, plus what a worker in
    another process needs beside it: the fp32 ``precision`` the plan is to be built with and,
    for a task that was registered at run time, ``task_spec`` - what rebuilds the task there.

    The reference forks its measurement children, which therefore inherit ``TASK_TABLE``
    (flextensor/scheduler.py:715-752); workers here are spawned (a forked child cannot use CUDA),
    so a task the parent registered after import has to travel with the job.
    """

    def __new__(cls, task_key, config, op_pos, precision=None, task_spec=None):
        self = super().__new__(cls, (task_key, config, op_pos))
        self.precision = precision
        self.task_spec = task_spec
        return self

    def __reduce__(self):
        return (Job, (self[0], self[1], self[2], self.precision, self.task_spec))


def task_spec(task):
    """``(category, name, module, function, args, target, dev_id)`` of a task whose builder is a
    module-level function, or None when the builder cannot be named (a lambda, a closure): such
    a task can only be measured in the registering process."""
    func = task.func
    module, name = getattr(func, "__module__", None), getattr(func, "__qualname__", "")
    if not module or not name or "<" in name or "." in name:
        return None
    category = task.category
    prefix, suffix = category + "_", "_%s_%s(%d)" % (task.args, task.target, task.dev_id)
    if not (task.key.startswith(prefix) and task.key.endswith(suffix)):
        return None
    task_name = task.key[len(prefix):len(task.key) - len(suffix)]
    return (category, task_name, module, name, tuple(task.args), task.target, task.dev_id)


def make_job(task_key, config, op_pos, precision=None):
    """A ``Job`` for a registered task, carrying the task's spec so that any worker can resolve it."""
    from .task import TASK_TABLE
    task = TASK_TABLE.get(task_key)
    return Job(task_key, config, op_pos, precision, task_spec(task) if task is not None else None)


def resolve_task(job):
    """The task of a job in this process: from ``TASK_TABLE``, or rebuilt from the job's spec and
    registered (a worker's table only holds the import-time registrations)."""
    from .task import TASK_TABLE, Task, register_task
    task_key = job[0]
    task = TASK_TABLE.get(task_key)
    if task is not None:
        return task
    spec = getattr(job, "task_spec", None)
    if spec is None:
        raise KeyError("task %r is not registered in this process and the job carries no way to rebuild it "
                       "(its builder must be a module-level function)" % (task_key,))
    category, name, module, func_name, args, target, dev_id = spec
    func = getattr(importlib.import_module(module), func_name)
    task = Task(category, name, func, tuple(args), target, dev_id)
    if task.key != task_key:
        raise KeyError("job spec rebuilds %r, not %r" % (task.key, task_key))
    register_task(task)
    return task


def _evaluate_job(job, number, dev_id):
    """One candidate: (task_key, Config, op_pos) -> milliseconds on GPU ``dev_id``."""
    from .scheduler import schedule_with_config
    task_key, config, op_pos = job
    task = resolve_task(job)
    s, bufs = schedule_with_config(task_key, config, op_pos=op_pos, precision=getattr(job, "precision", None))
    return build_and_eval(None, s, bufs, task.target, dev_id, None, number)


def _load_evaluate(evaluate):
    """``"module:function"`` -> the function (the evaluator a worker runs per job)."""
    if evaluate is None:
        return _evaluate_job
    module, _, name = evaluate.partition(":")
    return getattr(importlib.import_module(module), name)


def _worker_main(dev_id, jobs, results, evaluate=None, sys_path=None):
    """Worker process: pinned to one GPU, serves jobs until it receives ``None``."""
    os.environ.setdefault("CUDA_DEVICE_ORDER", "PCI_BUS_ID")
    for entry in reversed(sys_path or []):
        if entry not in sys.path:
            sys.path.insert(0, entry)
    from . import task as _task  # noqa: F401  (fills TASK_TABLE in this process)
    run = _load_evaluate(evaluate)
    while True:
        item = jobs.get()
        if item is None:
            return
        job_id, job, number = item
        try:
            value = run(job, number, dev_id)
        except Exception as exc:  # sent as text: any exception type survives the queue
            value = RuntimeError("%s: %s" % (type(exc).__name__, exc))
        results.put((job_id, value))


class _Worker(object):
    def __init__(self, dev_id, evaluate=None):
        self.dev_id = dev_id
        self.jobs = mp.Queue()
        self.results = mp.Queue()
        self.proc = mp.Process(target=_worker_main, args=(dev_id, self.jobs, self.results, evaluate, list(sys.path)),
                               daemon=True)
        self.proc.start()

    def stop(self, kill=False):
        if self.proc.is_alive():
            if kill:
                self.proc.terminate()
            else:
                self.jobs.put(None)
            self.proc.join(timeout=5)
            if self.proc.is_alive():
                self.proc.kill()
                self.proc.join()


class GpuPoolMeasurer(object):
    """Measures batches of candidates, one candidate at a time per GPU.

    ``devices``: GPU ordinals to use (default: all visible).  A measurer is a callable
    ``(jobs, number, timeout, parallel) -> [ms or inf]`` where each job is
    ``(task_key, Config, op_pos)``; ``parallel`` caps how many GPUs are used for the call
    (``parallel == 1`` is the serial re-measurement of the search's leaders).
    """

    def __init__(self, devices=None, startup_timeout=120.0, evaluate=None):
        """``evaluate``: ``"module:function"`` naming what a worker runs per job, called as
        ``function(job, number, dev_id) -> milliseconds`` (default: plan, build and time the
        candidate on the worker's GPU).  Host-side tests of the pool's failure handling pass
        evaluators that sleep, raise or exit without touching a GPU."""
        self.evaluate = evaluate
        self.replaced = 0  # workers killed after a timeout or found dead, and replaced
        if devices is None:
            import torch
            devices = list(range(torch.cuda.device_count()))
        if not devices:
            raise RuntimeError("GpuPoolMeasurer needs at least one CUDA device")
        self.devices = list(devices)
        self.startup_timeout = startup_timeout
        self.workers = {}
        self.fresh = set()
        self.trace = []  # (task_key, op_pos, ms, device) of every measurement

    def _worker(self, dev_id):
        w = self.workers.get(dev_id)
        if w is None or not w.proc.is_alive():
            w = _Worker(dev_id, self.evaluate)
            self.workers[dev_id] = w
            self.fresh.add(dev_id)
        return w

    def __call__(self, jobs, number=1, timeout=5.0, parallel=None):
        results = [float("inf")] * len(jobs)
        if not jobs:
            return results
        lanes = self.devices[:max(1, min(len(self.devices), parallel or len(self.devices)))]
        pending = list(enumerate(jobs))
        running = {}  # dev_id -> (job_id, deadline)
        while pending or running:
            for dev in lanes:
                if dev not in running and pending:
                    job_id, job = pending.pop(0)
                    w = self._worker(dev)
                    w.jobs.put((job_id, job, number))
                    grace = self.startup_timeout if dev in self.fresh else 0.0
                    running[dev] = (job_id, time.time() + timeout + grace)
            progressed = False
            for dev in list(running):
                job_id, deadline = running[dev]
                w = self.workers[dev]
                try:
                    got_id, value = w.results.get(timeout=0.01)
                except _queue.Empty:
                    if time.time() > deadline or not w.proc.is_alive():
                        # the candidate hung or the worker died: inf, and a fresh worker next time
                        w.stop(kill=True)
                        del self.workers[dev]
                        del running[dev]
                        self.replaced += 1
                        progressed = True
                    continue
                self.fresh.discard(dev)
                del running[dev]
                progressed = True
                if got_id == job_id and not isinstance(value, Exception):
                    results[job_id] = float(value)
                self.trace.append((jobs[job_id][0], jobs[job_id][2], results[job_id], dev))
            if not progressed:
                time.sleep(0.002)
        return results

    def close(self):
        for w in self.workers.values():
            w.stop()
        self.workers.clear()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class InProcessMeasurer(object):
    """Measures candidates in the calling process on one GPU (no isolation, no timeout):
    for scripts that already own the device, e.g. the benchmark."""

    def __init__(self, dev_id=0):
        self.dev_id = dev_id

    def __call__(self, jobs, number=1, timeout=5.0, parallel=None):
        out = []
        for job in jobs:
            try:
                out.append(float(_evaluate_job(job, number, self.dev_id)))
            except Exception:
                out.append(float("inf"))
        return out


def default_measurer():
    """The process-wide measurer used when ``schedule`` is given none: a GPU pool over all
    visible devices.  Raises when no CUDA device is present (there is no CPU stand-in)."""
    if _DEFAULT["measurer"] is None:
        _DEFAULT["measurer"] = GpuPoolMeasurer()
    return _DEFAULT["measurer"]


def set_default_measurer(measurer):
    _DEFAULT["measurer"] = measurer
