"""The loop every per-operator driver runs (flextensor/optimize/optimize_gemm.py:18-128 and
its siblings share it): for each shape build the task key, search, print the configs, append
``key:json(configs)`` to the log, replay and time; ``--test file`` replays a log instead."""
import json
import sys
import time

from ..scheduler import schedule, schedule_with_config
from ..task import Task, register_task
from ..utils import Config
from .common import evaluate, test


def optimize(category, name, func, shapes, args_of, slevel=4, rlevel=3, target="cuda", dev_id=0, timeout=4.0,
             trials=100, parallel=1, method="searching", use_model=False, logfile=sys.stdout, trials_of=None,
             force_inline=False, precision=None, measurer=None):
    ret = {}
    for shape in shapes:
        print("Optimize %s shape %s [%.6f]" % (name, str(shape), time.time()), flush=True)
        task = Task(category, name, func, args_of(shape), target, dev_id)
        register_task(task, override=True)   # as the reference's drivers do before they schedule
        kwargs = {}
        if trials_of is not None:
            kwargs["trials"] = trials_of(trials)
        if force_inline:
            kwargs["force_inline"] = True
        if measurer is not None:
            kwargs["measurer"] = measurer
        if precision is not None:
            kwargs["precision"] = precision
        if use_model:
            kwargs["use_model"] = True
        beg = time.time()
        s, bufs, configs = schedule(task.key, slevel=slevel, rlevel=rlevel, op_trial=trials, timeout=timeout,
                                    op_stop=trials // 2, method=method, parallel=parallel, number=10, **kwargs)
        end = time.time()
        print("###################################### [%.6f]" % time.time())
        print("op schedules:")
        for config in configs.op_config_lst:
            print("----------------------------------")
            for key, value in config.items():
                if value:
                    print(key, value)
        print("graph schedules:")
        for key, value in (configs.graph_config or {}).items():
            if value:
                print(key, value)
        ret[task.key] = configs
        print(task.key + ":" + json.dumps(configs), file=logfile, flush=True)
        s, bufs = schedule_with_config(task.key, configs, precision=precision)
        print("Use", evaluate(task.key, s, bufs, target, dev_id), "ms")
        print("Cost", end - beg, "s")
        print()
    return ret


def _register_from_key(key, category, name, func):
    """A log line of this driver names a task that only ``optimize`` registered: rebuild it from
    the key, ``<category>_<name>_<args tuple>_<target>(<device>)``."""
    import ast
    prefix = "%s_%s_" % (category, name)
    if not key.startswith(prefix):
        return
    body = key[len(prefix):]
    args_text, _, tail = body.rpartition("_")
    target, _, dev_text = tail.partition("(")
    args = ast.literal_eval(args_text)
    register_task(Task(category, name, func, tuple(args), target, int(dev_text.rstrip(")") or 0)), override=True)


def replay(path, dev_id, check, category=None, name=None, func=None):
    from ..task import TASK_TABLE
    with open(path, "r") as fin:
        for line in fin:
            if not line.strip():
                continue
            key, string = line.split(":", 1)
            if key not in TASK_TABLE and func is not None:
                _register_from_key(key, category, name, func)
            obj = json.loads(string)
            test(key, Config(obj[0], obj[1]), dev_id, check_result=check)


def main(category, name, func, shapes, args_of, trials_of=None):
    import argparse
    import numpy as np
    import torch
    from .common import init_arg_parser
    parser = argparse.ArgumentParser()
    init_arg_parser(parser)
    args = parser.parse_args()
    if args.seed is not None:
        np.random.seed(args.seed)
        torch.manual_seed(args.seed)
    end = len(shapes) if args.to < 0 else args.to
    if args.test != "":
        replay(args.test, args.device, args.check, category, name, func)
        return
    kwargs = dict(slevel=args.slevel, rlevel=args.rlevel, target=args.target, dev_id=args.device,
                  timeout=args.timeout, trials=args.trials, parallel=args.parallel, method=args.method,
                  use_model=args.use_model, trials_of=trials_of, force_inline=args.force_inline,
                  precision=args.precision)
    if args.log != "":
        with open(args.log, "a") as flog:
            optimize(category, name, func, shapes[args.from_:end], args_of, logfile=flog, **kwargs)
    else:
        optimize(category, name, func, shapes[args.from_:end], args_of, logfile=sys.stdout, **kwargs)
