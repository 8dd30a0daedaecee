"""Search over kernel configurations and the entry points that return a runnable plan.

Public surface as in the reference's ``flextensor/scheduler.py``:
  schedule(task_key, slevel, rlevel, op_trial, graph_trial, op_stop, graph_stop, number,
           timeout, parallel, method, **kwargs) -> (s, bufs, configs)      (scheduler.py:969-1111)
  schedule_with_config(task_key, configs, op_pos=None, rewrite=False) -> (s, bufs)   (:1114-1130)
  schedule_with_config_ops(ops, bufs, configs, op_pos=None, target=...) -> (s, bufs) (:1133-1186)
  flatten_graph, OpState, Scheduler, OpScheduler, GraphScheduler.
``s`` is a ``runtime.KernelPlan`` (what ``runtime.build`` turns into the callable) instead
of a TVM schedule.  The search logic is the reference's: warm-up with random points,
then either neighbourhood expansion around remembered good points ("searching",
scheduler.py:293-442), epsilon-greedy Q-learning walks ("q", :444-540) or pure random
sampling ("random", :282-291), with the same rewards, heap memory, early-stop rules and
periodic re-measurement.  What is measured is different: candidates are knob sets of
pre-compiled kernels, handed to a pluggable *measurer* (``measure.GpuPoolMeasurer`` runs
one candidate per GPU; tests plug in a pure-Python cost function).
"""
import math
import time
from collections import deque

import numpy as np

from .measure import make_job
from .model import WalkerGroup
from .space import generate_space_inter_op, generate_space_intra_op
from .task import TASK_TABLE
from .utils import Config, assert_print

VERBOSE = True


def _log(*args, **kwargs):
    if VERBOSE:
        print(*args, **kwargs)


def flatten_graph(ops):
    """Compute ops in producer-first order plus the tensor -> consumers map."""
    order, down_graph, seen = [], {}, set()
    queue = deque()
    for op in ops:
        queue.append(op)
        seen.add(id(op))
    while queue:
        cur = queue.popleft()
        if hasattr(cur, "kind"):
            order.append(cur)
        for t in cur.input_tensors:
            if id(t.op) not in seen:
                seen.add(id(t.op))
                queue.append(t.op)
            down_graph.setdefault(t, []).append(cur)
    order.reverse()
    return order, down_graph


class OpState(object):
    def __init__(self):
        self.inline = False
        self.loop_lst = []
        self.loop_idx = []
        self.compute_at = False
        self.consumer_lst = []


def _op_states(op_lst, down_graph):
    states = [OpState() for _ in op_lst]
    for state, op in zip(states, op_lst):
        consumers = []
        for i in range(op.num_outputs):
            consumers.extend(down_graph.get(op.output(i), []))
        state.consumer_lst = list({id(c): c for c in consumers}.values())
    return states


def _fmt(values):
    return "[ " + "".join("%.6f " % v for v in values) + "]"


class Scheduler(object):
    """Search engine over one ``Space``; subclasses say how a candidate becomes a full Config."""

    def __init__(self, name, task_key, space, parallel=2, timeout=4.0, trial=100, number=1, early_stop=30,
                 rpc_info=None, rewrite=False, measurer=None):
        self.task_key = task_key
        self.space = space
        self.parallel = max(parallel, 1)
        self.timeout = timeout
        self.trial = trial
        self.number = number
        self.early_stop = early_stop
        self.task = TASK_TABLE[self.task_key]
        self.walker_group = WalkerGroup(self.task.category + "_" + name, self.space)
        self.rpc_info = rpc_info
        self.rewrite = rewrite
        self.measurer = measurer
        self.re_evalutate_number = 10
        self.warm_up_epoch = 20
        self.warm_up_number = 20
        self.early_stop_eps = 0.02  # milliseconds, as in the reference (capped at 1 % of the best, see below)
        self.precision = None  # fp32 mode ("tf32" | "3xtf32") the candidates are built with; None = default
        self.seeds = []  # configs to measure and remember before the warm-up (e.g. from a saved log)

    def _stop_eps(self, best_value):
        """'Best did not move' threshold of the early stop: the reference's 0.02 ms, but never more than
        1 % of the best time - its kernels ran for milliseconds, these often run for microseconds."""
        if best_value < float("inf") and best_value > 0:
            return min(self.early_stop_eps, 0.01 * best_value)
        return self.early_stop_eps

    # ------------------------------------------------------------ evaluation plumbing
    def parallel_evaluate(self, old_configs, new_configs, number=1):
        raise NotImplementedError()

    def _parallel_evaluate(self, old_configs, new_configs, mode="op", number=1):
        """Measure candidates; a failure of any kind is ``inf`` (scheduler.py:710-712,742-748)."""
        if not new_configs:
            return []
        jobs = []
        for config in new_configs:
            if mode == "op":
                full = Config(list(old_configs.op_config_lst) + [config], old_configs.graph_config)
                op_pos = self.op_pos
            elif mode == "graph":
                full = Config(list(old_configs.op_config_lst), config)
                op_pos = None
            else:
                raise RuntimeError("Unknown mode %s" % mode)
            jobs.append(make_job(self.task_key, full, op_pos, precision=self.precision))
        measurer = self.measurer
        if measurer is None:
            from .measure import default_measurer
            measurer = default_measurer()
        results = measurer(jobs, number=number, timeout=self.timeout, parallel=self.parallel)
        return [float(r) if (r is not None and not isinstance(r, Exception)) else float("inf") for r in results]

    def _evaluate(self, configs, indices_lst, use_model):
        """Costs of a list of points: measured, or predicted when ``use_model``."""
        if use_model:
            return self.walker_group.query_performance(indices_lst)
        candidates = [self.walker_group.to_config(ind) for ind in indices_lst]
        results = self.parallel_evaluate(configs, candidates, number=self.number)
        self.walker_group.add_perf_data(indices_lst, results)
        return results

    # ------------------------------------------------------------ seeding
    def _indices_of(self, config):
        """The point of this scheduler's space that a config names, or None when an entity of the
        config is not in its sub-space."""
        indices = {}
        for type_key, names in self.space.types.items():
            entities = config.get(type_key) or []
            if len(entities) != len(names):
                return None
            for name, entity in zip(names, entities):
                sub = self.space.subspaces[name]
                try:
                    indices[name] = [list(e) for e in sub.static_entities].index(list(entity))
                except ValueError:
                    return None
        return indices

    def _measure_seeds(self, configs, use_model):
        """Seed configs (from a saved log, or from the reference's logs through ``logcompat``) are
        measured first and go into the heap memory like warm-up points, so that the walk can start
        from them."""
        points = [ind for ind in (self._indices_of(c) for c in self.seeds) if ind is not None]
        if not points:
            return
        results = self._evaluate(configs, points, use_model)
        _log("seeds [%.6f] %s" % (time.time(), _fmt(results)))
        for indices, value in zip(points, results):
            if value < float("inf"):
                self.walker_group.record(indices, value)

    # ------------------------------------------------------------ warm-up
    def _warm_up(self, warm_up_epoches, warm_up_trials, configs, type_keys, max_repeat=20, use_model=False):
        """Random points into the heap memory; retries with a doubled timeout (<= 40 s) when
        nothing valid was found, at most ``max_repeat`` times (scheduler.py:222-280)."""
        repeats = 0
        old_timeout = self.timeout
        while True:
            for _ in range(warm_up_epoches):
                drawn = self.walker_group.forward(warm_up_trials, policy="random")
                indices_lst = [{name: int(drawn[name][1][i]) for name in drawn} for i in range(warm_up_trials)]
                results = self._evaluate(configs, indices_lst, use_model)
                _log("warm up [%.6f] %s" % (time.time(), _fmt(results)))
                for indices, value in zip(indices_lst, results):
                    if value < float("inf"):
                        self.walker_group.record(indices, value)
            if self.walker_group.top1():
                break
            _log("Warning: No valid schedule found in warm up process, please use more trials")
            _log("Now automatically use more trials, increase %d" % warm_up_trials)
            warm_up_epoches = 1
            repeats += 1
            self.timeout = min(2 * self.timeout, 40)
            if repeats >= max_repeat:
                _log("Fail to find valid schedule, too many errors")
                break
        self.timeout = old_timeout

    # ------------------------------------------------------------ the three methods
    def _random_schedule(self, configs, type_keys, use_model=False):
        if use_model:
            self.walker_group.load_or_create_model()
        for _ in range(self.trial):
            self._warm_up(1, self.parallel, configs, type_keys, use_model=use_model)
        return self.walker_group.to_config(self.walker_group.top1())

    def _searching_schedule(self, configs, type_keys, use_model=False):
        group = self.walker_group
        if use_model:
            group.load_or_create_model()
        self._warm_up(self.warm_up_epoch, self.warm_up_number, configs, type_keys, use_model=use_model)

        minimal = [{}, float("inf")]  # best retired local minimum
        retired = []                  # other retired local minima
        part = math.ceil(self.trial / 20)
        last_best = group.top1_value()
        unchanged = 0
        empty_walks = 0
        for trial in range(self.trial):
            if not group.has_more():
                self._warm_up(1, self.parallel, configs, type_keys, use_model=use_model)
                continue
            centre, centre_value = group.top_random(with_value=True)
            next_lst, action_lst = group.full_walk(centre, no_repeat=True)
            empty_walks = empty_walks + 1 if not next_lst else 0
            results = self._evaluate(configs, next_lst, use_model)
            _log("tune [%.6f] %s" % (time.time(), _fmt(results)))
            local_minimum = True
            for indices, (name, direction), value in zip(next_lst, action_lst, results):
                reward = np.tanh(max(centre_value - value, 0.0))
                group.add_data(name, centre, direction, indices, reward)
                group.record(indices, value, random_reject=True)
                if value < group.top1_value():
                    local_minimum = False
            if local_minimum or empty_walks > 0:
                top = group.pop_top()
                if top.value < minimal[1]:
                    if minimal[1] < float("inf"):
                        retired.append(minimal)
                    minimal = [top.indices, top.value]
                else:
                    retired.append([top.indices, top.value])
            if group.top1_value() < minimal[1]:
                best_value, best = group.top1_value(), group.top1()
            else:
                best_value, best = minimal[1], minimal[0]
            _log("No. %d | [%.6f] The best currently %.6f" % (trial, time.time(), best_value), best)
            if empty_walks >= self.early_stop:
                _log("Early stop after continuous no trials %d times" % empty_walks)
                break
            if math.fabs(best_value - last_best) < self._stop_eps(best_value):
                unchanged += 1
            else:
                last_best = best_value
                unchanged = 0
            if unchanged >= self.early_stop:
                _log("Early stop with value %f repeats %d times" % (last_best, unchanged))
                break
            if (trial + 1) % part == 0:
                if not use_model:
                    # put the retired minima back and re-measure the leaders one at a time
                    if minimal[1] < float("inf"):
                        group.record(minimal[0], minimal[1], random_reject=False)
                    for indices, value in retired:
                        group.record(indices, value, random_reject=False)
                    minimal = [{}, float("inf")]
                    leaders = group.topk(self.re_evalutate_number, modify=True)
                    saved_parallel, self.parallel = self.parallel, 1
                    results = self._evaluate(configs, leaders, False)
                    self.parallel = saved_parallel
                    _log("re-evaluate [%.6f] %s" % (time.time(), _fmt(results)))
                    for indices, value in zip(leaders, results):
                        if value < float("inf"):
                            group.record(indices, value, random_reject=False)
                group.clear_data()
            self._warm_up(1, self.parallel, configs, type_keys, use_model=use_model)
        best = group.top1() if group.top1_value() < minimal[1] else minimal[0]
        return group.to_config(best)

    def _q_schedule(self, configs, type_keys, use_model=False):
        group = self.walker_group
        group.load_walker_model()
        if use_model:
            group.load_or_create_model()
        self._warm_up(10, 20, configs, type_keys, use_model=use_model)
        best, best_value = group.top1(), group.top1_value()
        retired = []
        last_best, unchanged = best_value, 0
        cur_lst = group.topk(self.parallel, modify=True, with_value=True)
        part = math.ceil(self.trial / 5)
        for trial in range(self.trial):
            from_lst, next_lst, action_lst = group.walk(cur_lst, trial)
            results = self._evaluate(configs, next_lst, use_model)
            for indices, (name, choice), (src, src_value), value in zip(next_lst, action_lst, from_lst, results):
                reward = np.tanh(max(src_value - value, 0.0))
                group.add_data(name, src, choice, indices, reward)
                group.record(indices, value, random_reject=True)
            if group.top1_value() < best_value:
                best_value, best = group.top1_value(), group.top1()
            _log("No. %d | [%.6f] The best currently %.6f" % (trial, time.time(), best_value), best)
            if math.fabs(best_value - last_best) < self._stop_eps(best_value):
                unchanged += 1
            else:
                last_best, unchanged = best_value, 0
            if unchanged >= self.early_stop:
                _log("Early stop with value %f repeats %d times" % (last_best, unchanged))
                break
            if not group.has_more():
                _log("No more points, end of scheduling")
                break
            retired.extend(cur_lst)
            cur_lst = group.topk(self.parallel, modify=True, with_value=True)
            if (trial + 1) % part == 0:
                group.train_walkers(verbose=VERBOSE)
                if not use_model:
                    if best_value < float("inf"):
                        group.record(best, best_value, random_reject=False)
                        best, best_value = {}, float("inf")
                    for indices, value in retired[-self.parallel:-1]:
                        group.record(indices, value, random_reject=False)
                    leaders = group.topk(self.parallel, modify=True)
                    results = self._evaluate(configs, leaders, False)
                    _log("re-evaluate [%.6f] %s" % (time.time(), _fmt(results)))
                    for indices, value in zip(leaders, results):
                        group.record(indices, value, random_reject=False)
                self._warm_up(1, self.parallel, configs, type_keys, use_model=use_model)
                if group.top1_value() < best_value:
                    best_value, best = group.top1_value(), group.top1()
        group.clear_data()
        if not best:
            best = group.top1()
        return group.to_config(best)

    def _dispatch(self, configs, type_keys, method, use_model):
        if not self.space.subspaces:
            return {}
        if len(self.space) == 1:
            # a single point: nothing to search (the reference would measure it 400 times in warm-up)
            only = {name: 0 for name in self.space.subspaces}
            return self.walker_group.to_config(only)
        if self.seeds:
            self._measure_seeds(configs, use_model)
        if method == "searching":
            return self._searching_schedule(configs, type_keys, use_model=use_model)
        if method == "q":
            return self._q_schedule(configs, type_keys, use_model=use_model)
        if method == "random":
            return self._random_schedule(configs, type_keys, use_model=use_model)
        raise RuntimeError("Currently no support for method %s" % method)


class OpScheduler(Scheduler):
    def __init__(self, task_key, op_pos, space, decay=0.7, parallel=1, timeout=4.0, trial=100, number=1,
                 early_stop=30, rpc_info=None, rewrite=False, measurer=None):
        super().__init__("op" + str(op_pos), task_key, space, parallel, timeout, trial, number, early_stop,
                         rpc_info, rewrite=rewrite, measurer=measurer)
        self.op_pos = op_pos

    def schedule(self, configs, method="searching", use_model=False, perf_path=None):
        if perf_path is not None:
            self.walker_group.model_path = perf_path
        return self._dispatch(configs, ["fuse", "reorder", "spatial", "reduce", "unroll"], method, use_model)

    def parallel_evaluate(self, configs, next_op_configs, number=1, rpc_info=None):
        return self._parallel_evaluate(configs, next_op_configs, mode="op", number=number)

    @staticmethod
    def generate_op_schedule(target, config):
        """Template of the target: a function ``op -> kernel knobs`` (cuda) ."""
        if target == "cuda":
            from .templates import config_to_knobs
            return lambda op: config_to_knobs(config, op)
        raise RuntimeError("Currently no support for target %s" % target)


class GraphScheduler(Scheduler):
    def __init__(self, task_key, space, decay=0.7, parallel=10, timeout=4.0, trial=100, number=1, early_stop=30,
                 rpc_info=None, rewrite=False, measurer=None):
        super().__init__("graph", task_key, space, parallel, timeout, trial, number, early_stop, rpc_info,
                         rewrite=rewrite, measurer=measurer)

    def schedule(self, configs, method="searching", use_model=False, perf_path=None):
        if perf_path is not None:
            self.walker_group.model_path = perf_path
        return self._dispatch(configs, ["inline", "merge"], method, use_model)

    def parallel_evaluate(self, configs, graph_configs, number=1):
        return self._parallel_evaluate(configs, graph_configs, mode="graph", number=number)


def schedule(task_key, slevel=4, rlevel=3, op_trial=50, graph_trial=10, op_stop=15, graph_stop=5, number=1,
             timeout=5, parallel=8, method="searching", **kwargs):
    """Search a schedule for a registered task; returns ``(plan, bufs, configs)``.

    Extra keyword arguments, as in the reference: ``trials`` (per-op trial budgets),
    ``op_perf_model_path`` ([(op_pos, path)]), ``graph_perf_model_path``, ``force_inline``,
    ``rpc_info`` (ignored: no remote boards).  New ones: ``measurer`` (callable measuring
    a batch of candidates), ``precision`` ("tf32" | "3xtf32") for fp32 contractions,
    ``use_model`` (search on the saved performance models instead of measuring), ``seeds`` ([(op_pos, op_config)]: configs measured before the warm-up, e.g. from
    ``logcompat.seeds_from_log``).
    """
    task = TASK_TABLE[task_key]
    ops, bufs = task.func(*task.args)
    op_lst, down_graph = flatten_graph(ops)
    measurer = kwargs.get("measurer")
    force_trials = kwargs.get("trials", [op_trial for _ in op_lst])
    assert_print(len(force_trials) == len(op_lst), str(len(op_lst)))
    op_perf_paths = [None for _ in op_lst]
    for op_pos, path in kwargs.get("op_perf_model_path", []):
        op_perf_paths[op_pos] = path
    graph_perf_path = kwargs.get("graph_perf_model_path")
    # ``use_model=True`` (what the drivers' --use_model passes): every op's search queries its
    # performance model, stored under the default file names, instead of measuring
    use_model_everywhere = bool(kwargs.get("use_model", False))
    force_inline = bool(kwargs.get("force_inline", False))
    if kwargs.get("rewrite"):
        # search the channels-last form of the task: its twin is registered and searched in its place
        # (the reference evaluates the rewritten layout during the search too, scheduler.py:1055,1085)
        twin = Rewriter.rewritten_task(task)
        passed = {k: v for k, v in kwargs.items() if k != "rewrite"}
        return schedule(twin.key, slevel=slevel, rlevel=rlevel, op_trial=op_trial, graph_trial=graph_trial,
                        op_stop=op_stop, graph_stop=graph_stop, number=number, timeout=timeout, parallel=parallel,
                        method=method, **passed)

    graph_space = generate_space_inter_op(op_lst, down_graph, force_inline=force_inline,
                                          special_space=task.special_space)
    _log("graph space size", len(graph_space))
    total_size = len(graph_space)
    if force_inline:
        configs = Config([], {"inline": [graph_space.subspaces["inline"].static_entities[0]]})
    else:
        configs = Config([], None)

    for pos, op in enumerate(op_lst):
        if task.target == "cuda":
            space = generate_space_intra_op(op, down_graph, slevel=slevel, rlevel=rlevel, groups=3, target="cuda")
        elif task.target == "llvm":
            level = max(slevel, rlevel)
            space = generate_space_intra_op(op, down_graph, slevel=level, rlevel=level, unroll_policy="off",
                                            fuse_policy="off", reorder_policy="off", target="llvm")
        else:
            raise RuntimeError("Currently no support for target %s" % task.target)
        total_size *= len(space)
        _log("op", pos, "space size:", len(space))
        op_scheduler = OpScheduler(task_key, pos, space, parallel=parallel, timeout=timeout, trial=force_trials[pos],
                                   number=number, early_stop=op_stop, measurer=measurer)
        op_scheduler.seeds = [cfg for seed_pos, cfg in kwargs.get("seeds", []) if seed_pos == pos]
        op_scheduler.precision = kwargs.get("precision")
        if (force_inline and graph_space.subspaces["inline"].able_inline(pos)) or not space.subspaces:
            op_config = {}
        else:
            op_config = op_scheduler.schedule(configs, method=method,
                                              use_model=op_perf_paths[pos] is not None or use_model_everywhere,
                                              perf_path=op_perf_paths[pos])
        configs.op_config_lst.append(op_config)
    _log("space size", total_size)

    graph_scheduler = GraphScheduler(task_key, graph_space, parallel=parallel, timeout=timeout, trial=graph_trial,
                                     number=number, early_stop=graph_stop, measurer=measurer)
    graph_scheduler.precision = kwargs.get("precision")
    graph_config = graph_scheduler.schedule(configs, method=method, use_model=graph_perf_path is not None,
                                            perf_path=graph_perf_path)
    configs = Config(configs.op_config_lst, graph_config)
    s, bufs = schedule_with_config(task_key, configs, precision=kwargs.get("precision"))
    return s, bufs, configs


class Rewriter(object):
    """Layout rewrite of a conv2d task, the counterpart of the reference's ``Rewriter``
    (scheduler.py:825-862).  There it turns an NCHW conv2d into the blocked NCHWc form its CPU
    kernels vectorise over; here it turns it into the channels-last form the tensor-core kernels
    read in place (``task.conv2d_nhwc_layout``: NCHWc with one block holding all channels), which
    removes the layout pass from every call.  ``bufs`` change shape, as in the reference:
    [N,H,W,C] input, [K,C/groups,R,S] filter, [N,P,Q,K] result.  The knobs carry over; an
    ``algo`` choice that only exists for NCHW tensors (3: batched GEMM on the tensors as they
    are, 4: im2col form) is left to the library."""

    def __init__(self, configs):
        if not isinstance(configs, Config):
            configs = Config(configs[0], configs[1])
        self.graph_config = configs.graph_config
        self.op_config_lst = configs.op_config_lst

    @staticmethod
    def rewritten_task(task):
        from .task import Task, register_task, conv2d, conv2d_nhwc_layout
        assert_print(task.target == "cuda", "the channels-last rewrite is for the sm_100a kernels")
        assert_print(task.category == "conv2d" and task.func is conv2d, "only conv2d tasks are rewritten")
        twin = Task(task.category, task.name + "-nhwc", conv2d_nhwc_layout, task.args, task.target, task.dev_id)
        register_task(twin)
        return twin

    def rewrite(self, task):
        import copy
        twin = self.rewritten_task(task)
        new_graph_config = copy.deepcopy(self.graph_config)
        new_op_config_lst = copy.deepcopy(self.op_config_lst)
        for cfg in new_op_config_lst:
            if cfg and cfg.get("inline") and cfg["inline"][0] and cfg["inline"][0][0] in (3, 4):
                cfg["inline"] = []
        ops, bufs = twin.func(*twin.args)
        return ops, bufs, new_graph_config, new_op_config_lst


def schedule_with_config(task_key, configs, op_pos=None, rewrite=False, precision=None):
    """Plan a registered task with the given configs; returns ``(plan, bufs)``.  ``rewrite``: plan
    the channels-last form of a conv2d task instead (see ``Rewriter``)."""
    task = TASK_TABLE[task_key]
    if rewrite:
        ops, bufs, graph_config, op_config_lst = Rewriter(configs).rewrite(task)
        configs = Config(op_config_lst, graph_config)
    else:
        ops, bufs = task.func(*task.args)
    return schedule_with_config_ops(ops, bufs, configs, op_pos=op_pos, target=task.target, precision=precision,
                                    dev_id=task.dev_id)


def schedule_with_config_ops(ops, bufs, configs, op_pos=None, target="cuda", precision=None, dev_id=0):
    """Plan an op graph with the given configs (``Config`` or ``[op_config_lst, graph_config]``)."""
    from .runtime import KernelPlan
    if not isinstance(configs, Config):
        configs = Config(configs[0], configs[1])
    op_lst, down_graph = flatten_graph(ops)
    op_states = _op_states(op_lst, down_graph)
    op_config_lst = list(configs.op_config_lst)
    if op_pos is not None:
        assert_print(isinstance(op_pos, int), "op_pos should be int")
        assert_print(op_pos < len(op_lst) and op_pos < len(op_config_lst), "op_pos too big")
    else:
        assert_print(len(op_config_lst) <= len(op_lst), "config length exceed op_lst")
    graph_config = configs.graph_config
    if graph_config and graph_config.get("inline"):
        for state, flag in zip(op_states, graph_config["inline"][0]):
            state.inline = bool(flag)
    plan = KernelPlan(ops, op_lst, op_states, bufs, Config(op_config_lst, graph_config), target=target,
                      op_pos=op_pos, precision=precision, dev_id=dev_id)
    return plan, bufs


def schedule_ops_with_config(s, op_lst, configs, target):
    """Re-plan an already flattened op list (kept for API parity, scheduler.py:1189-1220)."""
    plan, _ = schedule_with_config_ops([op_lst[-1]], s.bufs if hasattr(s, "bufs") else [], configs, target=target)
    return plan
