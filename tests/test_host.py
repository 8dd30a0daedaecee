"""Host-side mirror of the reference interface: helpers, op definitions, task registry,
config space, walkers, search (with a pure-Python cost function standing in for the GPU),
templates and the log-line format.  Runs without a GPU."""
import json
import math
import os
import time

import numpy as np
import pytest
import torch

from flextensor_b200 import scheduler as S
from flextensor_b200 import space as SP
from flextensor_b200.ir import placeholder
from flextensor_b200.model import WalkerGroup, Walker, PerformanceModel, rank_loss
from flextensor_b200.nn import ops
from flextensor_b200.scheduler import schedule, schedule_with_config, flatten_graph
from flextensor_b200.task import Task, TASK_TABLE, register_task, conv2d, gemm
from flextensor_b200.templates import config_to_knobs, knobs_to_config
from flextensor_b200.utils import (Config, any_factor_split, get_factor_lst, gen_enum, gen_group, test_allclose,
                                   assert_print, to_tuple)

S.VERBOSE = False


# ---------------------------------------------------------------- utils
def test_factor_helpers():
    assert get_factor_lst(16) == [1, 16, 2, 8, 4]
    assert get_factor_lst(12) == [1, 12, 2, 6, 3, 4]
    assert get_factor_lst(1) == [1]
    splits = any_factor_split(1024, 4)
    assert len(splits) == 286                      # C(10+3, 3): space size of a 1024-extent axis
    assert all(math.prod(s) == 1024 for s in splits)
    assert len(any_factor_split(1024, 3)) == 66
    assert len(any_factor_split(8192, 4)) == 560 and len(any_factor_split(8192, 3)) == 105
    assert [1, 1, 1, 7] in any_factor_split(7, 4)
    assert gen_enum([1, 0], 2) == [[1, 1], [1, 0], [0, 1], [0, 0]]
    assert gen_group(["a", "b", "c", "d"], most_groups=3) == [[1, 2, 4], [1, 3, 4], [2, 3, 4]]
    assert gen_group(["a", "b"], most_groups=3) == [[1, 2, 2]]
    assert test_allclose(np.ones(3), np.ones(3) * (1 + 1e-7)) == 1
    assert test_allclose(np.ones(3), np.ones(3) * 1.1) == 0
    with pytest.raises(AssertionError):
        assert_print(False, "x")
    assert to_tuple(placeholder((3, 4)).shape) == (3, 4)


# ---------------------------------------------------------------- op definitions
def test_op_definitions_shapes_and_axes():
    x = placeholder((1, 64, 56, 56))
    w = placeholder((64, 64, 3, 3))
    out = ops.conv2d_nchw(x, w, stride=1, padding=1)
    assert to_tuple(out.shape) == (1, 64, 56, 56)
    assert [a.var.name for a in out.op.axis] == ["b", "c", "h", "w"]
    assert [(a.var.name, a.dom.extent.value) for a in out.op.reduce_axis] == [("rc", 64), ("rw", 3), ("rh", 3)]
    padded = out.op.input_tensors[0]
    assert padded.op.name == "Padding" and to_tuple(padded.shape) == (1, 64, 58, 58)
    out = ops.conv2d_nchw(placeholder((4, 6, 7, 7)), placeholder((9, 2, 3, 3)), placeholder((9,)), stride=2,
                          padding=1, dilation=2, groups=3)
    assert to_tuple(out.shape) == (4, 9, 3, 3) and out.op.kind == "bias_add"
    with pytest.raises(AssertionError):
        ops.conv2d_nchw(placeholder((1, 6, 7, 7)), placeholder((9, 4, 3, 3)), groups=3)
    dw = ops.depthwise_conv2d_nchw(placeholder((4, 6, 7, 7)), placeholder((6, 3, 3, 3)), stride=2, padding=1,
                                   dilation=2)
    assert to_tuple(dw.shape) == (4, 18, 3, 3)
    # conv3d: the reference's test case shape (flextensor/test/test_ops.py:187-214) and per-axis parameters
    c3 = ops.conv3d_ncdhw(placeholder((4, 6, 7, 7, 7)), placeholder((9, 2, 3, 3, 3)), placeholder((9,)), stride=2,
                          padding=1, dilation=2, groups=3)
    assert to_tuple(c3.shape) == (4, 9, 3, 3, 3) and c3.op.kind == "bias_add"
    conv = c3.op.input_tensors[0].op
    assert [a.var.name for a in conv.axis] == ["b", "c", "d", "h", "w"]
    assert [(a.var.name, a.dom.extent.value) for a in conv.reduce_axis] == [("rc", 2), ("rd", 3), ("rw", 3), ("rh", 3)]
    assert to_tuple(conv.input_tensors[0].shape) == (4, 6, 9, 9, 9)
    c3 = ops.conv3d_ncdhw(placeholder((1, 8, 5, 9, 6)), placeholder((4, 8, 2, 3, 1)), stride=(1, 2, 3), padding=(1, 0, 2),
                          dilation=(2, 1, 1))
    assert to_tuple(c3.shape) == (1, 4, 5, 4, 4)
    assert to_tuple(ops.zero_pad3d(placeholder((1, 2, 3, 4, 5)), (1, 2, 0, 1, 3, 0)).shape) == (1, 2, 6, 5, 8)
    with pytest.raises(AssertionError):
        ops.conv3d_ncdhw(placeholder((1, 6, 7, 7, 7)), placeholder((9, 4, 3, 3, 3)), groups=3)
    a, b = placeholder((8, 16)), placeholder((16, 4))
    assert to_tuple(ops.gemm(a, b).shape) == (8, 4)
    assert to_tuple(ops.gemm(placeholder((16, 8)), b, transposeA=True).shape) == (8, 4)
    assert to_tuple(ops.gemm(a, placeholder((4, 16)), transposeB=True).shape) == (8, 4)
    assert to_tuple(ops.gemm(placeholder((16, 8)), placeholder((4, 16)), True, True).shape) == (8, 4)
    with pytest.raises(AssertionError):
        ops.gemm(a, placeholder((15, 4)))
    bg = ops.batch_gemm(placeholder((3, 8, 16), "bfloat16"), placeholder((3, 16, 4), "bfloat16"))
    assert to_tuple(bg.shape) == (3, 8, 4) and bg.dtype == "bfloat16"
    with pytest.raises(AssertionError):
        ops.batch_gemm(placeholder((3, 8, 16)), placeholder((2, 16, 4)))
    i8 = ops.gemm_int8(placeholder((8, 16), "int8"), placeholder((16, 4), "int8"))
    assert i8.dtype == "int32"
    with pytest.raises(AssertionError):
        ops.gemm_int8(a, b)


def test_flatten_graph_is_producer_first():
    ops_, bufs = conv2d(1, 8, 6, 6, 4, 3, 1, 1, 1, 1)
    op_lst, down = flatten_graph(ops_)
    assert [op.kind for op in op_lst] == ["pad2d", "conv2d"]
    assert SP.able_inline(op_lst[0], down) and not SP.able_inline(op_lst[1], down)


# ---------------------------------------------------------------- task registry
def test_task_keys_and_registry():
    t = Task("gemm", "gemm", None, (1024, 1024, 1024), "cuda", 0)
    assert t.key == "gemm_gemm_(1024, 1024, 1024)_cuda(0)"
    assert t.key in TASK_TABLE and TASK_TABLE[t.key].func is gemm
    assert "conv2d_res5_(64, 256, 56, 56, 512, 1, 2, 0, 1, 1)_cuda(3)" in TASK_TABLE
    assert "conv2d_res_b13_(1, 64, 56, 56, 64, 3, 1, 1, 1, 1)_cuda(0)" in TASK_TABLE
    assert "conv2d_depthwise_(1, 256, 56, 56, 1, 3, 1, 1, 1)_cuda(0)" in TASK_TABLE
    assert "gemm_batch_gemm_(64, 2048, 2048, 2048)_cuda(7)" in TASK_TABLE
    assert "gemm_gemm_int8_(8192, 8192, 8192)_cuda(0)" in TASK_TABLE
    assert "conv3d_conv3d_(1, 64, 8, 28, 28, 128, 3, 2, 1, 1, 1)_cuda(0)" in TASK_TABLE
    marker = Task("gemm", "gemm", "replaced", (32, 32, 32), "cuda", 0)
    old = TASK_TABLE[marker.key]
    register_task(marker)                          # silent overwrite, as in the reference
    assert TASK_TABLE[marker.key].func == "replaced"
    register_task(old)
    t.set_specific_space("layout", "enum", [[0, 0], [1, 0]])
    assert len(t.special_space["layout"]) == 2
    with pytest.raises(RuntimeError):
        t.set_specific_space("x", "grid", [])


# ---------------------------------------------------------------- space
def test_split_space_invariants_and_moves():
    sp = SP.SplitSpace(4, 1024)
    assert len(sp) == 286 and sp.num_direction == 12
    assert all(math.prod(e) == 1024 for e in sp.static_entities)
    pos = sp.static_entities.index([1, 1, 1, 1024])
    nxt = sp.next_entity(pos, (0, 3))             # move a factor from part 3 to part 0
    assert sp.static_entities[nxt] == [2, 1, 1, 512]
    assert sp.next_entity(pos, (3, 0)) == pos      # nothing left to take from part 0
    assert sp.next_entity(5, (1,)) == 6 and sp.next_entity(0, (-1,)) == len(sp) - 1
    sp7 = SP.SplitSpace(3, 7)
    assert all(math.prod(e) == 7 for e in sp7.static_entities)
    p2 = SP.SplitSpace(2, 6, allow_non_divisible="power2")
    assert [4, 1] in p2.static_entities or [4, 2] in p2.static_entities


def test_reference_style_space_sizes():
    ops_, _ = gemm(1024, 1024, 1024)
    space = SP.generate_space_intra_op(ops_[0], {}, slevel=4, rlevel=3, groups=3, target="llvm")
    sizes = space.length()
    assert sizes["split_i_0"] == 286 and sizes["split_j_1"] == 286 and sizes["split_k_0"] == 66
    assert sizes["reorder"] == 3 and sizes["unroll"] == 8
    assert space.dim == 3 + 4 + 4 + 3 + 1 + 2     # fuse (3 cut positions) + splits + reorder + unroll


def test_b200_space_per_family():
    ops_, _ = gemm(1024, 1024, 1024)
    space = SP.generate_space_intra_op(ops_[0], {}, target="cuda")
    assert list(space.subspaces) == ["tile_n", "cluster", "stages", "split_k", "release", "raster", "ctas"]
    assert space.types["spatial"] == ["tile_n", "cluster"] and space.types["reduce"] == ["stages", "split_k", "release"]
    assert [e[0] for e in space.subspaces["tile_n"].static_entities] == [32, 64, 128, 256, 512]
    for sub in space.subspaces.values():          # every sub-space speaks the walker protocol
        assert sub.num_direction == len(sub.directions) == 2 and len(sub) == len(sub.static_entities) > 0
        assert all(len(e) == sub.dim for e in sub.static_entities)
        assert sub.next_entity(len(sub) - 1, (1,)) == 0
    from flextensor_b200.task import gemm_int8, batch_gemm, depthwise_conv2d
    i8 = SP.generate_space_intra_op(gemm_int8(512, 512, 512)[0][0], {}, target="cuda")
    assert [e[0] for e in i8.subspaces["tile_n"].static_entities] == [128, 256, 512]   # N-contiguous int8 B: 128-wide boxes
    assert [e[0] for e in i8.subspaces["split_k"].static_entities] == [1]         # integer output: no atomics
    bg = SP.generate_space_intra_op(batch_gemm(4, 256, 256, 256)[0][0], {}, target="cuda")
    assert [e[0] for e in bg.subspaces["tile_n"].static_entities] == [64, 128, 256]          # N = 256: no room for a 512 tile
    ops_, _ = conv2d(1, 64, 56, 56, 64, 3, 1, 1, 1, 1)
    op_lst, down = flatten_graph(ops_)
    assert len(SP.generate_space_intra_op(op_lst[0], down, target="cuda").subspaces) == 0   # padding: no kernel
    cv = SP.generate_space_intra_op(op_lst[1], down, target="cuda")
    assert [e[0] for e in cv.subspaces["tile_h"].static_entities] == [1, 2]
    assert 9 in [e[0] for e in cv.subspaces["split_k"].static_entities]
    assert [e[0] for e in cv.subspaces["algo"].static_entities] == [1, 2, 5] and cv.types["inline"] == ["algo"]
    strided = flatten_graph(conv2d(1, 64, 56, 56, 64, 3, 2, 1, 1, 1)[0])
    assert [e[0] for e in SP.generate_space_intra_op(strided[0][1], strided[1], target="cuda")
            .subspaces["algo"].static_entities] == [1]                    # the slab kernel is stride 1 only
    knobs = config_to_knobs({"spatial": [[64], [2], [1]], "inline": [[2]]}, op_lst[1])
    assert knobs == {"tile_n": 64, "tile_h": 2, "cluster": 1, "algo": 2}
    from flextensor_b200.task import conv3d
    c3 = flatten_graph(conv3d(1, 64, 8, 28, 28, 64, 3, 1, 1, 1, 1)[0])
    assert [op.kind for op in c3[0]] == ["pad2d", "conv2d"]
    c3s = SP.generate_space_intra_op(c3[0][1], c3[1], target="cuda")
    assert [e[0] for e in c3s.subspaces["algo"].static_entities] == [1, 5]   # per-tap with a depth-tap loop; slab kernel
    c3_strided = flatten_graph(conv3d(1, 64, 8, 28, 28, 128, 3, 2, 1, 1, 1)[0])
    assert [e[0] for e in SP.generate_space_intra_op(c3_strided[0][1], c3_strided[1], target="cuda")
            .subspaces["algo"].static_entities] == [1]
    assert [e[0] for e in c3s.subspaces["tile_h"].static_entities] == [1, 2, 3, 4]   # rows of the 28 x 28 plane
    assert 9 in [e[0] for e in c3s.subspaces["split_k"].static_entities]      # 27 taps x 2 channel chunks
    dw = SP.generate_space_intra_op(flatten_graph(depthwise_conv2d(1, 256, 56, 56, 1, 3, 1, 1, 1)[0])[0][1], {},
                                    target="cuda")
    assert list(dw.subspaces) == ["tile_h", "threads"]
    inter = SP.generate_space_inter_op(op_lst, down)
    assert inter.subspaces["inline"].static_entities == [[1, 0], [0, 0]]
    assert SP.generate_space_inter_op(op_lst, down, force_inline=True).subspaces["inline"].static_entities == [[1, 0]]


# ---------------------------------------------------------------- templates
def test_config_knob_round_trip():
    ops_, _ = gemm(1024, 1024, 1024)
    op = ops_[0]
    knobs = {"tile_n": 128, "cluster": 2, "stages": 6, "split_k": 1, "release": 2, "raster": 3, "group_m": 8}
    cfg = knobs_to_config(knobs, op)
    assert cfg["spatial"] == [[128], [2]] and cfg["reduce"] == [[6], [1], [2]] and cfg["reorder"] == [[3, 8]]
    assert config_to_knobs(cfg, op) == knobs
    assert config_to_knobs({}, op) == {}
    assert config_to_knobs({"spatial": [[64]]}, op) == {"tile_n": 64}


# ---------------------------------------------------------------- walkers and models
def _toy_space():
    space = SP.Space()
    space.add_subspace("a", SP.KnobSpace("a", [1, 2, 4, 8]), "spatial")
    space.add_subspace("b", SP.KnobSpace("b", [[0, 0], [1, 0], [2, 4]]), "reorder")
    return space


def test_walker_group_memory_and_moves():
    np.random.seed(1)
    torch.manual_seed(1)
    group = WalkerGroup("toy", _toy_space())
    assert group.top1() == {} and group.top1_value() == float("inf") and not group.has_more()
    group.record({"a": 0, "b": 0}, 3.0)
    group.record({"a": 1, "b": 0}, 1.0)
    group.record({"a": 2, "b": 1}, 2.0)
    assert group.top1() == {"a": 1, "b": 0} and group.top1_value() == 1.0
    assert group.ever_met({"a": 0, "b": 0}) and not group.ever_met({"a": 3, "b": 2})
    assert group.flatten({"a": 2, "b": 2}) == [4, 2, 4]
    assert group.to_config({"a": 3, "b": 1})["spatial"] == [[8]]
    assert group.to_config({"a": 3, "b": 1})["reorder"] == [[1, 0]]
    nxt, acts = group.full_walk({"a": 1, "b": 0}, no_repeat=True)
    assert {"a": 0, "b": 0} not in nxt and {"a": 2, "b": 0} in nxt and len(nxt) == len(acts)
    assert group.topk(2) == [{"a": 1, "b": 0}, {"a": 2, "b": 1}] and group.mem_size == 3
    assert group.topk(2, modify=True, with_value=True)[0][1] == 1.0 and group.mem_size == 1
    assert group.pop_top().value == 3.0 and group.pop_top().value == float("inf")
    # a much worse point is (almost surely) rejected when random_reject is on
    group.record({"a": 1, "b": 0}, 1.0)
    before = group.mem_size
    for _ in range(20):
        group.record({"a": 3, "b": 2}, 1e6, random_reject=True)
    assert group.mem_size == before
    frm, nxt, acts = group.walk([({"a": 1, "b": 0}, 1.0)], trial=0)
    assert len(frm) == len(nxt) == len(acts) and all(not group.ever_met(n) or True for n in nxt)


def test_walker_training_and_persistence(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)
    torch.manual_seed(0)
    np.random.seed(0)
    group = WalkerGroup("persist", _toy_space())
    for i in range(40):
        pre = {"a": i % 4, "b": i % 3}
        post = {"a": (i + 1) % 4, "b": i % 3}
        group.add_data("a", pre, (1,), post, 0.5)
        group.add_data("b", pre, 0, {"a": i % 4, "b": (i + 2) % 3}, 0.1)
    group.train_walkers(save=True, verbose=False)
    walker = group.walkers["a"]
    assert os.path.exists(walker.model_path)
    q_before = walker.pre_judger(torch.ones(group.space.dim)).detach().clone()
    fresh = WalkerGroup("persist", _toy_space())
    fresh.load_walker_model()
    assert torch.allclose(fresh.walkers["a"].pre_judger(torch.ones(group.space.dim)), q_before)
    assert torch.allclose(fresh.walkers["a"].post_judger(torch.ones(group.space.dim)), q_before)  # target synced
    group.dump_data()
    fresh.load_walker_data()
    assert fresh.walkers["a"].mem_size == 40
    # performance model: rank loss trains towards the right order
    group.add_perf_data([{"a": 0, "b": 0}, {"a": 3, "b": 2}, {"a": 1, "b": 1}], [3.0, 1.0, 2.0])
    group.train_on_perf(save=True, verbose=False)
    assert len(group.query_performance([{"a": 0, "b": 0}, {"a": 3, "b": 2}])) == 2
    y = torch.tensor([3.0, 1.0])
    assert rank_loss(y, torch.tensor([3.0, 1.0])) < rank_loss(y, torch.tensor([1.0, 3.0]))
    assert PerformanceModel(5)(torch.zeros(2, 5)).shape == (2, 1)


# ---------------------------------------------------------------- search with a fake measurer
def _fake_measurer(log=None):
    def measure(jobs, number=1, timeout=1.0, parallel=1):
        out = []
        for task_key, cfg, op_pos in jobs:
            plan, _ = schedule_with_config(task_key, cfg, op_pos=op_pos)
            kn = plan.steps[-1].knobs if plan.steps else {}
            cost = (1.0 + abs(kn.get("tile_n", 64) - 128) / 64 + abs(kn.get("stages", 4) - 5) * 0.1 +
                    (0.5 if kn.get("cluster", 1) == 1 else 0.0) + 0.05 * kn.get("split_k", 1))
            if kn.get("stages") == 8:
                cost = float("inf")                # a candidate that "fails to run"
            out.append(cost)
            if log is not None:
                log.append((task_key, op_pos, parallel))
        return out
    return measure


GEMM_KEY = "gemm_batch_gemm_(4, 256, 512, 384)_cuda(0)"


@pytest.mark.parametrize("method", ["searching", "random"])
def test_schedule_finds_the_optimum_of_a_fake_cost(method):
    np.random.seed(0)
    torch.manual_seed(0)
    plan, bufs, configs = schedule(GEMM_KEY, op_trial=12, op_stop=6, timeout=1, parallel=4, method=method,
                                   measurer=_fake_measurer())
    knobs = plan.steps[0].knobs
    assert knobs["tile_n"] == 128 and knobs["cluster"] == 2 and knobs["stages"] in (4, 5, 6)
    assert isinstance(configs, Config) and len(configs.op_config_lst) == 1
    assert [to_tuple(b.shape) for b in bufs] == [(4, 256, 512), (4, 512, 384), (4, 256, 384)]


def test_schedule_is_deterministic_under_a_seed():
    results = []
    for _ in range(2):
        np.random.seed(123)
        torch.manual_seed(123)
        _, _, configs = schedule(GEMM_KEY, op_trial=4, op_stop=3, timeout=1, parallel=2, method="searching",
                                 measurer=_fake_measurer())
        results.append(json.dumps(configs))
    assert results[0] == results[1]


def test_q_method_runs_and_trains(tmp_path, monkeypatch):
    monkeypatch.chdir(tmp_path)                    # walker checkpoints land in the working directory
    np.random.seed(0)
    torch.manual_seed(0)
    plan, _, _ = schedule(GEMM_KEY, op_trial=5, op_stop=5, timeout=1, parallel=2, method="q",
                          measurer=_fake_measurer())
    assert plan.steps[0].knobs["tile_n"] in (64, 128, 256)
    assert any(f.startswith("walker_judger_model_") for f in os.listdir(tmp_path))


def test_conv_graph_search_and_log_round_trip():
    np.random.seed(0)
    torch.manual_seed(0)
    key = "conv2d_res_b13_(1, 64, 56, 56, 64, 3, 1, 1, 1, 1)_cuda(0)"
    log = []
    plan, bufs, configs = schedule(key, op_trial=6, op_stop=3, timeout=1, parallel=2, trials=[1, 6],
                                   measurer=_fake_measurer(log))
    assert configs.op_config_lst[0] == {}          # the padding stage has no kernel of its own
    assert [s.op.kind for s in plan.steps] == ["conv2d"]
    assert any(p == 1 for _, _, p in log)          # leaders were re-measured serially
    line = key + ":" + json.dumps(configs)         # the drivers' log line
    name, string = line.split(":", 1)
    obj = json.loads(string)
    replay, _ = schedule_with_config(name, Config(obj[0], obj[1]))
    assert replay.steps[0].knobs == plan.steps[0].knobs
    # defaults when no config is given
    default_plan, _ = schedule_with_config(key, Config([{}, {}], None))
    assert default_plan.steps[0].knobs == {"fp32_mode": 0}
    strict, _ = schedule_with_config(key, Config([{}, {}], None), precision="3xtf32")
    assert strict.steps[0].knobs == {"fp32_mode": 1}


def test_all_candidates_failing_gives_up_cleanly():
    def broken(jobs, number=1, timeout=1.0, parallel=1):
        return [float("inf")] * len(jobs)
    sched = S.OpScheduler(GEMM_KEY, 0, SP.generate_space_intra_op(TASK_TABLE[GEMM_KEY].func(
        *TASK_TABLE[GEMM_KEY].args)[0][0], {}, target="cuda"), parallel=2, timeout=1.0, trial=2, measurer=broken)
    sched._warm_up(1, 3, Config([], None), [], max_repeat=3)
    assert sched.walker_group.top1() == {} and sched.timeout == 1.0     # timeout restored after the doubling


def test_bias_is_folded_and_unsupported_targets_refused():
    x, w, b = placeholder((1, 8, 6, 6)), placeholder((4, 8, 3, 3)), placeholder((4,))
    out = ops.conv2d_nchw(x, w, b, padding=1)
    plan, _ = S.schedule_with_config_ops([out.op], [x, w, b, out], Config([], None))
    assert [s.op.kind for s in plan.steps] == ["conv2d"] and plan.steps[0].bias is b and plan.steps[0].out is out
    llvm_plan, _ = schedule_with_config("gemm_gemm_(32, 32, 32)_llvm(0)", Config([{}], None))
    with pytest.raises(RuntimeError):
        llvm_plan.build()
    with pytest.raises(AssertionError):        # only conv2d tasks have a layout rewrite
        schedule_with_config(GEMM_KEY, Config([{}], None), rewrite=True)


def test_layout_rewrite_of_a_conv2d_task():
    """schedule_with_config(..., rewrite=True) plans the channels-last twin of a conv2d task (the reference's
    Rewriter, scheduler.py:825-862, produces NCHWc buffers for its CPU target)."""
    key = "conv2d_res_b13_(1, 64, 56, 56, 64, 3, 1, 1, 1, 1)_cuda(0)"
    cfg = Config([{}, {"spatial": [[64], [2], [1]], "inline": [[3]]}], None)
    plan, bufs = schedule_with_config(key, cfg, rewrite=True)
    assert [to_tuple(b.shape) for b in bufs] == [(1, 56, 56, 64), (64, 64, 3, 3), (1, 56, 56, 64)]
    assert [s.op.kind for s in plan.steps] == ["conv2d"] and plan.steps[0].op.attrs["form"] == "nhwc"
    assert plan.steps[0].knobs == {"tile_n": 64, "tile_h": 2, "cluster": 1, "fp32_mode": 0}   # algo 3 is NCHW-only
    assert cfg.op_config_lst[1]["inline"] == [[3]]                                           # the caller's config is untouched
    assert "conv2d_res_b13-nhwc_(1, 64, 56, 56, 64, 3, 1, 1, 1, 1)_cuda(0)" in TASK_TABLE
    ops_, _ = S.Rewriter(cfg).rewrite(TASK_TABLE[key])[:2]
    op_lst, down = flatten_graph(ops_)
    space = SP.generate_space_intra_op(op_lst[1], down, target="cuda")
    assert [e[0] for e in space.subspaces["algo"].static_entities] == [1, 2, 5]
    out = ops.conv2d_nhwc(placeholder((4, 7, 7, 8)), placeholder((12, 4, 3, 3)), placeholder((12,)), stride=2, padding=1,
                          dilation=2, groups=2)
    assert to_tuple(out.shape) == (4, 3, 3, 12) and out.op.attrs["axis"] == 3
    with pytest.raises(AssertionError):
        schedule_with_config("conv2d_depthwise_(1, 256, 56, 56, 1, 3, 1, 1, 1)_cuda(0)", Config([], None), rewrite=True)


# ---------------------------------------------------------------- measurement plumbing (host-side failures)
def _sleepy(seconds):
    time.sleep(seconds)
    return 42.0


def _raiser():
    raise ValueError("candidate failed")


def test_master_routine_timeout_and_failure():
    from flextensor_b200.measure import master_routine
    assert master_routine(20, _sleepy, 0.01) == 42.0
    res = master_routine(0.5, _sleepy, 30)
    assert isinstance(res, Exception)
    res = master_routine(20, _raiser)
    assert isinstance(res, ValueError)


def test_offline_training_round_trip(tmp_path, monkeypatch):
    """Search data dumped by one run trains the models another run searches against
    (flextensor/train.py flow): dump -> train -> schedule(use the performance model, no measurements)."""
    from flextensor_b200 import train
    monkeypatch.chdir(tmp_path)
    np.random.seed(0)
    torch.manual_seed(0)
    group = train.group_for(GEMM_KEY, 0)
    measure = _fake_measurer()
    names = list(group.walkers)
    for i in range(12):
        drawn = group.forward(4)
        points = [{n: int(drawn[n][1][j]) for n in names} for j in range(4)]
        costs = measure([(GEMM_KEY, Config([group.to_config(p)], None), 0) for p in points])
        costs = [min(c, 50.0) for c in costs]
        group.add_perf_data(points, costs)
        for p in points:
            nxt, acts = group.full_walk(p, no_repeat=False)
            group.add_data(acts[0][0], p, acts[0][1], nxt[0], 0.25)
    group.dump_data()
    trained, loss = train.train_performance(GEMM_KEY, 0, verbose=False)
    assert os.path.exists(trained.model_path) and loss >= 0.0
    train.train_walkers(GEMM_KEY, 0, verbose=False)
    calls = []

    def counting(jobs, number=1, timeout=1.0, parallel=1):
        calls.append(len(jobs))
        return measure(jobs)

    plan, _, _ = schedule(GEMM_KEY, op_trial=3, op_stop=2, timeout=1, parallel=2, measurer=counting,
                          op_perf_model_path=[(0, trained.model_path)])
    assert plan.steps[0].knobs["tile_n"] in (64, 128, 256)
    assert sum(calls) <= 4      # the op search ran on the model; only the tiny graph search measured


def test_saved_search_log_replays():
    """flextensor_b200/optimize/b200-config.log holds `key:json(configs)` lines found by searches on a
    B200; every line must plan (the drivers' --test path reads it the same way)."""
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "flextensor_b200", "optimize",
                        "b200-config.log")
    count = 0
    with open(path) as fin:
        for line in fin:
            name, string = line.split(":", 1)
            obj = json.loads(string)
            plan, bufs = schedule_with_config(name, Config(obj[0], obj[1]))
            assert plan.steps and name in TASK_TABLE
            count += 1
    assert count >= 5


def test_driver_registers_the_tasks_it_creates(monkeypatch, tmp_path):
    """The per-operator drivers build task keys that are not in the table beforehand: the search
    leg registers them, and the --test leg rebuilds them from the keys of the log."""
    from flextensor_b200.optimize import driver
    from flextensor_b200.task import conv2d
    monkeypatch.setattr(driver, "evaluate", lambda *a, **k: 0.0)
    shape = (2, 16, 10, 12, 24, 3, 1, 1, 1, 1)
    key = "conv2d_conv2d_%s_cuda(0)" % (shape,)
    TASK_TABLE.pop(key, None)
    log = tmp_path / "conv.log"
    with open(log, "w") as flog:
        got = driver.optimize("conv2d", "conv2d", conv2d, [shape], lambda s_: tuple(s_), trials=2, timeout=1,
                              parallel=1, logfile=flog, trials_of=lambda t: [1, t], measurer=_fake_measurer())
    assert key in got and key in TASK_TABLE
    line = open(log).read().strip()
    assert line.startswith(key + ":")
    TASK_TABLE.pop(key)
    driver._register_from_key(key, "conv2d", "conv2d", conv2d)
    assert TASK_TABLE[key].args == shape and TASK_TABLE[key].target == "cuda" and TASK_TABLE[key].dev_id == 0
    obj = json.loads(line.split(":", 1)[1])
    plan, _ = schedule_with_config(key, Config(obj[0], obj[1]))
    assert plan.steps


# ---------------------------------------------------------------- reference config logs as search seeds
def _reference_lines():
    # line 1 of flextensor/optimize/gemm-config.log and line 2 of
    # flextensor/baselines/flextensor/yolo-conv2d-b32-v100.txt, verbatim
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "reference_config_lines.txt")
    with open(path) as fin:
        return [ln for ln in fin.read().splitlines() if ln.strip()]


def test_logcompat_parses_reference_lines():
    from flextensor_b200 import logcompat as L
    gemm_line, conv_line = _reference_lines()
    key, cfg = L.parse_line(gemm_line)
    assert key == "gemm_gemm_(256, 128, 128)_opencl(0)"
    assert L.parse_key(key) == ("gemm", "gemm", (256, 128, 128), "opencl", 0)
    assert cfg.op_config_lst[0]["spatial"] == [[64, 1, 2, 2], [1, 1, 32, 4]]
    assert cfg.op_config_lst[0]["reduce"] == [[2, 32, 2]]
    # one thread block covered 1*2*2 = 4 rows and 1*32*4 = 128 columns; K came in 2 refills of 64
    assert L.block_tiles(cfg.op_config_lst[0]) == ([4, 128], [(2, 64)])
    key, cfg = L.parse_line(conv_line)
    category, name, args, target, dev = L.parse_key(key)
    assert (category, name, target, dev) == ("conv2d", "conv2d_yolo_batch32", "cuda", 0)
    assert args == (32, 64, 112, 112, 192, 3, 1, 1, 1, 1)
    assert len(cfg.op_config_lst) == 2 and cfg.graph_config["inline"] == [[0, 0]]
    with pytest.raises(ValueError):
        L.parse_line("no payload here")


def test_logcompat_maps_reference_factors_to_legal_knobs():
    from flextensor_b200 import logcompat as L
    from flextensor_b200.space import generate_space_intra_op
    from flextensor_b200.task import Task, conv2d, gemm
    from flextensor_b200.templates import config_to_knobs
    gemm_line, conv_line = _reference_lines()
    _, cfg = L.parse_line(gemm_line)
    op = gemm(256, 128, 128)[0][0]
    knobs = L.knobs_from_reference(op, cfg.op_config_lst[0])
    assert knobs["tile_n"] == 128 and knobs["cluster"] == 1 and knobs["split_k"] == 1 and knobs["stages"] == 3
    seed = L.seed_for(op, cfg.op_config_lst[0])
    space = generate_space_intra_op(op, None, target="cuda")
    for type_key, names in space.types.items():                     # every entity is a member of its sub-space
        for name, entity in zip(names, seed[type_key]):
            assert list(entity) in [list(e) for e in space.subspaces[name].static_entities]
    assert config_to_knobs(seed, op)["tile_n"] == 128
    # conv2d: the second op config of the line belongs to the convolution (the first to its padding stage)
    key, cfg = L.parse_line(conv_line)
    args = L.parse_key(key)[2]
    op = conv2d(*args)[0][0]
    knobs = L.knobs_from_reference(op, cfg.op_config_lst[1])
    # spatial [[8,2,2,1],[2,6,2,8],[14,1,8,1],[28,1,4,1]]: 96 channels x (4 images x 8 rows x 4 columns) per block
    assert knobs["tile_n"] == 96 and knobs["tile_h"] == 8 and knobs["cluster"] == 1
    seed = L.seed_for(op, cfg.op_config_lst[1])
    got = config_to_knobs(seed, op)
    assert got["tile_n"] == 128                                       # smallest legal tile not below 96
    assert got["tile_h"] == 1                                         # a 112-pixel row fills a 128-row tile
    assert got["algo"] == 2                                           # 3x3 stride 1: the slab kernel


def test_schedule_measures_seeds_first(tmp_path):
    """Seeds from a reference log are measured before the warm-up and can win the search."""
    from flextensor_b200 import logcompat as L
    from flextensor_b200.scheduler import schedule
    from flextensor_b200.templates import config_to_knobs
    path = tmp_path / "ref.log"
    path.write_text(_reference_lines()[0] + "\n")
    seeds = L.seeds_from_log(str(path))
    key = "gemm_gemm_(256, 128, 128)_cuda(0)"
    assert list(seeds) == [key]
    seen = []

    def measurer(jobs, number=1, timeout=5.0, parallel=None):
        out = []
        for task_key, config, op_pos in jobs:
            from flextensor_b200.task import TASK_TABLE
            op = TASK_TABLE[task_key].func(*TASK_TABLE[task_key].args)[0][0]
            knobs = config_to_knobs(config.op_config_lst[-1], op)
            seen.append(knobs)
            # the seed (tile 128, one CTA, 3 stages) is the optimum of this made-up cost
            out.append(1.0 + abs(knobs["tile_n"] - 128) / 64.0 + abs(knobs["stages"] - 3) + (knobs["cluster"] - 1))
        return out

    import flextensor_b200.scheduler as S
    old = S.VERBOSE
    S.VERBOSE = False
    try:
        s, bufs, configs = schedule(key, op_trial=2, op_stop=1, graph_trial=1, parallel=2, method="searching",
                                    measurer=measurer, seeds=seeds[key])
    finally:
        S.VERBOSE = old
    assert seen[0]["tile_n"] == 128 and seen[0]["stages"] == 3 and seen[0]["cluster"] == 1   # measured first
    op = s.steps[0].op
    final = config_to_knobs(configs.op_config_lst[0], op)
    assert (final["tile_n"], final["stages"], final["cluster"]) == (128, 3, 1)
