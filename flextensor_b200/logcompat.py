"""Reads the reference's saved configuration logs and turns them into search seeds.

The reference appends one line per tuned task, ``<task key>:<json of [op_config_lst,
graph_config]>`` (flextensor/optimize/optimize_gemm.py:62-64; files such as
flextensor/optimize/gemm-config.log and flextensor/baselines/flextensor/*-v100.txt).  An op
config there holds loop-split factors of its CUDA template
(flextensor/templates/cuda.py:417-446,546-605): every spatial axis is split four ways into
``[blocks, vthreads, threads, serial]`` and every reduce axis three ways into
``[outer, middle, inner]``.  Those factors do not replay on this backend - its configs hold
the knobs of pre-compiled tcgen05 kernels - but they carry what the reference's search learnt
about a shape: how large a thread block's output tile was along each axis and how the reduction
was staged.  ``knobs_from_reference`` maps that onto the nearest legal knob values, and
``seed_for`` snaps the result into the knob space of the same shape here, ready to be given
to ``schedule(..., seeds=[(op_pos, op_config)])`` as a starting point of the walk.
"""
import json
import math
import re

from .space import B200_LAYOUT, generate_space_intra_op, op_family
from .templates import knobs_to_config
from .utils import Config

_KEY_RE = re.compile(r"^(?P<category>[A-Za-z0-9]+)_(?P<name>.+)_\((?P<args>[^()]*)\)_(?P<target>[a-z]+)\((?P<dev>\d+)\)$")


def parse_line(line):
    """``(task_key, Config)`` of one log line; raises ``ValueError`` on anything else."""
    line = line.strip()
    cut = line.find(":[")
    if cut <= 0:
        raise ValueError("not a '<task key>:<json>' line: %r" % (line[:60],))
    key, payload = line[:cut], line[cut + 1:]
    obj = json.loads(payload)
    if not (isinstance(obj, list) and len(obj) == 2 and isinstance(obj[0], list)):
        raise ValueError("payload is not [op_config_lst, graph_config]")
    return key, Config(obj[0], obj[1])


def read_log(path):
    """All ``(task_key, Config)`` pairs of a log file, blank lines skipped."""
    out = []
    with open(path, "r") as fin:
        for line in fin:
            if line.strip():
                out.append(parse_line(line))
    return out


def parse_key(task_key):
    """Splits ``"{category}_{name}_{args}_{target}({dev})"`` (flextensor/task.py:34) into its
    parts; ``args`` comes back as a tuple of ints."""
    m = _KEY_RE.match(task_key)
    if not m:
        raise ValueError("not a task key: %r" % (task_key,))
    args = tuple(int(x) for x in m.group("args").replace(" ", "").split(",") if x != "")
    return m.group("category"), m.group("name"), args, m.group("target"), int(m.group("dev"))


def block_tiles(op_config):
    """What one thread block of the reference's CUDA template covered: per spatial axis the
    product of the vthread, thread and serial parts, per reduce axis ``(outer, middle * inner)``,
    i.e. the number of shared-memory refills and the extent staged per refill."""
    spatial = [int(f[1]) * int(f[2]) * int(f[3]) for f in op_config.get("spatial", []) if len(f) >= 4]
    reduce_ = [(int(f[0]), int(f[1]) * int(f[2])) for f in op_config.get("reduce", []) if len(f) >= 3]
    return spatial, reduce_


def _depth_for(refills):
    # the more often the reference refilled shared memory, the more a deep pipeline has to hide
    return max(2, min(8, 2 + int(math.ceil(math.log2(max(1, refills))))))


def knobs_from_reference(op, op_config):
    """Kernel knobs suggested by a reference op config for ``op`` (same shape); only knobs the
    reference's factors say something about are set."""
    family = op_family(op)
    spatial, reduce_ = block_tiles(op_config)
    knobs = {}
    if family is None or not spatial:
        return knobs
    refills = 1
    for outer, _ in reduce_:
        refills *= max(1, outer)
    reorder = op_config.get("reorder") or [[0]]
    order = int(reorder[0][0]) if reorder and reorder[0] else 0
    if family == "contraction":
        # axes (i, j) for gemm, (b, i, j) for batch_gemm
        m_tile, n_tile = spatial[-2], spatial[-1]
        knobs["tile_n"] = n_tile
        knobs["cluster"] = 2 if m_tile >= 256 else 1
        knobs["stages"] = _depth_for(refills)
        knobs["split_k"] = 1
        knobs["raster"], knobs["group_m"] = ((1, 0), (2, 0), (3, 8))[min(order, 2)]
    elif family == "conv2d":
        # axes (b, k, h, w); one block covered b*h*w output pixels of k_tile channels
        b_tile, k_tile, h_tile, w_tile = (spatial + [1, 1, 1, 1])[:4]
        knobs["tile_n"] = k_tile
        knobs["tile_h"] = h_tile
        knobs["cluster"] = 2 if b_tile * h_tile * w_tile >= 256 else 1
        knobs["stages"] = _depth_for(refills)
        knobs["split_k"] = 1
        knobs["raster"], knobs["group_m"] = ((1, 0), (2, 0))[min(order, 1)]
    elif family == "depthwise_conv2d":
        # axes (b, c, h, w): rows per strip, threads of the block
        h_tile = spatial[2] if len(spatial) > 2 else 0
        threads = 1
        for f in op_config.get("spatial", []):
            if len(f) >= 4:
                threads *= int(f[2])
        knobs["tile_h"] = h_tile
        knobs["threads"] = threads
    return knobs


def _nearest(entities, wanted):
    """Index of the entity closest to ``wanted`` (first component: smallest not below it, else the
    largest; further components: closest)."""
    wanted = list(wanted) if isinstance(wanted, (list, tuple)) else [wanted]
    firsts = sorted({e[0] for e in entities})
    at_least = [v for v in firsts if v >= wanted[0]]
    first = at_least[0] if at_least else firsts[-1]
    best, best_d = 0, None
    for i, e in enumerate(entities):
        if e[0] != first:
            continue
        d = sum(abs(int(a) - int(b)) for a, b in zip(e[1:], wanted[1:]))
        if best_d is None or d < best_d:
            best, best_d = i, d
    return best


def snap_to_space(space, knobs):
    """``{subspace name: index}`` of the point of ``space`` nearest to ``knobs``; knobs that are
    not given take the sub-space's first entity."""
    indices = {}
    for name, sub in space.subspaces.items():
        entities = sub.static_entities
        if name == "raster":
            wanted = [knobs.get("raster", entities[0][0]), knobs.get("group_m", 0)]
        elif name == "ctas":
            wanted = [8]
        elif name == "algo":
            firsts = [e[0] for e in entities]
            pick = next((a for a in (3, 4, 2, 1) if a in firsts), firsts[0])  # the library's own preference
            wanted = [knobs.get("algo", pick)]
        elif name in knobs:
            wanted = [knobs[name]]
        else:
            indices[name] = 0
            continue
        indices[name] = _nearest(entities, wanted)
    return indices


def seed_for(op, op_config, target="cuda"):
    """A config of this backend's knob space for ``op`` that is nearest to what the reference's
    ``op_config`` says; ``{}`` for ops without a kernel of their own (the padding stage)."""
    space = generate_space_intra_op(op, None, target=target)
    if not space.subspaces:
        return {}
    indices = snap_to_space(space, knobs_from_reference(op, op_config))
    family = op_family(op)
    knobs = {}
    for type_key, names in B200_LAYOUT[family].items():
        for name in names:
            if name not in space.subspaces:
                continue
            entity = space.subspaces[name].static_entities[indices[name]]
            if name == "raster":
                knobs["raster"], knobs["group_m"] = int(entity[0]), int(entity[1])
            elif name == "ctas":
                continue
            else:
                knobs[name] = int(entity[0])
    return knobs_to_config(knobs, op)


def seeds_from_log(path, task_table=None):
    """``{task_key: [(op_pos, op_config), ...]}`` for every line of a reference log whose task
    (same category and argument tuple) is registered here for the CUDA target on device 0.

    The reference's name part of a key varies from file to file ("yolo_batch32", "yolo7", ...):
    tasks are matched by category and argument tuple, not by name.
    """
    if task_table is None:
        from .task import TASK_TABLE as task_table
    by_shape = {}
    for key, task in task_table.items():
        if task.target == "cuda" and task.dev_id == 0:
            by_shape.setdefault((task.category, tuple(task.args)), key)
    out = {}
    for ref_key, config in read_log(path):
        try:
            category, _, args, _, _ = parse_key(ref_key)
        except ValueError:
            continue
        ours = by_shape.get((category, args))
        if ours is None:
            continue
        task = task_table[ours]
        from .scheduler import flatten_graph
        ops, _ = task.func(*task.args)
        op_lst, _ = flatten_graph(ops)
        seeds = []
        for pos, op in enumerate(op_lst):
            if pos < len(config.op_config_lst) and config.op_config_lst[pos]:
                seed = seed_for(op, config.op_config_lst[pos])
                if seed:
                    seeds.append((pos, seed))
        if seeds:
            out[ours] = seeds
    return out
