"""Schedule design space.

The container types (``Space``, ``SubSpace`` and its kinds) behave as in the reference's
``flextensor/space.py`` so that the walkers of ``model.py`` drive them unchanged: every
sub-space has ``static_entities``, ``dim`` (length of one entity), ``directions``,
``num_direction``, ``next_entity(pos, direction)`` and ``get_direction(num)``
(space.py:85-365).  ``SplitSpace`` keeps the factor-split entities and the
"move a factor from one position to another" neighbourhood (space.py:112-167).

What changed is what the sub-spaces of a CUDA task *mean*.  The reference's knobs are
loop-split factors for a generated CUDA-core kernel (templates/cuda.py:390-661); here
they are the launch parameters of the hand-written sm_100a kernels (``struct
ftb_config``).  ``generate_space_intra_op`` builds, per op kind:

  type key   sub-space (entity)                      reference knob it takes the place of
  spatial    tile_n [n]      cluster [c]             thread x serial tile / vthread split
             tile_h [h]      threads [t]             (conv rows per tile; depthwise rows per thread/strip, CTA size)
  reduce     stages [s]      split_k [k]             reduce split [outer, mid, inner]
  reorder    raster [mode, group_m]                  reorder position
  unroll     ctas   [fraction of SMs in eighths]     unroll depth (how much work is in flight)

An llvm task (CPU baseline harness) still gets the reference's factor-split space.
"""
import math

import numpy as np

from .utils import any_factor_split, assert_print, gen_enum, gen_group, is_power_of_x


def able_inline(op, down_graph):
    """A compute op with no reduction whose outputs are all consumed inside the graph."""
    is_compute = hasattr(op, "axis") and hasattr(op, "kind")
    has_reduce = bool(getattr(op, "reduce_axis", None))
    is_output = any(op.output(i) not in down_graph for i in range(op.num_outputs))
    return is_compute and (not has_reduce) and (not is_output)


class Space(object):
    valid_type_keys = ["fuse", "spatial", "reduce", "reorder", "inline", "unroll", "merge", "special"]

    def __init__(self):
        self.subspaces = {}
        self.types = {key: [] for key in self.valid_type_keys}
        self.dim = 0

    def add_subspace(self, name, subspace, type_key, override=False):
        if name in self.subspaces and not override:
            raise RuntimeError("Same subspace name")
        assert_print(type_key in self.valid_type_keys)
        self.subspaces[name] = subspace
        self.types[type_key].append(name)
        self.dim += subspace.dim

    def items(self):
        return self.subspaces.items()

    def __len__(self):
        total = 1
        for sub in self.subspaces.values():
            total *= len(sub)
        return total

    def length(self):
        sizes = {name: len(sub) for name, sub in self.subspaces.items()}
        total, added = 1, 0
        for v in sizes.values():
            total *= v
            added += v
        sizes["total"] = total
        sizes["added"] = added
        return sizes


DirectedSubSpaceTypeKeys = ["spatial", "reduce"]
UndirectedSubSpaceTypeKeys = ["fuse", "reorder", "unroll", "inline", "merge", "special"]


class SubSpace(object):
    """Base: an ordered list of entities with a cyclic +-1 neighbourhood."""

    type_key = None

    def __init__(self, entities=None, dim=0):
        self.static_entities = list(entities) if entities is not None else []
        self.dim = dim
        self.size = len(self.static_entities)
        self.num_direction = 2
        self.directions = [(-1,), (1,)]

    def random_entity(self):
        return self.static_entities[np.random.randint(0, self.size)]

    def next_entity(self, pos, d):
        if len(d) == 1:
            return (pos + d[0]) % self.size
        raise RuntimeError("Not support for direction more than one dim: {}".format(d))

    def get_entity(self, p):
        return self.static_entities[p]

    def get_direction(self, num):
        return self.directions[num % self.num_direction]

    def __len__(self):
        return self.size


class SplitSpace(SubSpace):
    """All ordered factorisations of ``total`` into ``dim`` parts."""

    type_key = "split"

    def __init__(self, dim, total, allow_non_divisible="off"):
        super().__init__(any_factor_split(total, dim, allow_non_divisible=allow_non_divisible), dim)
        self.total = total
        self.allow_non_divisible = allow_non_divisible
        self.directions = [(i, j) for i in range(dim) for j in range(dim) if i != j]
        self.num_direction = dim * (dim - 1)
        self._index = {tuple(e): i for i, e in enumerate(self.static_entities)}

    def _admissible(self, cand, product):
        if self.allow_non_divisible == "continuous":
            return True
        if self.allow_non_divisible == "power2" and is_power_of_x(2, cand):
            return True
        return product % cand == 0

    def next_entity(self, pos, d):
        if len(d) == 1:
            return (pos + d[0]) % self.size
        if len(d) != 2:
            raise RuntimeError("Not support for direction more than two dims: {}".format(d))
        asc, dec = d
        assert_print(0 <= asc < self.dim and 0 <= dec < self.dim and asc != dec)
        cur = list(self.static_entities[pos])
        product = cur[asc] * cur[dec]
        # grow the ascending factor to its next admissible value, give the rest to the other
        while True:
            cand = cur[asc] + 1
            while cand <= product and not self._admissible(cand, product):
                cand += 1
            cand = min(cand, product)
            cur[asc] = cand
            cur[dec] = math.ceil(product / cand)
            hit = self._index.get(tuple(cur))
            if hit is not None:
                return hit
            if cand >= product:  # cannot grow further: stay (the reference would spin here)
                return pos


class FuseSpace(SubSpace):
    type_key = "fuse"

    def __init__(self, dim, elements):
        super().__init__(gen_group(elements, most_groups=dim), dim)


class ReorderSpace(SubSpace):
    type_key = "reorder"

    def __init__(self, num_spatial_axis):
        super().__init__([[i] for i in range(num_spatial_axis)], 1)


class UnrollSpace(SubSpace):
    type_key = "unroll"

    def __init__(self, steps, explicit=False):
        flags = [1] if explicit else [0, 1]
        super().__init__([[step, flag] for step in steps for flag in flags], 2)
        self.steps = steps


class PosSpace(SubSpace):
    type_key = "local"

    def __init__(self, parts, num_axis):
        super().__init__([[i, j] for i in range(parts) for j in range(num_axis)], 2)
        self.parts = parts
        self.num_axis = num_axis


class _MaskSpace(SubSpace):
    """0/1 choice per op over a list of eligible op positions (inline / merge)."""

    def __init__(self, eligible, op_num, force=False):
        entities = []
        combos = [[1] * len(eligible)] if force else gen_enum([1, 0], len(eligible))
        for combo in combos:
            entity = [0] * op_num
            for pos, bit in zip(eligible, combo):
                entity[pos] = bit
            entities.append(entity)
        super().__init__(entities, op_num)
        self._eligible = list(eligible)


class InlineSpace(_MaskSpace):
    type_key = "inline"

    def __init__(self, inline_op_pos, op_num, force_inline=False):
        super().__init__(inline_op_pos, op_num, force=force_inline)
        self.able_inline_list = self._eligible

    def able_inline(self, pos):
        return pos in self.able_inline_list


class MergeSpce(_MaskSpace):
    type_key = "merge"

    def __init__(self, merge_op_pos, op_num, force_merge=False):
        super().__init__(merge_op_pos, op_num, force=force_merge)
        self.able_merge_list = self._eligible

    def able_merge(self, pos):
        return pos in self.able_merge_list


class EnumSpace(SubSpace):
    """User-supplied list of knob values (``Task.set_specific_space``)."""

    type_key = "special"

    def __init__(self, knobs):
        super().__init__(knobs, 2)


class KnobSpace(SubSpace):
    """One kernel launch parameter with an ordered list of legal values."""

    type_key = "knob"

    def __init__(self, name, values):
        values = [v if isinstance(v, (list, tuple)) else [v] for v in values]
        super().__init__([list(v) for v in values], len(values[0]))
        self.name = name


def generate_inline_space(op_lst, down_graph, force_inline=False):
    eligible = [i for i, op in enumerate(op_lst) if able_inline(op, down_graph)]
    return InlineSpace(eligible, len(op_lst), force_inline=force_inline)


def generate_merge_space(op_lst, down_graph, force_merge=False):
    return MergeSpce(list(range(len(op_lst))), len(op_lst), force_merge=force_merge)


def generate_fuse_space(loops, groups):
    return FuseSpace(groups, loops)


def generate_split_space(extent, nparts, allow_non_divisible="off"):
    return SplitSpace(nparts, extent, allow_non_divisible=allow_non_divisible)


def generate_reorder_space(num_spatial_axis):
    return ReorderSpace(num_spatial_axis)


def generate_unroll_space(explicit=False):
    return UnrollSpace([0, 1, 512, 1500], explicit=explicit)


def generate_space_intra_op_llvm(op, down_graph, slevel=4, rlevel=3, groups=3, split_policy="off",
                                 unroll_policy="off", fuse_policy="fuse_spatial", reorder_policy="last"):
    """The reference's loop-split space (space.py:397-432); used for llvm-target tasks."""
    space = Space()
    names = [x.var.name for x in op.axis]
    extents = [x.dom.extent.value for x in op.axis]
    rnames = [x.var.name for x in op.reduce_axis]
    rextents = [x.dom.extent.value for x in op.reduce_axis]
    if fuse_policy == "fuse_spatial":
        space.add_subspace("fuse_spatial", generate_fuse_space(names, groups), "fuse")
    for i, (name, extent) in enumerate(zip(names, extents)):
        space.add_subspace("split_{}_{}".format(name, i),
                           generate_split_space(extent, slevel, allow_non_divisible=split_policy), "spatial")
    for i, (name, extent) in enumerate(zip(rnames, rextents)):
        space.add_subspace("split_{}_{}".format(name, i),
                           generate_split_space(extent, rlevel, allow_non_divisible=split_policy), "reduce")
    if reorder_policy == "last":
        space.add_subspace("reorder", generate_reorder_space(groups), "reorder")
    space.add_subspace("unroll", generate_unroll_space(explicit=(unroll_policy == "explicit")), "unroll")
    return space


# ---------------------------------------------------------------- B200 kernel knobs
# Positional layout of a CUDA-target op config (what ``to_config`` emits and the kernel
# template in ``templates.py`` reads back).
B200_LAYOUT = {
    "contraction": {"spatial": ["tile_n", "cluster"], "reduce": ["stages", "split_k", "release"], "reorder": ["raster"],
                    "unroll": ["ctas"]},
    "conv2d": {"spatial": ["tile_n", "tile_h", "cluster"], "reduce": ["stages", "split_k"], "reorder": ["raster"],
               "unroll": ["ctas"], "inline": ["algo"]},
    "depthwise_conv2d": {"spatial": ["tile_h", "threads"], "reduce": [], "reorder": [], "unroll": []},
}

_ELEM_BYTES = {"float32": 4, "bfloat16": 2, "int8": 1}


def op_family(op):
    kind = getattr(op, "kind", None)
    if kind in ("gemm", "batch_gemm", "gemm_int8"):
        return "contraction"
    if kind in ("conv2d", "depthwise_conv2d"):
        return kind
    return None


def _divisor_like(extent, candidates):
    vals = [c for c in candidates if c <= extent]
    return vals or [min(candidates)]


def generate_space_intra_op_b200(op, down_graph=None):
    """Knob space of the sm_100a kernel that serves ``op`` (empty for ops that need no kernel
    of their own, e.g. the padding stage, which the conv kernels fold into their loads)."""
    space = Space()
    family = op_family(op)
    if family is None:
        return space
    extents = {x.var.name: x.dom.extent.value for x in op.axis}
    if family == "contraction":
        n_extent = extents["j"]
        m_extent = extents["i"]
        in_dtype = op.input_tensors[0].dtype
        esize = _ELEM_BYTES.get(in_dtype, 4)
        transposed_b = op.attrs.get("transposeB", False)
        # an N-contiguous B is staged in 128-byte wide column blocks per CTA
        gran = 32 if transposed_b else max(32, 128 // esize)
        tiles = [t for t in (32, 64, 128, 256) if t % gran == 0]
        clusters = [1, 2] if m_extent > 128 else [1]
        if 2 in clusters and n_extent > 256:
            tiles.append(512)                       # 256 x 512 tile of a CTA pair (refused with cluster 1)
        space.add_subspace("tile_n", KnobSpace("tile_n", tiles), "spatial")
        space.add_subspace("cluster", KnobSpace("cluster", clusters), "spatial")
        k_extent = op.reduce_axis[0].dom.extent.value
        num_kb = max(1, math.ceil(k_extent * esize / 128))
        space.add_subspace("stages", KnobSpace("stages", [2, 3, 4, 5, 6, 7, 8]), "reduce")
        f32_out = op.output(0).dtype == "float32"
        splits = [s for s in (1, 2, 4, 8) if s <= num_kb] if f32_out else [1]
        space.add_subspace("split_k", KnobSpace("split_k", splits), "reduce")
        # stages handed back to the loader one by one, or two at a time (half the commits)
        space.add_subspace("release", KnobSpace("release", [1, 2]), "reduce")
        space.add_subspace("raster", KnobSpace("raster", [[1, 0], [2, 0], [3, 2], [3, 4], [3, 8], [3, 16]]), "reorder")
        space.add_subspace("ctas", KnobSpace("ctas", [8, 7, 6, 4]), "unroll")
    elif family == "conv2d":
        # axes (b, c, h, w); a conv1d has (b, c, l) and runs as a one-row image, the packed 1x1 form
        # has (b, k, i) and runs as a one-column image, a conv3d has (b, c, d, h, w) and tiles the
        # (h, w) plane of every output depth
        form = op.attrs.get("form")
        k_out = extents.get("c", extents.get("k")) // op.attrs.get("groups", 1)
        if form == "conv1d":
            out_h, out_w = 1, extents["l"]
        elif form == "packed_1x1":
            out_h, out_w = extents["i"], 1
        else:
            out_h, out_w = extents["h"], extents["w"]
        tiles = [t for t in (32, 64, 128, 256) if t <= max(32, 2 * k_out)]
        space.add_subspace("tile_n", KnobSpace("tile_n", tiles), "spatial")
        tile_w = min(out_w, 128)
        max_h = max(1, 128 // tile_w)
        space.add_subspace("tile_h", KnobSpace("tile_h", [h for h in range(1, max_h + 1) if h <= out_h]), "spatial")
        space.add_subspace("cluster", KnobSpace("cluster", [1, 2]), "spatial")
        rc = op.reduce_axis[0].dom.extent.value
        taps = 1
        for axis in op.reduce_axis[1:]:
            taps *= axis.dom.extent.value
        num_kb = taps * math.ceil(rc / 32)
        space.add_subspace("stages", KnobSpace("stages", [2, 3, 4, 5, 6, 7, 8]), "reduce")
        space.add_subspace("split_k", KnobSpace("split_k", [s for s in (1, 2, 3, 4, 6, 9) if s <= num_kb]), "reduce")
        space.add_subspace("raster", KnobSpace("raster", [[1, 0], [2, 0]]), "reorder")
        space.add_subspace("ctas", KnobSpace("ctas", [8, 6, 4]), "unroll")
        # 1 = one shifted input tile per filter tap; 2 = one input slab per channel chunk shared by
        # all taps with the filter resident in shared memory (stride 1, one group, <= 256 channels
        # out) or, when it does not fit, streamed through a ring of stages; 5 = the same kernel with
        # the filter streamed whatever its size; 3 = batched GEMM on the NCHW tensors as they are (1x1,
        # stride 1, no padding)
        unit_stride = tuple(op.attrs.get("stride", (1, 1))) == (1, 1)
        one_group = op.attrs.get("groups", 1) == 1
        slab_ok = taps > 1 and one_group and k_out <= 256 and unit_stride
        # (the padding stage feeding this op is the identity when padding is 0)
        gemm_ok = (taps == 1 and one_group and unit_stride and tuple(op.attrs.get("padding", (0, 0))) == (0, 0)
                   and (out_h * out_w) % 4 == 0 and rc % 4 == 0)
        # 4 = a 1x1 conv over the im2col form (at most 8 input channels under a filter of 4 taps or more)
        im2col_ok = one_group and rc <= 8 and taps >= 4
        algos = [1] + ([2, 5] if slab_ok else []) + ([3] if gemm_ok else []) + ([4] if im2col_ok else [])
        if form == "conv3d":
            # the per-tap lowering with its depth-tap loop; at stride 1 also the slab kernel with one
            # slab per (depth tap, channel chunk) and a streamed filter
            unit3 = tuple(op.attrs.get("stride", (1, 1, 1))) == (1, 1, 1)
            algos = [1] + ([5] if taps > 1 and one_group and k_out <= 256 and unit3 else [])
        elif form == "nhwc":
            algos = [1] + ([2, 5] if slab_ok else [])  # read in place: no NCHW batched GEMM, no im2col form
        space.add_subspace("algo", KnobSpace("algo", algos), "inline")
    else:  # depthwise
        out_h = extents["h"]
        strips = sorted(set(_divisor_like(out_h, [1, 2, 4, 7, 8, 14, 16, 28, 32, 56, 64, 112]) + [out_h]))
        # 0 = no staging: the register-tiled 3x3 kernel or the window kernel, whichever takes the shape
        space.add_subspace("tile_h", KnobSpace("tile_h", [0] + [s for s in strips if s <= out_h]), "spatial")
        space.add_subspace("threads", KnobSpace("threads", [64, 128, 256, 512]), "spatial")
    return space


def generate_space_intra_op(op, down_graph, slevel=4, rlevel=3, groups=3, split_policy="off",
                            unroll_policy="off", fuse_policy="fuse_spatial", reorder_policy="last",
                            target="cuda"):
    """Per-op space; ``target`` selects the B200 knob space ("cuda") or the reference's
    loop-split space ("llvm")."""
    if target == "cuda":
        return generate_space_intra_op_b200(op, down_graph)
    return generate_space_intra_op_llvm(op, down_graph, slevel=slevel, rlevel=rlevel, groups=groups,
                                        split_policy=split_policy, unroll_policy=unroll_policy,
                                        fuse_policy=fuse_policy, reorder_policy=reorder_policy)


def generate_space_inter_op(op_lst, down_graph, force_inline=False, force_merge=False, special_space=None):
    """Graph-level space: the inline choice per op plus the task's special sub-spaces."""
    space = Space()
    space.add_subspace("inline", generate_inline_space(op_lst, down_graph, force_inline=force_inline), "inline")
    for key, sub in (special_space or {}).items():
        space.add_subspace(key, sub, "special")
    return space
