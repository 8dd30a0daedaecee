"""A minimal tensor-expression IR standing where ``tvm.te`` stood for the reference.

The reference builds its operators as ``tvm.te.compute`` lambdas; the search only ever
reads a handful of attributes from them (flextensor/space.py:399-402,
flextensor/scheduler.py:36-55,983-988): ``op.axis[i].var.name``,
``op.axis[i].dom.extent.value``, ``op.reduce_axis``, ``op.input_tensors``,
``op.num_outputs``, ``op.output(i)`` and ``tensor.shape/.dtype/.op``.  The classes
below expose exactly those, and add what the B200 backend needs to pick a kernel:
``ComputeOp.kind`` and ``ComputeOp.attrs``.
"""
from collections import namedtuple

_Var = namedtuple("_Var", ("name",))


class _Imm(object):
    """An integer literal with the ``.value`` accessor TVM's IntImm has."""

    __slots__ = ("value",)

    def __init__(self, value):
        self.value = int(value)

    def __int__(self):
        return self.value

    def __index__(self):
        return self.value

    def __eq__(self, other):
        return self.value == int(other)

    def __hash__(self):
        return hash(self.value)

    def __repr__(self):
        return str(self.value)


_Range = namedtuple("_Range", ("min", "extent"))


class IterVar(object):
    """A loop axis: ``.var.name`` and ``.dom.extent.value``."""

    def __init__(self, name, extent, kind="spatial"):
        self.var = _Var(name)
        self.dom = _Range(_Imm(0), _Imm(extent))
        self.kind = kind

    def __repr__(self):
        return "IterVar(%s, 0..%d, %s)" % (self.var.name, self.dom.extent.value, self.kind)


def reduce_axis(dom, name="rv"):
    lo, hi = dom
    assert int(lo) == 0
    return IterVar(name, int(hi), "reduce")


class Tensor(object):
    def __init__(self, shape, dtype, op, value_index=0, name=None):
        self.shape = tuple(_Imm(s) for s in shape)
        self.dtype = dtype
        self.op = op
        self.value_index = value_index
        self.name = name or (op.name if op is not None else "tensor")

    @property
    def ndim(self):
        return len(self.shape)

    def __repr__(self):
        return "Tensor(%s, %s, %s)" % (self.name, tuple(int(s) for s in self.shape), self.dtype)

    # identity semantics: tensors are dict keys in the graph walk
    __hash__ = object.__hash__

    def __eq__(self, other):
        return self is other


class Operation(object):
    num_outputs = 1

    def __init__(self, name):
        self.name = name
        self._outputs = []

    def output(self, i):
        return self._outputs[i]

    @property
    def input_tensors(self):
        return []


class PlaceholderOp(Operation):
    def __init__(self, shape, dtype, name):
        super().__init__(name)
        self._outputs = [Tensor(shape, dtype, self, 0, name)]


class ComputeOp(Operation):
    """One stage of the graph.

    kind  : 'pad2d' | 'gemm' | 'batch_gemm' | 'gemm_int8' | 'conv2d' | 'depthwise_conv2d' |
            'bias_add'
    attrs : kind-specific parameters (stride, padding, transposes, ...)
    axis / reduce_axis : loop axes with the names and extents the reference's lambdas have
    """

    def __init__(self, kind, name, out_shape, dtype, inputs, axis_names, reduce_axes=(), attrs=None):
        super().__init__(name)
        self.kind = kind
        self.attrs = dict(attrs or {})
        self._inputs = list(inputs)
        assert len(axis_names) == len(out_shape)
        self.axis = [IterVar(n, int(e)) for n, e in zip(axis_names, out_shape)]
        self.reduce_axis = list(reduce_axes)
        self._outputs = [Tensor(out_shape, dtype, self, 0, name)]

    @property
    def input_tensors(self):
        return list(self._inputs)

    def __repr__(self):
        return "ComputeOp(%s:%s)" % (self.kind, self.name)


_counter = [0]


def placeholder(shape, dtype="float32", name=None):
    """Counterpart of ``tvm.te.placeholder`` (default dtype float32, as in TVM)."""
    if name is None:
        _counter[0] += 1
        name = "placeholder%d" % _counter[0]
    return PlaceholderOp(tuple(int(s) for s in shape), dtype, name).output(0)
