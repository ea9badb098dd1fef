"""A minimal symbolic tensor-expression layer.

The reference describes a chain as a TVM `te` compute DAG and inspects it through
`tensor.op`, `op.input_tensors`, `op.axis`, `op.reduce_axis` and `op.name`
(benchmark/chimera/cuda/bmm_softmax_bmm_cuda.py:169-182).  TVM is not a dependency here, so the
chain builders in `auto_compute.nn.functional` produce the same graph shape out of these light
objects: they carry names, shapes, dtypes and iteration variables, but no expression bodies --
the arithmetic of every supported chain is fixed by its kernel.
"""
from dataclasses import dataclass, field
from typing import List, Tuple

_DTYPES = ("float16", "bfloat16", "float32")


@dataclass(eq=False)
class IterVar:
    name: str
    extent: int
    kind: str = "spatial"  # or "reduce"

    @property
    def dom(self):
        return (0, self.extent)

    def __repr__(self):
        return f"iter_var({self.name}, range(min=0, ext={self.extent}))"


@dataclass(eq=False)
class Operation:
    name: str
    shape: Tuple[int, ...]
    dtype: str
    input_tensors: List["Tensor"] = field(default_factory=list)
    axis: List[IterVar] = field(default_factory=list)
    reduce_axis: List[IterVar] = field(default_factory=list)
    # role of the op inside a chain: "placeholder", "view" (tiling reshape / cast),
    # "cubic" (GEMM-like contraction), "exp", "relu", "pad_ones", "normalize", "identity"
    tag: str = "view"
    attrs: dict = field(default_factory=dict)

    def output(self, idx=0):
        assert idx == 0
        return Tensor(self)

    def __hash__(self):
        return id(self)

    def __eq__(self, other):
        return self is other

    def __repr__(self):
        return f"{'placeholder' if self.tag == 'placeholder' else 'compute'}({self.name}, {self.shape}, {self.dtype})"


class PlaceholderOp(Operation):
    pass


class ComputeOp(Operation):
    pass


class Tensor:
    """A value in the DAG; two Tensors of the same op compare equal."""

    def __init__(self, op: Operation):
        self.op = op

    @property
    def shape(self):
        return self.op.shape

    @property
    def dtype(self):
        return self.op.dtype

    @property
    def name(self):
        return self.op.name

    def __hash__(self):
        return hash(self.op)

    def __eq__(self, other):
        return isinstance(other, Tensor) and other.op is self.op

    def __repr__(self):
        return f"Tensor(shape={list(self.shape)}, op.name={self.op.name})"


def placeholder(shape, name="placeholder", dtype="float32") -> Tensor:
    if dtype not in _DTYPES:
        raise ValueError(f"dtype {dtype!r} not supported; expected one of {_DTYPES}")
    return Tensor(PlaceholderOp(name, tuple(int(s) for s in shape), dtype, tag="placeholder"))


def compute(shape, inputs, name, dtype, tag="view", axis_names=None, reduce=None, attrs=None) -> Tensor:
    shape = tuple(int(s) for s in shape)
    names = axis_names or [f"ax{i}" for i in range(len(shape))]
    axis = [IterVar(n, e) for n, e in zip(names, shape)]
    raxis = [IterVar(n, e, "reduce") for n, e in (reduce or [])]
    return Tensor(ComputeOp(name, shape, dtype, list(inputs), axis, raxis, tag, dict(attrs or {})))


def reduce_axis(dom, name="rv") -> IterVar:
    lo, hi = dom
    return IterVar(name, int(hi) - int(lo), "reduce")


def all_ops(outputs: List[Operation]) -> List[Operation]:
    """Post-order (producers first) list of every op reachable from `outputs`."""
    seen, order = set(), []

    def visit(op):
        if id(op) in seen:
            return
        seen.add(id(op))
        for t in op.input_tensors:
            visit(t.op)
        order.append(op)

    for op in outputs:
        visit(op)
    return order
