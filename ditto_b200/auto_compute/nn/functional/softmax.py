"""Softmax op (python/ditto/auto_compute/nn/functional/softmax.py:4-35)."""
from .... import te


def softmax(x, dim=-1):
    """exp(x) / sum(exp(x)) along `dim`, without subtracting the maximum -- the reference's semantics, which
    the fused attention chain shares (there the same function is evaluated in the max-subtracted form).
    Two ops like the reference: "sum_val" (the row sums) and "softmax"."""
    assert -len(x.shape) <= dim < len(x.shape)
    dim = dim + len(x.shape) if dim < 0 else dim
    sum_shape = [e for i, e in enumerate(x.shape) if i != dim]
    sum_val = te.compute(sum_shape, [x], "sum_val", x.dtype, tag="exp_sum", reduce=[("r", x.shape[dim])],
                         attrs={"dim": dim})
    return te.compute(x.shape, [x, sum_val], "softmax", x.dtype, tag="softmax", attrs={"dim": dim})
