"""Element-wise activations (python/ditto/auto_compute/nn/functional/activation.py:9-39)."""
from .... import te


def ReLU(x):
    """if_then_else(x > 0, x, 0), same shape and dtype as x; op name "ReLU" as in the reference."""
    return te.compute(x.shape, [x], "ReLU", x.dtype, tag="relu")


def GELU(x):
    """0.5 x (1 + tanh(0.7978845608 x (1 + 0.044715 x^2))): the reference's tanh form; op name "gelu"."""
    return te.compute(x.shape, [x], "gelu", x.dtype, tag="gelu")
