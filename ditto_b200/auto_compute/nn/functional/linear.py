"""Linear op (python/ditto/auto_compute/nn/functional/linear.py:4-41)."""
from .... import te


def linear(inputs, weight, bias=None, out_dtype="float32"):
    """inputs [batch, ..., in_feature] x weight [out_feature, in_feature] (+ bias [out_feature]) ->
    [batch, ..., out_feature].  As in the reference the product and the bias add are two ops; the
    contraction carries the tag "linear" (a GEMM with a K-major weight), the add "bias_add"."""
    assert inputs.shape[-1] == weight.shape[1], f"in_feature {inputs.shape[-1]} != weight {weight.shape}"
    out_shape = (*inputs.shape[:-1], weight.shape[0])
    output = te.compute(out_shape, [inputs, weight], "linear", out_dtype, tag="linear",
                        reduce=[("k", inputs.shape[-1])])
    if bias is not None:
        assert bias.shape[0] == weight.shape[0], f"bias {bias.shape} does not match weight {weight.shape}"
        output = te.compute(out_shape, [output, bias], "linear_bias", out_dtype, tag="bias_add")
    return output
