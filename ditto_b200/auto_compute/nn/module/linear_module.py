"""Linear module (python/ditto/auto_compute/nn/module/linear_module.py): weight [out_features, in_features],
optional bias [out_features], one "linear_layer" per call."""
from ...graph import layer
from ..functional import linear
from .module import Module, Parameter

LINEAR_LAYER = "linear_layer"


class Linear(Module):
    def __init__(self, in_features, out_features, bias=False, dtype="float32", out_dtype="float32"):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = Parameter([out_features, in_features], dtype=dtype, name="linear_weight")
        self.bias = Parameter([out_features], dtype=out_dtype, name="linear_bias") if bias else None
        self.dtype, self.out_dtype = dtype, out_dtype

    def forward(self, inputs):
        src = self.preprocess(inputs)
        weights = [self.weight.tensor] + ([self.bias.tensor] if self.bias is not None else [])
        outputs = linear(src.tensor, *weights, out_dtype=self.out_dtype)
        linear_layer = layer(outputs.op, inputs=[src.tensor], weights=weights, requires_grad=self.training,
                             name=LINEAR_LAYER)
        return linear_layer(inputs)
