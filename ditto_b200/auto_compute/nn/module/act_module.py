"""Activation modules (python/ditto/auto_compute/nn/module/act_module.py): one layer per activation, which
`chimera.graph_fusion` later folds into the chain that produces its input."""
from ...graph import layer
from ..functional import GELU as gelu
from ..functional import ReLU as relu
from .module import Module

RELU_LAYER = "relu_layer"
GELU_LAYER = "gelu_layer"
ACT_MODULE_REG = {RELU_LAYER, GELU_LAYER}


def is_act_layer(lay):
    return lay.name in ACT_MODULE_REG


class _Activation(Module):
    fn, layer_name = None, None

    def forward(self, inputs):
        src = self.preprocess(inputs)
        outputs = type(self).fn(src.tensor)
        act_layer = layer(outputs.op, inputs=[src.tensor], requires_grad=self.training, name=self.layer_name)
        return act_layer(inputs)


class ReLU(_Activation):
    fn, layer_name = staticmethod(relu), RELU_LAYER


class GELU(_Activation):
    fn, layer_name = staticmethod(gelu), GELU_LAYER
