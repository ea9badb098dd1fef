"""Modules of the fused-chain path (`ditto.auto_compute.nn.module`)."""
from .act_module import GELU, ReLU, is_act_layer
from .linear_module import Linear
from .module import Module, Parameter
from .self_attention import MultiHeadAttentionMMA, is_self_attention_layer
