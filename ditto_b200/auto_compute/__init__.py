"""Op / graph construction for the fused-chain path (`ditto.auto_compute`)."""
from .graph import Graph, Layer, LayerTensor, graph, layer, layer_tensor
from . import nn
