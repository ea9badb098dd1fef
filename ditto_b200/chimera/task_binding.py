"""Task binding (python/ditto/chimera/task_binding.py)."""
from collections import OrderedDict

from .. import auto_tensorize as at
from ..auto_compute.nn.module import is_self_attention_layer
from .graph_fusion import is_ffn_layer


def task_binding(tasks):
    """Assign a scheduler to each task (python/ditto/chimera/task_binding.py:6-20): self-attention
    layers, feed-forward layers and fused GEMM chains go to "chimera" (the sm_100a kernels); anything else would go to
    "ansor", which this path does not have -- such layers are listed there so the caller sees them."""
    ret = OrderedDict(chimera=OrderedDict(), ansor=OrderedDict())
    for key, layers in tasks.items():
        layer = layers[0]
        fused = is_self_attention_layer(layer) or is_ffn_layer(layer)
        if not fused:
            try:
                at.validate(layer)
                fused = True
            except at.FusionError:
                fused = False
        ret["chimera" if fused else "ansor"][key] = layers
    return ret
