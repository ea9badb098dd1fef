"""Graph-level glue (`ditto.chimera`): fuse layers into chains, bind tasks to schedulers."""
from .graph_fusion import FFN_LAYER, graph_fusion, is_ffn_layer
from .task_binding import task_binding
