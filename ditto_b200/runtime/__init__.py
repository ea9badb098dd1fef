"""Runtime module that launches compiled chains (`ditto.runtime` + the `tvm.build` result the
reference's callers use)."""
from .module import ChainModule, build
from .graph_engine import GraphEngine, create_cuda_graph_engine, create_graph_engine
