"""GraphEngine: runs a graph's layers in order through their compiled modules
(src/runtime/graph_runtime.cc:14-247; CUDA-graph variant src/runtime/cuda_graph_runtime.cc:13-81).

Same protocol as the reference: `create_graph_engine(graph, built_mods, dev)` and then
`engine.get_function(name)` for name in init / set_inputs / set_weight / compile / run / timeit /
get_outputs.  Buffers are torch CUDA tensors; `built_mods` maps a layer fingerprint to the module
returned by `runtime.build`.
"""
import torch

_TORCH_DTYPE = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}


class TimeCost(float):
    """Milliseconds; a float that also answers `.value` like the reference's boxed result."""

    @property
    def value(self):
        return float(self)


class GraphEngine:
    def __init__(self, graph, built_mods, dev="cuda"):
        self.graph = graph
        self.built_mods = dict(built_mods)
        self.device = torch.device(dev if isinstance(dev, (str, torch.device)) else "cuda")
        self.buffers = {}
        self.calls = []
        self._functions = {
            "init": self.init, "set_inputs": self.set_inputs, "set_weight": self.set_weight,
            "compile": self.compile, "run": self.run, "timeit": self.timeit, "get_outputs": self.get_outputs,
        }

    def get_function(self, name):
        if name not in self._functions:
            raise AttributeError(f"GraphEngine has no function {name!r}")
        return self._functions[name]

    def _buffer(self, tensor):
        key = id(tensor.op)
        if key not in self.buffers:
            # the reference fills every buffer with U(-10, 10) (graph_runtime.cc:51-101)
            buf = torch.empty(tuple(tensor.shape), dtype=torch.float32, device=self.device).uniform_(-10, 10)
            self.buffers[key] = buf.to(_TORCH_DTYPE[tensor.dtype])
        return self.buffers[key]

    def init(self):
        for lay in self.graph.all_layers:
            for t in lay.schedule_tensors:
                self._buffer(t)
            # a layer's inputs alias the outputs of its producers
            for inp_lt, t in zip(getattr(lay, "input_layer_tensors", []), lay.inputs):
                if inp_lt.layer is not None:
                    self.buffers[id(t.op)] = self._buffer(inp_lt.tensor)

    def set_inputs(self, *arrays):
        for lt, arr in zip(self.graph.graph_inputs, arrays):
            self._buffer(lt.tensor).copy_(arr)

    def set_weight(self, layer, tensor, array):
        self._buffer(tensor).copy_(array)

    def compile(self):
        self.calls = []
        for lay in self.graph.all_layers:
            key = lay.fingerprint
            if key not in self.built_mods:
                raise KeyError(f"no built module for layer {lay.name!r} (fingerprint {key})")
            fn = self.built_mods[key].get_function("default_function")
            self.calls.append((fn, [self._buffer(t) for t in lay.schedule_tensors]))

    def run(self):
        for fn, args in self.calls:
            fn(*args)

    def timeit(self, repeat=10):
        """Mean milliseconds per run over `repeat` runs, after one warm-up, as an object whose `.value` is that
        number -- the reference's timeit returns a boxed float and callers read `ftimeit(600).value`
        (benchmark/chimera/cuda/bert_inference.py:128)."""
        self.run()
        torch.cuda.synchronize(self.device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(int(repeat)):
            self.run()
        e1.record()
        e1.synchronize()
        return TimeCost(e0.elapsed_time(e1) / int(repeat))

    def get_outputs(self):
        return [self._buffer(lt.tensor) for lt in self.graph.graph_outputs]


class CUDAGraphEngine(GraphEngine):
    """Captures one run into a CUDA graph at compile time and replays it."""

    def compile(self):
        super().compile()
        super().run()  # warm-up outside capture (sets kernel attributes)
        torch.cuda.synchronize(self.device)
        self._graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self._graph):
            GraphEngine.run(self)

    def run(self):
        self._graph.replay()


def create_graph_engine(graph, built_mods, dev="cuda"):
    return GraphEngine(graph, built_mods, dev)


def create_cuda_graph_engine(graph, built_mods, dev="cuda"):
    return CUDAGraphEngine(graph, built_mods, dev)
