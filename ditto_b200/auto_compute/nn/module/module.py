"""Parameter / Module base classes (python/ditto/auto_compute/nn/module/module.py)."""
from .... import te
from ...graph import LayerTensor, layer_tensor


class Parameter:
    """A weight: a placeholder tensor the layer lists among its `weights`."""

    def __init__(self, shape, name="param", dtype="float32"):
        self.tensor = te.placeholder(shape, name=name, dtype=dtype)

    @property
    def shape(self):
        return self.tensor.shape

    @property
    def name(self):
        return self.tensor.name

    @property
    def dtype(self):
        return self.tensor.dtype


class Module:
    def __init__(self):
        self.training = True

    def forward(self, *args, **kwargs):
        raise NotImplementedError()

    def __call__(self, *args, **kwargs):
        return self.forward(*args, **kwargs)

    def _children(self):
        for v in self.__dict__.values():
            if isinstance(v, Module):
                yield v
            elif isinstance(v, (list, tuple)):
                yield from (e for e in v if isinstance(e, Module))

    def parameters(self):
        for v in self.__dict__.values():
            if isinstance(v, Parameter):
                yield v.tensor
        for child in self._children():
            yield from child.parameters()

    def eval(self):
        self.training = False
        for child in self._children():
            child.eval()

    def train(self):
        self.training = True
        for child in self._children():
            child.train()

    def preprocess(self, *inputs):
        """Fresh placeholders standing for the producing layers' outputs: every layer owns its input
        tensors, and the graph keeps the producer in `LayerTensor.layer` (module.py:89-103 in the reference)."""
        ret = []
        for inp in inputs:
            assert isinstance(inp, LayerTensor), type(inp)
            ret.append(layer_tensor(inp.shape, name=inp.name + "_out", dtype=inp.dtype, layer=inp.layer, idx=inp.value_idx))
        return ret[0] if len(ret) == 1 else ret
