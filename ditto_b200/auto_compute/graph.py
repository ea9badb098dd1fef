"""Layer / LayerTensor / Graph containers (python/ditto/auto_compute/graph.py:8-274,
src/auto_compute/graph.cc:60-167) over the symbolic DAG of `ditto_b200.te`."""
import hashlib

from .. import te


class LayerTensor:
    """A tensor flowing between layers (graph.py:17-50 in the reference)."""

    def __init__(self, name, layer, tensor, value_idx=0):
        self.name, self.layer, self.tensor, self.value_idx = name, layer, tensor, value_idx

    @property
    def shape(self):
        return self.tensor.shape

    @property
    def dtype(self):
        return self.tensor.dtype

    def __repr__(self):
        return f"LayerTensor({self.name}, {list(self.shape)}, {self.dtype})"


def layer_tensor(shape, name="layer_tensor", dtype="float32", layer=None, idx=0):
    return LayerTensor(name, layer, te.placeholder(shape, name=name, dtype=dtype), idx)


class Layer:
    """A group of ops scheduled and launched as one unit."""

    def __init__(self, name, ops, inputs, weights, const_scalars, const_tensors):
        self.name = name
        self.ops = list(ops)
        self.inputs = list(inputs)
        self.weights = list(weights)
        self.const_scalars = list(const_scalars)
        self.const_tensors = list(const_tensors)
        declared = {t.op for t in (*self.inputs, *self.weights, *self.const_tensors)}
        for op in self.all_ops:
            if isinstance(op, te.PlaceholderOp) and op not in declared:
                raise ValueError(f"placeholder {op.name} is used by layer {name!r} but not declared as input/weight")

    def __call__(self, *inputs):
        if len(inputs) != self.num_inputs:
            raise ValueError(f"Need to provide {self.num_inputs} inputs, but get {len(inputs)}.")
        for inp in inputs:
            assert isinstance(inp, LayerTensor)
        self.input_layer_tensors = list(inputs)
        outs = [LayerTensor(op.name, self, op.output(0), i) for i, op in enumerate(self.ops)]
        return outs[0] if len(outs) == 1 else outs

    @property
    def all_ops(self):
        return te.all_ops(self.ops)

    @property
    def num_inputs(self):
        return len(self.inputs)

    @property
    def schedule_tensors(self):
        """Argument order of the compiled function: inputs, weights, const scalars, const tensors,
        outputs (graph.py:90-102 in the reference)."""
        return [*self.inputs, *self.weights, *self.const_scalars, *self.const_tensors,
                *[op.output(0) for op in self.ops]]

    @property
    def fingerprint(self):
        """Stable workload key: structure, shapes and dtypes, not object identity."""
        h = hashlib.sha1()
        for op in self.all_ops:
            h.update(f"{op.tag}|{op.shape}|{op.dtype}|{[t.op.tag for t in op.input_tensors]};".encode())
        return h.hexdigest()

    @property
    def gflops(self):
        """2 * MACs of the contraction ops, in GFLOP (src/auto_compute/graph.cc:86-130 counts the same ops)."""
        total = 0
        for op in self.all_ops:
            if op.tag == "cubic":
                n = 1
                for iv in (*op.axis, *op.reduce_axis):
                    n *= iv.extent
                total += 2 * n
        return total / 1e9

    @property
    def data_transfer_amount(self):
        """Bytes of every input, weight and output touched once."""
        size = {"float16": 2, "bfloat16": 2, "float32": 4}
        total = 0
        for t in (*self.inputs, *self.weights, *self.const_tensors, *[op.output(0) for op in self.ops]):
            n = 1
            for s in t.shape:
                n *= s
            total += n * size[t.dtype]
        return total

    def __repr__(self):
        lines = [f"====== Layer({self.name}) ======", f"{len(self.all_ops)} ops in this layer.", "inputs:"]
        lines += [repr(t) for t in self.inputs] + ["weights:"] + [repr(t) for t in self.weights]
        lines += ["ops: " + ", ".join(op.name for op in self.all_ops if op.tag != "placeholder")]
        return "\n".join(lines)


def layer(ops, inputs=None, weights=None, const_scalars=None, const_tensors=None, requires_grad=False,
          name="layer"):
    """Make a network layer from output operations (graph.py:136-203 in the reference)."""
    if not isinstance(ops, (list, tuple)):
        ops = [ops]
    unwrap = lambda xs: [x.tensor if isinstance(x, LayerTensor) else x for x in (xs or [])]
    return Layer(name, ops, unwrap(inputs), unwrap(weights), list(const_scalars or []), unwrap(const_tensors))


class Graph:
    """Inputs, outputs and the layers between them, in topological order
    (graph.py:205-274; src/auto_compute/graph.cc:300-454)."""

    def __init__(self, name, graph_inputs, graph_outputs):
        self.name = name
        self.graph_inputs = list(graph_inputs)
        self.graph_outputs = list(graph_outputs)

    @property
    def all_layers(self):
        seen, order = set(), []

        def visit(lt):
            lay = lt.layer
            if lay is None or id(lay) in seen:
                return
            seen.add(id(lay))
            for inp in getattr(lay, "input_layer_tensors", []):
                visit(inp)
            order.append(lay)

        for out in self.graph_outputs:
            visit(out)
        return order


def graph(graph_inputs, graph_outputs, name="graph"):
    return Graph(name, graph_inputs, graph_outputs)
