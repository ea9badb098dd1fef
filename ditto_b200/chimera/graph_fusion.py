"""Layer fusion at graph level (`ditto.chimera.graph_fusion`, python/ditto/chimera/graph_fusion.py).

The reference folds an activation layer into the layer that feeds it, so that `linear -> ReLU` is
scheduled as one layer.  The sm_100a path has a kernel for the whole feed-forward block, so the pattern
recognised here is one step longer:

    linear_layer -> relu_layer | gelu_layer -> linear_layer [-> relu_layer | gelu_layer]

(weights [out, in], optional biases; nn/model/transformer.py:21-34) becomes one "ffn_layer" whose hidden
activations never leave the chip.  Everything else in the graph is left as it is.
"""
from ..auto_compute.graph import Graph, LayerTensor, layer
from ..auto_compute.nn import functional as F
from ..auto_compute.nn.module.act_module import GELU_LAYER, RELU_LAYER, is_act_layer
from ..auto_compute.nn.module.linear_module import LINEAR_LAYER

FFN_LAYER = "ffn_layer"
_ACT_OF = {RELU_LAYER: "relu", GELU_LAYER: "gelu"}
_ACT_FN = {"relu": F.ReLU, "gelu": F.GELU}


def is_ffn_layer(lay):
    return lay.name == FFN_LAYER


def _consumers(layers, graph_outputs):
    """id(producing layer) -> number of uses of its output (by other layers or as a graph output)."""
    uses = {}
    for lay in layers:
        for lt in getattr(lay, "input_layer_tensors", []):
            if lt.layer is not None:
                uses[id(lt.layer)] = uses.get(id(lt.layer), 0) + 1
    for lt in graph_outputs:
        if lt.layer is not None:
            uses[id(lt.layer)] = uses.get(id(lt.layer), 0) + 1
    return uses


def _single_input_producer(lay):
    ins = getattr(lay, "input_layer_tensors", [])
    return ins[0].layer if len(ins) == 1 else None


def _match_ffn(last, uses):
    """The chain of layers ending in `last` if it is linear -> act -> linear [-> act], else None.
    Intermediate results must have no other consumer."""
    chain = [last]
    cur = last
    if is_act_layer(cur):
        cur = _single_input_producer(cur)
        if cur is None or uses.get(id(cur), 0) != 1:
            return None
        chain.append(cur)
    if cur.name != LINEAR_LAYER:
        return None
    act1 = _single_input_producer(cur)
    if act1 is None or not is_act_layer(act1) or uses.get(id(act1), 0) != 1:
        return None
    lin1 = _single_input_producer(act1)
    if lin1 is None or lin1.name != LINEAR_LAYER or uses.get(id(lin1), 0) != 1:
        return None
    chain += [act1, lin1]
    return list(reversed(chain))     # [lin1, act1, lin2] or [lin1, act1, lin2, act2]


def _fuse_ffn(chain):
    """One layer computing act2(act1(x W1^T + b1) W2^T + b2) from the layers of `chain`."""
    lin1, act1, lin2 = chain[:3]
    act2 = chain[3] if len(chain) == 4 else None
    (x,) = lin1.inputs
    w1, b1 = lin1.weights[0], (lin1.weights[1] if len(lin1.weights) > 1 else None)
    w2, b2 = lin2.weights[0], (lin2.weights[1] if len(lin2.weights) > 1 else None)
    a1 = _ACT_OF[act1.name]
    a2 = _ACT_OF[act2.name] if act2 is not None else "identity"
    out_dtype = lin2.ops[0].dtype
    h = _ACT_FN[a1](F.linear(x, w1, b1, out_dtype=lin1.ops[0].dtype))
    y = F.linear(h, w2, b2, out_dtype=out_dtype)
    if act2 is not None:
        y = _ACT_FN[a2](y)
    weights = [t for t in (w1, b1, w2, b2) if t is not None]
    fused = layer(y.op, inputs=[x], weights=weights, name=FFN_LAYER)
    fused.ffn_attrs = {"act1": a1, "act2": a2, "bias1": b1 is not None, "bias2": b2 is not None}
    return fused


def graph_fusion(graph):
    """Returns a graph in which every feed-forward pattern is one layer.  The input graph is not modified
    except that consumers of a fused pattern now read the fused layer's output."""
    layers = graph.all_layers
    uses = _consumers(layers, graph.graph_outputs)
    replaced = {}                       # id(old last layer) -> LayerTensor of the fused layer
    # longest patterns first: a trailing activation belongs to the block in front of it
    for last in sorted(layers, key=lambda l: 0 if is_act_layer(l) else 1):
        if any(id(l) in replaced for l in [last]):
            continue
        chain = _match_ffn(last, uses)
        if chain is None or any(getattr(l, "_fused_into", None) is not None for l in chain):
            continue
        fused = _fuse_ffn(chain)
        out = fused(*chain[0].input_layer_tensors)
        for l in chain:
            l._fused_into = fused
        replaced[id(last)] = out

    def rewire(lt):
        return replaced.get(id(lt.layer), lt) if isinstance(lt, LayerTensor) and lt.layer is not None else lt

    for lay in layers:
        if getattr(lay, "_fused_into", None) is None and hasattr(lay, "input_layer_tensors"):
            lay.input_layer_tensors = [rewire(lt) for lt in lay.input_layer_tensors]
    for fused_out in replaced.values():
        lay = fused_out.layer
        lay.input_layer_tensors = [rewire(lt) for lt in lay.input_layer_tensors]
    for l in layers:                     # the marks were only needed while matching
        if hasattr(l, "_fused_into"):
            del l._fused_into
    return Graph(graph.name, graph.graph_inputs, [rewire(lt) for lt in graph.graph_outputs])
