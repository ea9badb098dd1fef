"""Chain-fusion entry points (`ditto.auto_tensorize`) for the fused GEMM-chain path.

The reference searches a schedule for the two contractions and lowers it through TVM
(src/auto_tensorize/hyper_fusion.cc:609-1603).  Here the fusion decision is fixed -- both
contractions in one kernel, intermediate on chip -- so these functions validate the layer,
classify its ops exactly as the reference does, and hand the recognised chain to the sm_100a
kernels; tuning knobs are accepted so caller scripts run unchanged.
"""
from dataclasses import dataclass, field
from typing import Dict, List

from .. import te
from ..auto_compute.graph import Layer
from ..hardware import HardwareParam


class FusionError(ValueError):
    """The layer is not a chain the fused kernels cover (the reference's `validate`,
    src/auto_tensorize/api.cc:14-31, CHECK-fails on the same conditions)."""


# ------------------------------------------------------------------ intrinsics
@dataclass
class PackedIntrinsic:
    """Descriptor of the tensor-core tile (the reference packs WMMA load/mma/store intrinsics,
    python/ditto/auto_tensorize/intrinsic.py:24-48, 252-272; here it names the tcgen05 tile)."""
    M: int
    N: int
    K: int
    in_dtype: str
    out_dtype: str
    scope: str
    instruction: str = "tcgen05.mma.cta_group::1.kind::f16 (128 x N x 16, fp32 accumulate in TMEM)"


def cuda_wmma(M=16, N=16, K=16, in_dtype="float16", out_dtype="float32", scope="shared"):
    return PackedIntrinsic(M, N, K, in_dtype, out_dtype, scope)


def intrinsic_match(target: te.Tensor, packed: PackedIntrinsic, restrictions=None):
    """Axes of `target` that map onto the intrinsic's (m, n, k).  With the fixed chain templates
    the match is unique: the two innermost spatial axes and the innermost reduce axis
    (what src/auto_tensorize/intrin_match.cc:26-124 returns under InnerMost + SameRange)."""
    op = target.op
    if op.tag != "cubic":
        raise FusionError(f"{op.name} is not a GEMM-like op")
    mi, ni = op.axis[-2], op.axis[-1]
    ki = op.reduce_axis[-1]
    if (mi.extent, ni.extent, ki.extent) != (packed.M, packed.N, packed.K):
        return []
    return [[mi, ni, ki]]


@dataclass
class MatchInfo:
    axis: List[te.IterVar]
    intrin: PackedIntrinsic
    impl: str = ""


def match_info(axis, intrin, impl=""):
    return MatchInfo(list(axis), intrin, impl)


# ------------------------------------------------------------------ serial fusion state
@dataclass
class SerialFusionState:
    layer: Layer
    first_op: te.Operation
    second_op: te.Operation
    tensorize_axes: list = field(default_factory=list)

    def register_tensorize_axes(self, axes):
        self.tensorize_axes = list(axes)


def _cubic_ops(layer: Layer):
    return [op for op in layer.all_ops if op.tag == "cubic"]


def validate(layer: Layer):
    """One output, a tree-shaped producer graph, exactly two GEMM-like ops, the first feeding the
    second through element-wise ops only."""
    if len(layer.ops) != 1:
        raise FusionError("a fused chain has exactly one output op")
    cubic = _cubic_ops(layer)
    if len(cubic) != 2:
        raise FusionError(f"expected two GEMM-like ops in the layer, found {len(cubic)}")
    consumers: Dict[int, int] = {}
    for op in layer.all_ops:
        for t in op.input_tensors:
            consumers[id(t.op)] = consumers.get(id(t.op), 0) + 1
    for op in layer.all_ops:
        if op.tag != "placeholder" and consumers.get(id(op), 0) > 1:
            raise FusionError(f"{op.name} has more than one consumer; only linear chains are supported")
    first, second = cubic
    path, cur = [], second.input_tensors[0].op
    while cur is not first:
        if cur.tag in ("placeholder", "cubic") or len(cur.input_tensors) != 1:
            raise FusionError("the first GEMM does not feed the second one through element-wise ops")
        path.append(cur)
        cur = cur.input_tensors[0].op
    return first, second, list(reversed(path))


def build_serial_fusion_state(layer: Layer) -> SerialFusionState:
    first, second, _ = validate(layer)
    return SerialFusionState(layer, first, second)


# ------------------------------------------------------------------ fusion choice
@dataclass
class FusionChoice:
    first_op: te.Operation
    second_op: te.Operation
    ordered_iters: list
    attach_pos: int

    def __repr__(self):
        return f"FusionChoice(axis={self.ordered_iters}, pos={self.attach_pos})"


def fusion_choice(first_op, second_op, ordered_iters, attach_pos):
    return FusionChoice(first_op, second_op, list(ordered_iters), int(attach_pos))


def build_fusion_choice(sfs: SerialFusionState, hw_param=None, dtype="float16", simple_mode=-1):
    """The kernels use one fusion order: batch, row tile outermost, the shared L reduction next,
    tensor-core tile innermost -- the reference's [b, m, n, rlo | mi, ni, rli] with attach
    position 3 (benchmark/chimera/cuda/bmm_softmax_bmm_cuda.py:178-182).  No search is run."""
    op = sfs.second_op
    b, m, n, mi, ni = op.axis
    rlo, rli = op.reduce_axis
    return FusionChoice(sfs.first_op, op, [b, m, n, rlo, mi, ni, rli], 3)


# ------------------------------------------------------------------ hyper fusion state
@dataclass
class TensorizeHyperFusionState:
    """Partition of the layer's ops around the two contractions
    (src/auto_tensorize/hyper_fusion.cc:51-216)."""
    layer: Layer
    first_op: te.Operation
    second_op: te.Operation
    first_op_prologue: list
    second_op_prologue: list
    inter_path: list
    epilogue: list
    fuse_choice: FusionChoice
    tensorize_info: dict

    @property
    def chain_kind(self):
        tags = [op.tag for op in self.inter_path if op.tag != "view"]
        if tags == ["exp"]:
            return "softmax"
        if tags == ["relu"]:
            return "relu"
        if tags in ([], ["identity"]):
            return "identity"
        raise FusionError(f"unsupported ops between the two GEMMs: {tags}")

    def summary(self, verbose=False):
        fmt = lambda groups: " ".join("[" + " ".join(o.name for o in g) + "]" for g in groups)
        return "\n".join([
            "TensorizeHyperFusionState Summary:",
            f"First op: {self.first_op.name}", f"Second op: {self.second_op.name}",
            f"First op prologue: {fmt(self.first_op_prologue)}",
            f"Second op prologue: {fmt(self.second_op_prologue)}",
            "Inter Path: [" + " ".join(o.name for o in self.inter_path) + "]",
            "Epilogue: [" + " ".join(o.name for o in self.epilogue) + "]",
        ])


def _prologue(t: te.Tensor, stop):
    chain, cur = [], t.op
    while cur.tag != "placeholder" and cur is not stop:
        chain.append(cur)
        if len(cur.input_tensors) != 1:
            raise FusionError(f"prologue op {cur.name} must have one input")
        cur = cur.input_tensors[0].op
    return chain


def tensorize_hyper_fusion_state(layer: Layer, fuse_choice: FusionChoice, match_info: dict):
    first, second, inter = validate(layer)
    if fuse_choice.first_op is not first or fuse_choice.second_op is not second:
        raise FusionError("the fusion choice does not name the layer's two GEMM-like ops")
    for op in (first, second):
        if op not in match_info:
            raise FusionError(f"no tensorize match given for {op.name}")
    first_pro = [_prologue(t, None) for t in first.input_tensors]
    second_pro = [_prologue(t, first) for t in second.input_tensors[1:]]
    epilogue, cur = [], layer.ops[0]
    while cur is not second:
        epilogue.append(cur)
        cur = cur.input_tensors[0].op
    return TensorizeHyperFusionState(layer, first, second, first_pro, second_pro, inter, list(reversed(epilogue)),
                                     fuse_choice, dict(match_info))


# ------------------------------------------------------------------ tensorize
@dataclass
class CUDATensorizeParam:
    """The reference's thirteen tiling integers (include/auto_tensorize/hyper_fusion.h:365-442).
    The sm_100a kernels have fixed tiles (128-row query tiles, 128-row K/V blocks), so the values
    are recorded but do not change the generated code."""
    warp_size: int = 32
    ty_size: int = 4
    tz_size: int = 2
    input_vector_len: int = 4
    serial_y: int = 2
    serial_z: int = 1
    block_rx: int = 4
    block_ry: int = 1
    block_rz: int = 4
    warp_rx: int = 1
    warp_ry: int = 4
    warp_rz: int = 1
    unroll_steps: int = 1500

    def to_json(self):
        return dict(self.__dict__)


def cuda_tensorize_param(**kwargs):
    return CUDATensorizeParam(**kwargs)


@dataclass
class ChainSchedule:
    """What `tensorize_cuda` returns in place of a te.Schedule: the recognised chain, ready for
    `ditto_b200.build`."""
    layer: Layer
    kind: str          # "softmax" | "relu" | "identity" | "mha" | "ffn"
    batch: int
    M: int
    N: int
    K: int
    L: int
    dtype: str
    scale: float
    device: HardwareParam
    param: CUDATensorizeParam
    heads: int = 1     # "mha": heads folded into the packed [batch, M, 3 * heads * K] input
    act1: str = "identity"     # "ffn": activation after the first / second linear, and which biases exist
    act2: str = "identity"
    bias1: bool = False
    bias2: bool = False


def _schedule_self_attention(layer: Layer, cuda_param, tensorize_param) -> ChainSchedule:
    """The packed multi-head layer of nn/module/self_attention.py: one input [batch, M, 3 * hidden]."""
    first, second, inter = validate(layer)
    attrs = getattr(layer, "attention_attrs", None)
    if attrs is None or len(layer.inputs) != 1:
        raise FusionError("not a packed multi-head attention layer")
    (src,) = layer.inputs
    batch, M, k3 = src.shape
    heads, d = attrs["num_heads"], attrs["head_dim"]
    if k3 != 3 * heads * d:
        raise FusionError(f"packed input has {k3} columns, expected {3 * heads * d}")
    if src.dtype not in ("float16", "bfloat16"):
        raise FusionError(f"the sm_100a kernels take float16 or bfloat16 operands, got {src.dtype}")
    scale = 1.0
    for op in inter:
        scale = float(op.attrs.get("scale", scale))
    return ChainSchedule(layer, "mha", batch, M, heads * d, d, M, src.dtype, scale, cuda_param,
                         tensorize_param or CUDATensorizeParam(), heads)


def _schedule_ffn(layer: Layer, cuda_param, tensorize_param) -> ChainSchedule:
    """The feed-forward layer `chimera.graph_fusion` builds: x [..., K], W1 [L, K], (b1 [L]), W2 [N, L], (b2 [N]).
    The weights are shared by every row, so all leading dimensions of x fold into M (batch = 1)."""
    attrs = getattr(layer, "ffn_attrs", None)
    if attrs is None or len(layer.inputs) != 1:
        raise FusionError("not a feed-forward layer")
    (x,) = layer.inputs
    weights = list(layer.weights)
    w1 = weights.pop(0)
    b1 = weights.pop(0) if attrs["bias1"] else None
    w2 = weights.pop(0)
    b2 = weights.pop(0) if attrs["bias2"] else None
    if weights:
        raise FusionError("unexpected extra weights in a feed-forward layer")
    K = x.shape[-1]
    M = 1
    for e in x.shape[:-1]:
        M *= e
    L, N = w1.shape[0], w2.shape[0]
    if tuple(w1.shape) != (L, K) or tuple(w2.shape) != (N, L):
        raise FusionError(f"weights {tuple(w1.shape)}, {tuple(w2.shape)} do not chain with an input of {K} features")
    for bias, n in ((b1, L), (b2, N)):
        if bias is not None and tuple(bias.shape) != (n,):
            raise FusionError(f"bias of shape {tuple(bias.shape)}, expected {(n,)}")
    dtypes = {t.dtype for t in (x, w1, w2, b1, b2, layer.ops[0].output(0)) if t is not None}
    if len(dtypes) != 1 or x.dtype not in ("float16", "bfloat16"):
        raise FusionError(f"the sm_100a kernels take one 16-bit type for inputs, weights, biases and output, got {sorted(dtypes)}")
    for v, nm in ((M, "rows"), (N, "N"), (K, "K"), (L, "L")):
        if v % 16:
            raise FusionError(f"{nm}={v} must be a multiple of 16")
    return ChainSchedule(layer, "ffn", 1, M, N, K, L, x.dtype, 1.0, cuda_param, tensorize_param or CUDATensorizeParam(),
                         act1=attrs["act1"], act2=attrs["act2"], bias1=b1 is not None, bias2=b2 is not None)


def tensorize_cuda(layer: Layer, state: TensorizeHyperFusionState = None, cuda_param: HardwareParam = None,
                   tensorize_param: CUDATensorizeParam = None) -> ChainSchedule:
    if layer.name == "multi_head_attention_mma_layer":
        return _schedule_self_attention(layer, cuda_param, tensorize_param)
    if layer.name == "ffn_layer":
        return _schedule_ffn(layer, cuda_param, tensorize_param)
    if state is None:
        raise FusionError("tensorize_cuda needs the TensorizeHyperFusionState of the chain")
    kind = state.chain_kind
    A, B, C = (layer.schedule_tensors + [None] * 3)[:3]
    ph = [t for t in layer.schedule_tensors[:-1]]
    if len(ph) != 3:
        raise FusionError("a fused chain takes exactly three operands (A, B, C)")
    A, B, C = ph
    batch, M, K = A.shape
    L, N = C.shape[1], C.shape[2]
    if tuple(B.shape) != (batch, K, L):
        raise FusionError(f"second operand must be [batch, K, L] = {(batch, K, L)}, got {tuple(B.shape)}")
    dtype = A.dtype
    if dtype not in ("float16", "bfloat16"):
        raise FusionError(f"the sm_100a kernels take float16 or bfloat16 operands, got {dtype}")
    if state.first_op.dtype != "float32" or state.second_op.dtype != "float32":
        raise FusionError("accumulation is fp32 on this path (acc_dtype='float32')")
    scale = 1.0
    for op in state.inter_path:
        scale = float(op.attrs.get("scale", scale))
    return ChainSchedule(layer, kind, batch, M, N, K, L, dtype, scale, cuda_param,
                         tensorize_param or CUDATensorizeParam())
