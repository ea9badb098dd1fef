"""`build(schedule, tensors, "cuda")` -> callable module, standing in for `tvm.build`.

The reference calls the compiled chain as `func(*inputs, *outputs)` with every buffer
pre-allocated by the caller, and times it with `func.time_evaluator(func.entry_name, ctx,
min_repeat_ms=600)(*args).mean` (benchmark/chimera/cuda/bmm_softmax_bmm_cuda.py:23-42, 239-256).
ChainModule keeps that calling convention on torch CUDA tensors.
"""
import weakref
from dataclasses import dataclass
from typing import List

import torch

from .. import _lib, ops
from ..auto_tensorize import ChainSchedule

_TORCH_DTYPE = {"float16": torch.float16, "bfloat16": torch.bfloat16}


@dataclass
class TimeResult:
    mean: float          # seconds
    results: List[float]


class ChainModule:
    entry_name = "default_function"

    def __init__(self, sch: ChainSchedule, name="default_function"):
        self.schedule = sch
        self.entry_name = name
        self._fast = None

    def _check(self, tensors):
        s = self.schedule
        if s.kind == "mha":
            if len(tensors) != 2:
                raise TypeError(f"{self.entry_name} takes 1 input and 1 output, got {len(tensors)} tensors")
            want = [(s.batch, s.M, 3 * s.N), (s.batch, s.M, s.N)]
            for t, shp, nm in zip(tensors, want, ("qkv", "out")):
                if tuple(t.shape) != shp:
                    raise ValueError(f"{nm}: shape {tuple(t.shape)} does not match the compiled shape {shp}")
                if t.dtype != _TORCH_DTYPE[s.dtype]:
                    raise TypeError(f"{nm}: dtype {t.dtype} does not match the compiled dtype {s.dtype}")
            return
        if s.kind == "ffn":
            names, want = self._ffn_signature()
            if len(tensors) != len(want):
                raise TypeError(f"{self.entry_name} takes {', '.join(names)}: {len(want)} tensors, got {len(tensors)}")
            for t, shp, nm in zip(tensors, want, names):
                if shp is not None and tuple(t.shape) != shp:
                    raise ValueError(f"{nm}: shape {tuple(t.shape)} does not match the compiled shape {shp}")
                if t.dtype != _TORCH_DTYPE[s.dtype]:
                    raise TypeError(f"{nm}: dtype {t.dtype} does not match the compiled dtype {s.dtype}")
            for t, nm in ((tensors[0], "x"), (tensors[-1], "out")):
                if t.numel() != s.M * (s.K if nm == "x" else s.N):
                    raise ValueError(f"{nm}: {t.numel()} elements do not match the compiled {s.M} rows")
            return
        if len(tensors) != 4:
            raise TypeError(f"{self.entry_name} takes 3 inputs and 1 output, got {len(tensors)} tensors")
        want = [(s.batch, s.M, s.K), (s.batch, s.K, s.L), (s.batch, s.L, s.N), (s.batch, s.M, s.N)]
        for t, shp, nm in zip(tensors, want, ("A", "B", "C", "F")):
            if tuple(t.shape) != shp:
                raise ValueError(f"{nm}: shape {tuple(t.shape)} does not match the compiled shape {shp}")
            if t.dtype != _TORCH_DTYPE[s.dtype]:
                raise TypeError(f"{nm}: dtype {t.dtype} does not match the compiled dtype {s.dtype}")

    def _ffn_signature(self):
        """Argument names and shapes of a feed-forward module, in the layer's schedule_tensors order: the input,
        the weights ([out, in] matrices, each followed by its bias if it has one), the output.  x and out keep
        whatever leading dimensions the layer tensors have (None: only their sizes are checked)."""
        s = self.schedule
        names, shapes = ["x", "w1"], [None, (s.L, s.K)]
        if s.bias1:
            names.append("b1"); shapes.append((s.L,))
        names.append("w2"); shapes.append((s.N, s.L))
        if s.bias2:
            names.append("b2"); shapes.append((s.N,))
        names.append("out"); shapes.append(None)
        return names, shapes

    def _call_ffn(self, tensors):
        s = self.schedule
        args = dict(zip(self._ffn_signature()[0], tensors))
        ops.ffn(args["x"].reshape(s.M, s.K), args["w1"], args.get("b1"), args["w2"], args.get("b2"),
                out=args["out"].view(s.M, s.N), act1=s.act1, act2=s.act2, weight_layout="OI")

    def __call__(self, *tensors):
        # Shapes, dtypes and the argument order are fixed at build time, as in the reference, so a call
        # with the same tensor objects as the previous one (a benchmark loop, an inference engine with
        # pre-allocated buffers; held by weak reference) needs no re-validation: it fetches the current pointers and the current
        # stream and goes straight to the C ABI.  Anything else takes the checked path below once.
        fast = self._fast
        # (identity alone is not enough: resize_ / set_ / transpose_ change a tensor's metadata in place, and the
        # kernels address the compiled extent whatever the buffer holds -- so shape, dtype and layout are compared too)
        if fast is not None and len(tensors) == len(fast[0]) and all(
                r() is t and t.shape == shp and t.dtype == dt and t.is_contiguous()
                for r, (shp, dt), t in zip(fast[0], fast[5], tensors)):
            fn, head, tail, dev_index = fast[1:5]
            if torch.cuda.current_device() == dev_index:
                rc = fn(*[t.data_ptr() for t in tensors], *head, *tail, torch.cuda.current_stream().cuda_stream)
                if rc != 0:
                    _lib.check(rc, self.entry_name)
                ops.launch_count += 1
                return
        self._check(tensors)
        s = self.schedule
        if s.kind == "mha":
            ops.multi_head_attention(tensors[0], s.heads, out=tensors[1], scale=s.scale)
        elif s.kind == "ffn":
            self._call_ffn(tensors)
            return                      # no prepared fast path: ops.ffn is the checked path every time
        else:
            a, b, c, f = tensors
            if s.kind == "softmax":
                ops.bmm_softmax_bmm(a, b, c, out=f, scale=s.scale, key_layout="KL")
            else:
                ops.gemm_relu_gemm(a, b, c, out=f, activation="relu" if s.kind == "relu" else "identity")
        self._fast = self._prepare(tensors)

    def _prepare(self, tensors):
        """Arguments of the C entry point that do not change between calls with these tensor objects
        (everything but the data pointers and the stream), or None where the checked path must stay."""
        s = self.schedule
        if not all(t.is_cuda and t.is_contiguous() for t in tensors):
            return None
        dev = tensors[0].device
        if any(t.device != dev for t in tensors):
            return None
        lib = _lib.load()
        code = ops._DTYPE_CODE[_TORCH_DTYPE[s.dtype]]
        if s.kind == "softmax":
            fn = lib.ditto_b200_bmm_softmax_bmm
            head = (s.batch, s.M, s.N, s.K, s.L, code, 0, float(s.scale), 0, None, 0)
        elif s.kind == "mha":
            fn = lib.ditto_b200_multi_head_attention
            head = (s.batch, s.M, s.heads, s.N // s.heads, code, float(s.scale), 0)
        else:
            fn = lib.ditto_b200_gemm_relu_gemm
            head = (s.batch, s.M, s.N, s.K, s.L, code, 0, 1 if s.kind == "relu" else 0, None, 0)
        tail = (ops._status_word(dev).data_ptr(),)
        return (tuple(weakref.ref(t) for t in tensors), fn, head, tail,
                dev.index if dev.index is not None else torch.cuda.current_device(),
                tuple((t.shape, t.dtype) for t in tensors))

    def get_function(self, name):
        if name != self.entry_name:
            raise AttributeError(f"module has no function {name!r}")
        return self

    def time_evaluator(self, func_name=None, ctx=None, number=10, repeat=1, min_repeat_ms=0):
        """Mean seconds per call, measured with CUDA events on the current stream."""
        def evaluator(*tensors):
            self._check(tensors)
            self(*tensors)  # warm-up
            torch.cuda.synchronize()
            results = []
            for _ in range(repeat):
                n = number
                while True:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(n):
                        self(*tensors)
                    e1.record()
                    e1.synchronize()
                    ms = e0.elapsed_time(e1)
                    if ms >= min_repeat_ms or n >= (1 << 20):
                        break
                    n = max(n * 2, int(n * min_repeat_ms / max(ms, 1e-3)) + 1)
                results.append(ms / n / 1e3)
            return TimeResult(sum(results) / len(results), results)
        return evaluator


def build(sch, args=None, target="cuda", name="default_function"):
    """Turn the result of `auto_tensorize.tensorize_cuda` into a launchable module."""
    if not isinstance(sch, ChainSchedule):
        raise TypeError("build() expects the schedule returned by auto_tensorize.tensorize_cuda")
    if target != "cuda":
        raise ValueError("only the 'cuda' target exists on this path (no CPU fallback)")
    if args is not None and list(args) != sch.layer.schedule_tensors:
        raise ValueError("args must be layer.schedule_tensors (inputs, weights, outputs in that order)")
    return ChainModule(sch, name)
