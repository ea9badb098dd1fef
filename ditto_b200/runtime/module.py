"""`build(schedule, tensors, "cuda")` -> callable module, standing in for `tvm.build`.

The reference calls the compiled chain as `func(*inputs, *outputs)` with every buffer
pre-allocated by the caller, and times it with `func.time_evaluator(func.entry_name, ctx,
min_repeat_ms=600)(*args).mean` (benchmark/chimera/cuda/bmm_softmax_bmm_cuda.py:23-42, 239-256).
ChainModule keeps that calling convention on torch CUDA tensors.
"""
from dataclasses import dataclass
from typing import List

import torch

from .. import ops
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
        if len(tensors) != 4:
            raise TypeError(f"{self.entry_name} takes 3 inputs and 1 output, got {len(tensors)} tensors")
        want = [(s.batch, s.M, s.K), (s.batch, s.K, s.L), (s.batch, s.L, s.N), (s.batch, s.M, s.N)]
        for t, shp, nm in zip(tensors, want, ("A", "B", "C", "F")):
            if tuple(t.shape) != shp:
                raise ValueError(f"{nm}: shape {tuple(t.shape)} does not match the compiled shape {shp}")
            if t.dtype != _TORCH_DTYPE[s.dtype]:
                raise TypeError(f"{nm}: dtype {t.dtype} does not match the compiled dtype {s.dtype}")

    def __call__(self, *tensors):
        self._check(tensors)
        s = self.schedule
        if s.kind == "mha":
            ops.multi_head_attention(tensors[0], s.heads, out=tensors[1], scale=s.scale)
            return
        a, b, c, f = tensors
        if s.kind == "softmax":
            ops.bmm_softmax_bmm(a, b, c, out=f, scale=s.scale, key_layout="KL")
        else:
            ops.gemm_relu_gemm(a, b, c, out=f, activation="relu" if s.kind == "relu" else "identity")

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
