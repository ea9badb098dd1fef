"""The benchmark configurations of the fused-chain path and their seeded synthetic inputs.

Inputs are drawn with numpy from one seed per slice (attention) or per 128-row block (MLP rows)
and one seed per weight matrix, so a tensor is bit-identical whichever rank or GPU count
generates it and any shard can be regenerated on the CPU.  Values are drawn in fp32 and rounded
to the storage dtype; checkers receive the rounded values.
"""
from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class Workload:
    name: str
    kind: str        # "softmax" | "relu" | "identity"
    batch: int       # slices (attention) or 1 (MLP)
    M: int
    N: int
    K: int
    L: int
    dtype: str       # "float16" | "bfloat16" | "float32"
    scale: float
    dist: str        # "normal" | "uniform"
    cfg: int

    @property
    def flops(self):
        """Algorithmic FLOPs: 2 * MACs of the two GEMMs; softmax / ReLU are not credited."""
        return 2.0 * self.batch * self.M * self.L * (self.K + self.N)

    @property
    def bytes(self):
        """Algorithmic bytes: every input read once and the output written once."""
        esz = 4 if self.dtype == "float32" else 2
        per = self.M * self.K + self.K * self.L + self.L * self.N + self.M * self.N
        return float(self.batch * per * esz)

    @property
    def units(self):
        """Independent units the path shards over: slices for attention, 128-row blocks for the MLP."""
        return self.batch if self.kind == "softmax" else self.M // 128

    def shard(self, rank, world):
        """Contiguous range [lo, hi) of units owned by `rank`."""
        per = -(-self.units // world)
        lo = min(rank * per, self.units)
        return lo, min(lo + per, self.units)


WORKLOADS = {
    "cfg1": Workload("cfg1 bmm-bmm fp32 CPU case 8x512x64x64x512", "identity", 8, 512, 64, 64, 512, "float32", 1.0,
                     "uniform", 1),
    "cfg2": Workload("cfg2 attention fp16 12 slices S=512 d=64", "softmax", 12, 512, 64, 64, 512, "float16", 0.125,
                     "normal", 2),
    "cfg3": Workload("cfg3 attention fp16 512 slices S=512 d=64", "softmax", 512, 512, 64, 64, 512, "float16", 0.125,
                     "normal", 3),
    "cfg4": Workload("cfg4 MLP bf16 16384x1024 -> 4096 -> 1024", "relu", 1, 16384, 1024, 1024, 4096, "bfloat16", 1.0,
                     "normal", 4),
    "cfg5": Workload("cfg5 attention bf16 1024 slices S=2048 d=128", "softmax", 1024, 2048, 128, 128, 2048,
                     "bfloat16", 128 ** -0.5, "normal", 5),
}


def _round(x, dtype):
    if dtype == "float16":
        return x.astype(np.float16).astype(np.float32)
    if dtype == "bfloat16":
        u = x.view(np.uint32).astype(np.uint64)
        u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
        return u.astype(np.uint32).view(np.float32)
    return x


def _draw(seed, shape, dist, std=1.0):
    rng = np.random.default_rng(seed)
    if dist == "uniform":
        return rng.uniform(-1.0, 1.0, shape).astype(np.float32)
    if dist == "uniform_half":
        return rng.uniform(-0.5, 0.5, shape).astype(np.float32)
    return (rng.standard_normal(shape, dtype=np.float32) * np.float32(std)).astype(np.float32)


def attention_slice(w: Workload, index: int):
    """(Q [M, K], K [L, K], V [L, N]) of slice `index` as float32 arrays holding dtype-rounded values."""
    base = 1000 * w.cfg + index
    q = _round(_draw((base, 0), (w.M, w.K), w.dist), w.dtype)
    k = _round(_draw((base, 1), (w.L, w.K), w.dist), w.dtype)
    v = _round(_draw((base, 2), (w.L, w.N), w.dist), w.dtype)
    return q, k, v


def attention_inputs(w: Workload, lo: int, hi: int):
    """Stacked slices [lo, hi): Q [n, M, K], K [n, L, K], V [n, L, N]."""
    qs, ks, vs = zip(*(attention_slice(w, i) for i in range(lo, hi)))
    return np.stack(qs), np.stack(ks), np.stack(vs)


def mlp_rows(w: Workload, block: int):
    """Rows [128 * block, 128 * block + 128) of X."""
    return _round(_draw((1000 * w.cfg + block, 0), (128, w.K), w.dist), w.dtype)


def mlp_weights(w: Workload):
    """W1 [K, L] ~ N(0, 1/K), W2 [L, N] ~ N(0, 1/L) -- variance 1 / fan_in."""
    w1 = _round(_draw((1000 * w.cfg, 101), (w.K, w.L), w.dist, w.K ** -0.5), w.dtype)
    w2 = _round(_draw((1000 * w.cfg, 102), (w.L, w.N), w.dist, w.L ** -0.5), w.dtype)
    return w1, w2


def mlp_inputs(w: Workload, lo: int, hi: int):
    """X rows of blocks [lo, hi) stacked to [(hi - lo) * 128, K]."""
    return np.concatenate([mlp_rows(w, b) for b in range(lo, hi)], axis=0)


def chain_inputs(w: Workload):
    """(A [batch, M, K], B [batch, K, L], C [batch, L, N]) for the plain / ReLU chains at full size."""
    base = 1000 * w.cfg
    a = _round(_draw((base, 0), (w.batch, w.M, w.K), w.dist), w.dtype)
    b = _round(_draw((base, 1), (w.batch, w.K, w.L), w.dist), w.dtype)
    c = _round(_draw((base, 2), (w.batch, w.L, w.N), w.dist), w.dtype)
    return a, b, c


# ------------------------------------------------------------------ the same seeding, drawn on the GPU
# Config 5 holds 805 M input values; drawing them with numpy takes minutes.  The benchmark therefore draws
# its inputs on the device, with the same rule -- one seed per slice / per 128-row block / per weight
# matrix, `1000 * cfg + index` -- so that a unit's data does not depend on the number of GPUs or on which
# rank generates it.  (The values differ from the numpy ones above: another generator.  Parity tests use
# the numpy inputs; the benchmark checks its own inputs against the oracle after copying them back.)
def device_seed(w: Workload, index: int, tensor: int):
    return (1000 * w.cfg + index) * 8 + tensor


def _device_draw(torch, seed, shape, w, device, std=1.0):
    g = torch.Generator(device=device).manual_seed(seed)
    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[w.dtype]
    if w.dist == "uniform":
        return (torch.rand(*shape, device=device, generator=g) * 2 - 1).to(tdt)
    return (torch.randn(*shape, device=device, generator=g) * std).to(tdt)


def device_attention_inputs(w: Workload, lo: int, hi: int, device):
    """Q [n, M, K], K [n, L, K], V [n, L, N] of slices [lo, hi) as device tensors in the storage type."""
    import torch
    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[w.dtype]
    n = hi - lo
    q = torch.empty(n, w.M, w.K, dtype=tdt, device=device)
    k = torch.empty(n, w.L, w.K, dtype=tdt, device=device)
    v = torch.empty(n, w.L, w.N, dtype=tdt, device=device)
    for i in range(lo, hi):
        q[i - lo] = _device_draw(torch, device_seed(w, i, 0), (w.M, w.K), w, device)
        k[i - lo] = _device_draw(torch, device_seed(w, i, 1), (w.L, w.K), w, device)
        v[i - lo] = _device_draw(torch, device_seed(w, i, 2), (w.L, w.N), w, device)
    return q, k, v


def device_mlp_inputs(w: Workload, lo: int, hi: int, device):
    """X rows of 128-row blocks [lo, hi) as a device tensor [(hi - lo) * 128, K]."""
    import torch
    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[w.dtype]
    x = torch.empty((hi - lo) * 128, w.K, dtype=tdt, device=device)
    for b in range(lo, hi):
        x[(b - lo) * 128:(b - lo + 1) * 128] = _device_draw(torch, device_seed(w, b, 0), (128, w.K), w, device)
    return x


def device_mlp_weights(w: Workload, device):
    """W1 [K, L] ~ N(0, 1/K), W2 [L, N] ~ N(0, 1/L): the same on every rank."""
    import torch
    w1 = _device_draw(torch, device_seed(w, 0, 5), (w.K, w.L), w, device, w.K ** -0.5)
    w2 = _device_draw(torch, device_seed(w, 0, 6), (w.L, w.N), w, device, w.L ** -0.5)
    return w1, w2
