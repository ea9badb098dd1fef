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


def _mix64(torch, k):
    """murmur3's 64-bit finaliser on int64 tensors (multiplication wraps; shifts are made logical by masking)."""
    k = k ^ ((k >> 33) & 0x7FFFFFFF)
    k = k * -49064778989728563          # 0xff51afd7ed558ccd
    k = k ^ ((k >> 33) & 0x7FFFFFFF)
    k = k * -4265267296055464877        # 0xc4ceb9fe1a85ec53
    return k ^ ((k >> 33) & 0x7FFFFFFF)


def _device_units(torch, w, seeds, elems, device, std=1.0):
    """[len(seeds), elems] values in the storage type: unit u depends only on seeds[u] (a counter-based
    generator: value j of a unit = hash(seed, j) -> Box-Muller), so it is the same whichever units are drawn
    beside it.  A few element-wise launches per call, whatever the number of units."""
    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[w.dtype]
    base = torch.tensor([_mix64_int(s) for s in seeds], dtype=torch.int64, device=device).reshape(-1, 1)
    k = _mix64(torch, base + torch.arange(elems, dtype=torch.int64, device=device).reshape(1, -1))
    u1 = (((k >> 40) & 0xFFFFFF).to(torch.float32) + 0.5) * (1.0 / (1 << 24))
    u2 = (((k >> 16) & 0xFFFFFF).to(torch.float32) + 0.5) * (1.0 / (1 << 24))
    del k
    if w.dist == "uniform":
        return (u1 * 2 - 1).to(tdt)
    u1.log_().mul_(-2.0).sqrt_()
    u2.mul_(6.283185307179586).cos_()
    return u1.mul_(u2).mul_(std).to(tdt)


def _mix64_int(x):
    """The same finaliser on a Python int (wrapping to signed 64 bit), for the per-unit seeds."""
    m = (1 << 64) - 1
    x &= m
    x ^= x >> 33
    x = (x * 0xff51afd7ed558ccd) & m
    x ^= x >> 33
    x = (x * 0xc4ceb9fe1a85ec53) & m
    x ^= x >> 33
    return x - (1 << 64) if x >= (1 << 63) else x


def device_attention_inputs(w: Workload, lo: int, hi: int, device, units_per_call=512):
    """Q [n, M, K], K [n, L, K], V [n, L, N] of slices [lo, hi) as device tensors in the storage type."""
    import torch
    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[w.dtype]
    n = hi - lo
    out = []
    for t, (rows, cols) in enumerate(((w.M, w.K), (w.L, w.K), (w.L, w.N))):
        x = torch.empty(n, rows, cols, dtype=tdt, device=device)
        for a in range(lo, hi, units_per_call):
            b = min(a + units_per_call, hi)
            seeds = [device_seed(w, i, t) for i in range(a, b)]
            x[a - lo:b - lo] = _device_units(torch, w, seeds, rows * cols, device).reshape(b - a, rows, cols)
        out.append(x)
    return tuple(out)


def device_mlp_inputs(w: Workload, lo: int, hi: int, device):
    """X rows of 128-row blocks [lo, hi) as a device tensor [(hi - lo) * 128, K]."""
    import torch
    seeds = [device_seed(w, b, 0) for b in range(lo, hi)]
    if not seeds:
        tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[w.dtype]
        return torch.empty(0, w.K, dtype=tdt, device=device)
    return _device_units(torch, w, seeds, 128 * w.K, device).reshape((hi - lo) * 128, w.K)


def device_mlp_weights(w: Workload, device):
    """W1 [K, L] ~ N(0, 1/K), W2 [L, N] ~ N(0, 1/L): the same on every rank."""
    import torch
    w1 = _device_units(torch, w, [device_seed(w, 0, 5)], w.K * w.L, device, w.K ** -0.5).reshape(w.K, w.L)
    w2 = _device_units(torch, w, [device_seed(w, 0, 6)], w.L * w.N, device, w.L ** -0.5).reshape(w.L, w.N)
    return w1, w2
