"""Seeded sweeps over random shapes of every fused entry point, against float32 PyTorch products of the same
(rounded) inputs.  The fixed-shape parity tests pin the reference's configurations and the corner cases someone
thought of; this file walks the supported shape space -- row counts that are and are not multiples of the
128-row block, any K in steps of 16, hidden sizes in steps of 64, result widths in steps of 256 (several column
groups above 1024), one to thousands of work items (work loops with uneven item counts), both weight / key
layouts, both 16-bit types -- so that a shape-dependent indexing or phase error somewhere else shows up.
Tolerances: relative 2e-2 (fp16) / 3e-2 (bf16) plus a floor scaled by the largest result."""
import random

import pytest
import torch

from ditto_b200 import ops

pytestmark = pytest.mark.gpu


def _assert_close(out, ref, dtype, what, cuda):
    tol = 2e-2 if dtype == torch.float16 else 3e-2
    err = (out.float() - ref).abs()
    bound = tol * ref.abs() + (2e-3 if dtype == torch.float16 else 8e-3) * max(1.0, ref.abs().max().item())
    assert ops.device_status(cuda) == 0, what
    assert not torch.isnan(out).any(), what
    assert bool((err <= bound).all()), (what, err.max().item())


def _act(v, name):
    if name == "relu":
        return torch.relu(v)
    if name == "gelu":     # the reference's tanh form (nn/functional/activation.py:29-39)
        return 0.5 * v * (1 + torch.tanh(0.7978845608 * v * (1 + 0.044715 * v * v)))
    return v


def test_random_mlp_chains(cuda):
    rnd = random.Random(11)
    g = torch.Generator(device=cuda).manual_seed(12)
    for _ in range(60):
        dtype = rnd.choice([torch.float16, torch.bfloat16])
        layout = rnd.choice(["IO", "OI"])
        N = 256 * rnd.choice([1, 1, 2, 3, 4, 4, 5, 6, 8])
        K = 16 * rnd.randint(1, 40)
        L = 64 * rnd.randint(1, 40)
        batch = rnd.choice([1, 1, 1, 2, 3])
        M = 16 * rnd.randint(1, rnd.choice([8, 40, 300, 700]))
        act = rnd.choice(["relu", "identity"])
        ws = rnd.choice(["auto", None])
        x = torch.randn(batch, M, K, device=cuda, generator=g).to(dtype)
        w1 = (torch.randn(batch, K, L, device=cuda, generator=g) * K ** -0.5).to(dtype)
        w2 = (torch.randn(batch, L, N, device=cuda, generator=g) * L ** -0.5).to(dtype)
        a1, a2 = (w1.transpose(1, 2).contiguous(), w2.transpose(1, 2).contiguous()) if layout == "OI" else (w1, w2)
        out = torch.full((batch, M, N), float("nan"), dtype=dtype, device=cuda)
        ops.gemm_relu_gemm(x, a1, a2, out=out, activation=act, weight_layout=layout, workspace=ws)
        ref = _act(x.float() @ w1.float(), act).to(dtype).float() @ w2.float()
        _assert_close(out, ref, dtype, ("mlp", batch, M, N, K, L, str(dtype), layout, act, ws), cuda)


def test_random_feed_forward_blocks(cuda):
    rnd = random.Random(13)
    g = torch.Generator(device=cuda).manual_seed(14)
    for _ in range(60):
        dtype = rnd.choice([torch.float16, torch.bfloat16])
        layout = rnd.choice(["IO", "OI"])
        N = 256 * rnd.choice([1, 2, 4, 5])
        K = 16 * rnd.randint(1, 24)
        L = 64 * rnd.randint(1, 24)
        M = 16 * rnd.randint(1, rnd.choice([8, 100, 400]))
        acts = rnd.choice([("relu", "relu"), ("gelu", "identity"), ("relu", "identity"), ("identity", "gelu"), ("gelu", "gelu")])
        x = torch.randn(1, M, K, device=cuda, generator=g).to(dtype)
        w1 = (torch.randn(1, K, L, device=cuda, generator=g) * K ** -0.5).to(dtype)
        w2 = (torch.randn(1, L, N, device=cuda, generator=g) * L ** -0.5).to(dtype)
        b1 = (torch.randn(1, L, device=cuda, generator=g) * 0.5).to(dtype) if rnd.random() < 0.8 else None
        b2 = (torch.randn(1, N, device=cuda, generator=g) * 0.5).to(dtype) if rnd.random() < 0.8 else None
        a1, a2 = (w1.transpose(1, 2).contiguous(), w2.transpose(1, 2).contiguous()) if layout == "OI" else (w1, w2)
        out = torch.full((1, M, N), float("nan"), dtype=dtype, device=cuda)
        ops.ffn(x, a1, b1, a2, b2, out=out, act1=acts[0], act2=acts[1], weight_layout=layout)
        h = x.float() @ w1.float()
        if b1 is not None:
            h = h + b1.float()[:, None, :]
        y = _act(h, acts[0]).to(dtype).float() @ w2.float()
        if b2 is not None:
            y = y + b2.float()[:, None, :]
        _assert_close(out, _act(y, acts[1]), dtype, ("ffn", M, N, K, L, str(dtype), layout, acts, b1 is not None, b2 is not None), cuda)


def test_random_attention(cuda):
    rnd = random.Random(15)
    g = torch.Generator(device=cuda).manual_seed(16)
    for _ in range(80):
        dtype = rnd.choice([torch.float16, torch.bfloat16])
        d = 16 * rnd.randint(1, 8)
        dv = rnd.choice([d, d, 16 * rnd.randint(1, 8)])
        M = 16 * rnd.randint(1, 70)
        L = 16 * rnd.randint(1, rnd.choice([8, 40, 140]))
        b = rnd.choice([1, 3, 20, 150, 400])
        if b * M * L * 4 > 1.5e9:
            continue
        layout = rnd.choice(["LK", "KL"])
        q = (torch.rand(b, M, d, device=cuda, generator=g) - 0.5).to(dtype)
        k = (torch.rand(b, L, d, device=cuda, generator=g) - 0.5).to(dtype)
        v = (torch.rand(b, L, dv, device=cuda, generator=g) - 0.5).to(dtype)
        kk = k.transpose(1, 2).contiguous() if layout == "KL" else k
        out = torch.full((b, M, dv), float("nan"), dtype=dtype, device=cuda)
        scale = rnd.choice([1.0, d ** -0.5])
        ops.bmm_softmax_bmm(q, kk, v, out=out, scale=scale, key_layout=layout)
        ref = torch.softmax(q.float() @ k.float().transpose(1, 2) * scale, -1) @ v.float()
        _assert_close(out, ref, dtype, ("attention", b, M, L, d, dv, str(dtype), layout, scale), cuda)


def test_random_small_chains(cuda):
    rnd = random.Random(17)
    g = torch.Generator(device=cuda).manual_seed(18)
    dtype = torch.float16
    for _ in range(80):
        N, K = 16 * rnd.randint(1, 8), 16 * rnd.randint(1, 8)
        L = 16 * rnd.randint(1, 70)
        M = 16 * rnd.randint(1, 40)
        batch = rnd.choice([1, 4, 60, 200])
        layout = rnd.choice(["IO", "OI"])
        act = rnd.choice(["relu", "identity"])
        a = (torch.rand(batch, M, K, device=cuda, generator=g) * 2 - 1).to(dtype)
        b = (torch.rand(batch, K, L, device=cuda, generator=g) * 2 - 1).to(dtype)
        c = (torch.rand(batch, L, N, device=cuda, generator=g) * 2 - 1).to(dtype)
        a1, a2 = (b.transpose(1, 2).contiguous(), c.transpose(1, 2).contiguous()) if layout == "OI" else (b, c)
        out = torch.full((batch, M, N), float("nan"), dtype=dtype, device=cuda)
        ops.gemm_relu_gemm(a, a1, a2, out=out, activation=act, weight_layout=layout)
        ref = _act(a.float() @ b.float(), act).to(dtype).float() @ c.float()
        _assert_close(out, ref, dtype, ("small chain", batch, M, N, K, L, layout, act), cuda)
