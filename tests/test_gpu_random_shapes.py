"""Seeded sweep over random shapes the reference's asserts allow (multiples of 16, bmm_chain.py:34-38):
every fused entry point against a float32 torch evaluation of the same rounded inputs, outputs
poison-filled first, status word checked after every call."""
import random

import pytest
import torch

from ditto_b200 import _lib, ops

pytestmark = pytest.mark.gpu


def _check(name, got, ref, dtype, cuda):
    tol, floor = (2e-2, 1e-3) if dtype == torch.float16 else (3e-2, 4e-3)   # the tolerances of tests/tolerances.py
    assert ops.device_status(cuda) == 0, name
    assert not torch.isnan(got).any(), name
    err = (got.float() - ref).abs()
    assert bool((err <= tol * ref.abs() + floor).all()), (name, err.max().item())


def test_attention_random_shapes(cuda):
    rng = random.Random(20240)
    g = torch.Generator(device=cuda).manual_seed(7)
    for _ in range(48):
        dtype = rng.choice([torch.float16, torch.bfloat16])
        b, M, L, d = rng.randint(1, 5), 16 * rng.randint(1, 70), 16 * rng.randint(1, 70), 16 * rng.randint(1, 8)
        layout = rng.choice(["LK", "KL"])
        flags = rng.choice([0, 0, 0, _lib.FLAG_ONE_TILE, _lib.FLAG_TWO_TILES])
        q, k, v = ((torch.rand(b, n, d, device=cuda, generator=g) - 0.5).to(dtype) for n in (M, L, L))
        key = k.transpose(1, 2).contiguous() if layout == "KL" else k
        out = torch.full((b, M, d), float("nan"), device=cuda, dtype=dtype)
        ops.bmm_softmax_bmm(q, key, v, out=out, scale=1.0, key_layout=layout, flags=flags)
        ref = torch.softmax(q.float() @ k.float().transpose(1, 2), -1) @ v.float()
        _check(f"attention {dtype} {layout} flags={flags} {(b, M, L, d)}", out, ref, dtype, cuda)


def test_mlp_random_shapes(cuda):
    rng = random.Random(20241)
    g = torch.Generator(device=cuda).manual_seed(8)
    for _ in range(24):
        dtype = rng.choice([torch.float16, torch.bfloat16])
        b, M, K, L = rng.randint(1, 2), 16 * rng.randint(1, 40), 64 * rng.randint(1, 8), 128 * rng.randint(1, 16)
        N = rng.choice([256, 512, 768, 1024])
        layout, act = rng.choice(["IO", "OI"]), rng.choice(["relu", "identity"])
        x = torch.randn(b, M, K, device=cuda, generator=g).to(dtype)
        w1 = (torch.randn(b, K, L, device=cuda, generator=g) * K ** -0.5).to(dtype)
        w2 = (torch.randn(b, L, N, device=cuda, generator=g) * L ** -0.5).to(dtype)
        a1, a2 = (w1, w2) if layout == "IO" else (w1.transpose(1, 2).contiguous(), w2.transpose(1, 2).contiguous())
        out = torch.full((b, M, N), float("nan"), device=cuda, dtype=dtype)
        ops.gemm_relu_gemm(x, a1, a2, out=out, activation=act, weight_layout=layout)
        h = x.float() @ w1.float()
        h = torch.relu(h) if act == "relu" else h
        ref = h.to(dtype).float() @ w2.float()       # hidden activations rounded to the input type, as the kernel does
        _check(f"mlp {dtype} {layout} {act} {(b, M, N, K, L)}", out, ref, dtype, cuda)


def test_small_n_chain_and_packed_heads_random_shapes(cuda):
    rng = random.Random(20242)
    g = torch.Generator(device=cuda).manual_seed(9)
    for _ in range(16):
        dtype = rng.choice([torch.float16, torch.bfloat16])
        b, M, L, d = rng.randint(1, 4), 16 * rng.randint(1, 40), 16 * rng.randint(1, 40), 16 * rng.randint(1, 8)
        act = rng.choice(["relu", "identity"])
        x, w1, w2 = ((torch.rand(*s, device=cuda, generator=g) - 0.5).to(dtype) for s in ((b, M, d), (b, d, L), (b, L, d)))
        out = torch.full((b, M, d), float("nan"), device=cuda, dtype=dtype)
        ops.gemm_relu_gemm(x, w1, w2, out=out, activation=act)
        h = x.float() @ w1.float()
        h = torch.relu(h) if act == "relu" else h
        _check(f"small-N chain {dtype} {act} {(b, M, d, L)}", out, h.to(dtype).float() @ w2.float(), dtype, cuda)
    for _ in range(12):
        dtype = rng.choice([torch.float16, torch.bfloat16])
        b, M, heads, d = rng.randint(1, 3), 16 * rng.randint(1, 40), rng.randint(1, 6), 16 * rng.randint(1, 8)
        hidden = heads * d
        qkv = (torch.rand(b, M, 3 * hidden, device=cuda, generator=g) - 0.5).to(dtype)
        out = ops.multi_head_attention(qkv, heads, scale=1.0)
        qq, kk, vv = (qkv[..., i * hidden:(i + 1) * hidden].reshape(b, M, heads, d).permute(0, 2, 1, 3).float() for i in range(3))
        ref = (torch.softmax(qq @ kk.transpose(-1, -2), -1) @ vv).permute(0, 2, 1, 3).reshape(b, M, hidden)
        _check(f"packed heads {dtype} {(b, M, heads, d)}", out, ref, dtype, cuda)
