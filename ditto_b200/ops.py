"""Operators on torch CUDA tensors: thin argument marshalling over the C ABI.

PyTorch supplies device memory and the stream; all arithmetic happens in the hand-written
sm_100a kernels of libditto_b200.so.  There is no CPU path: tensors must live on a CUDA device.
"""
import torch

from . import _lib

_DTYPE_CODE = {torch.float16: _lib.DTYPE_FP16, torch.bfloat16: _lib.DTYPE_BF16}


class _NoGuard:
    def __enter__(self):
        return self

    def __exit__(self, *exc):
        return False


_NO_GUARD = _NoGuard()


def _on_device(device):
    """Context that makes `device` current for the launch; free when it already is (the common case)."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_GUARD
    return torch.cuda.device(device)
_status_words = {}

# number of kernel launches issued through this module (benchmarks report it)
launch_count = 0


_status_ptrs = {}


def _status_word(device):
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    if key not in _status_words:
        _status_words[key] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
    return _status_words[key]


def _status_ptr(device):
    """Device address of the status word of `device` (a torch.device), looked up once per device object."""
    p = _status_ptrs.get(device)
    if p is None:
        p = _status_ptrs[device] = _status_word(device).data_ptr()
    return p


def device_status(device=None, reset=True):
    """Synchronise and return the device-side status word (0 = no bounded wait has expired)."""
    dev = torch.device(device) if device is not None else torch.device("cuda", torch.cuda.current_device())
    w = _status_word(dev)
    torch.cuda.synchronize(dev)
    v = int(w.item())
    if reset and v:
        w.zero_()
    return v


def _check_tensor(t, name, dtype=None):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError(f"{name} must be a CUDA tensor (ditto_b200 has no CPU path)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous (compact row-major)")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} has dtype {t.dtype}, expected {dtype}")


def bmm_softmax_bmm(query, key, value, out=None, scale=1.0, key_layout="KL", flags=0):
    """out = softmax(scale * query @ key) @ value, fused in one kernel.

    query [batch, M, K]; key [batch, K, L] when key_layout == "KL" (the reference's layout,
    bmm_chain.py:30-31) or [batch, L, K] when "LK"; value [batch, L, N]; out [batch, M, N].
    scale = 1 gives the reference's exp / row-sum semantics.
    """
    global launch_count
    _check_tensor(query, "query")
    if query.dtype not in _DTYPE_CODE:
        raise TypeError(f"query dtype {query.dtype} not supported (float16 / bfloat16)")
    _check_tensor(key, "key", query.dtype)
    _check_tensor(value, "value", query.dtype)
    if query.dim() != 3 or key.dim() != 3 or value.dim() != 3:
        raise ValueError("query, key and value must be 3-D")
    batch, M, K = query.shape
    if key_layout == "KL":
        kb, kK, L = key.shape
        klay = 0
    elif key_layout == "LK":
        kb, L, kK = key.shape
        klay = 1
    else:
        raise ValueError("key_layout must be 'KL' or 'LK'")
    vb, vL, N = value.shape
    if not (kb == batch and vb == batch and kK == K and vL == L):
        raise ValueError(f"inconsistent shapes: {tuple(query.shape)}, {tuple(key.shape)} ({key_layout}), {tuple(value.shape)}")
    if out is None:
        out = torch.empty((batch, M, N), dtype=query.dtype, device=query.device)
    else:
        _check_tensor(out, "out", query.dtype)
        if tuple(out.shape) != (batch, M, N):
            raise ValueError(f"out has shape {tuple(out.shape)}, expected {(batch, M, N)}")
    lib = _lib.load()
    with _on_device(query.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.ditto_b200_bmm_softmax_bmm(query.data_ptr(), key.data_ptr(), value.data_ptr(), out.data_ptr(),
                                            batch, M, N, K, L, _DTYPE_CODE[query.dtype], klay, float(scale),
                                            int(flags), None, 0, _status_ptr(query.device), stream)
    _lib.check(rc, "ditto_b200_bmm_softmax_bmm")
    launch_count += 1
    return out


def multi_head_attention(qkv, num_heads, out=None, scale=1.0, flags=0):
    """Self-attention over a packed tensor: qkv [batch, M, 3 * hidden] = [Q | K | V] per row,
    hidden = num_heads * head_dim; returns [batch, M, hidden].  The head split / merge of
    nn/module/self_attention.py:46-73 is folded into the kernel's addressing (no reshape passes)."""
    global launch_count
    _check_tensor(qkv, "qkv")
    if qkv.dtype not in _DTYPE_CODE:
        raise TypeError(f"qkv dtype {qkv.dtype} not supported (float16 / bfloat16)")
    if qkv.dim() != 3 or qkv.shape[2] % (3 * num_heads):
        raise ValueError(f"qkv must be [batch, M, 3 * hidden] with hidden divisible by num_heads, got {tuple(qkv.shape)}")
    batch, M, k3 = qkv.shape
    hidden = k3 // 3
    if out is None:
        out = torch.empty((batch, M, hidden), dtype=qkv.dtype, device=qkv.device)
    else:
        _check_tensor(out, "out", qkv.dtype)
        if tuple(out.shape) != (batch, M, hidden):
            raise ValueError(f"out has shape {tuple(out.shape)}, expected {(batch, M, hidden)}")
    lib = _lib.load()
    with _on_device(qkv.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.ditto_b200_multi_head_attention(qkv.data_ptr(), out.data_ptr(), batch, M, num_heads, hidden // num_heads,
                                                 _DTYPE_CODE[qkv.dtype], float(scale), int(flags),
                                                 _status_ptr(qkv.device), stream)
    _lib.check(rc, "ditto_b200_multi_head_attention")
    launch_count += 1
    return out


_VARIANT_BITS = {"auto": 0, "pair": 0x200, "quad": 0x400, "wide": 0x800}
_workspaces = {}


def _workspace(device, nbytes):
    """A scratch buffer of at least `nbytes` on `device`, kept and grown per device (the C ABI itself
    allocates nothing: scratch memory is the caller's, and this module is that caller)."""
    key = device.index if device.index is not None else torch.cuda.current_device()
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = _workspaces[key] = torch.empty(nbytes, dtype=torch.uint8, device=f"cuda:{key}")
    return buf


def gemm_relu_gemm(x, w1, w2, out=None, activation="relu", weight_layout="IO", variant="auto", workspace="auto"):
    """out = act(x @ w1) @ w2 with the hidden activations kept on chip.

    x [batch, M, K] or [M, K]; w1 [batch, K, L] / [K, L]; w2 [batch, L, N] / [L, N] when
    weight_layout == "IO" ([in, out]); "OI" takes the transposed [out, in] weights of
    nn/functional/linear.py.  activation: "relu" or "identity".  variant: "auto" (by shape), "pair"
    (eight-CTA clusters of CTA pairs, 2-SM MMAs), "quad" (four-CTA clusters, 128-wide hidden chunks) or "wide"
    (four-CTA clusters, 256-wide hidden chunks).  workspace: "auto" (this
    module keeps a scratch buffer of ditto_b200_workspace_bytes() per device), None (no scratch: every row
    block is computed by one cluster) or a uint8 CUDA tensor.
    """
    global launch_count
    _check_tensor(x, "x")
    if x.dtype not in _DTYPE_CODE:
        raise TypeError(f"x dtype {x.dtype} not supported (float16 / bfloat16)")
    squeeze = x.dim() == 2
    x3 = x.unsqueeze(0) if squeeze else x
    w13 = w1.unsqueeze(0) if w1.dim() == 2 else w1
    w23 = w2.unsqueeze(0) if w2.dim() == 2 else w2
    _check_tensor(w13, "w1", x.dtype)
    _check_tensor(w23, "w2", x.dtype)
    batch, M, K = x3.shape
    if weight_layout == "IO":
        (b1, K1, L), (b2, L2, N) = w13.shape, w23.shape
        wl = 0
    elif weight_layout == "OI":
        (b1, L, K1), (b2, N, L2) = w13.shape, w23.shape
        wl = 1
    else:
        raise ValueError("weight_layout must be 'IO' or 'OI'")
    if not (b1 == batch and b2 == batch and K1 == K and L2 == L):
        raise ValueError(f"inconsistent shapes: {tuple(x.shape)}, {tuple(w1.shape)}, {tuple(w2.shape)}")
    if activation not in ("relu", "identity"):
        raise ValueError("activation must be 'relu' or 'identity'")
    if out is None:
        out = torch.empty((batch, M, N), dtype=x.dtype, device=x.device)
        out3 = out
        if squeeze:
            out = out[0]
    else:
        _check_tensor(out, "out", x.dtype)
        out3 = out.unsqueeze(0) if out.dim() == 2 else out
        if tuple(out3.shape) != (batch, M, N):
            raise ValueError(f"out has shape {tuple(out.shape)}, expected {(batch, M, N)}")
    if variant not in _VARIANT_BITS:
        raise ValueError(f"variant must be one of {sorted(_VARIANT_BITS)}")
    lib = _lib.load()
    with _on_device(x.device):
        ws_ptr, ws_bytes = None, 0
        if isinstance(workspace, torch.Tensor):
            _check_tensor(workspace, "workspace", torch.uint8)
            ws_ptr, ws_bytes = workspace.data_ptr(), workspace.numel()
        elif isinstance(workspace, str) and workspace == "auto":
            need = lib.ditto_b200_workspace_bytes(_lib.OP_GEMM_RELU_GEMM | _VARIANT_BITS[variant], batch, M, N, K, L,
                                                  _DTYPE_CODE[x.dtype])
            if need:
                buf = _workspace(x.device, need)
                ws_ptr, ws_bytes = buf.data_ptr(), buf.numel()
        elif workspace is not None:
            raise TypeError("workspace must be 'auto', None or a uint8 CUDA tensor")
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.ditto_b200_gemm_relu_gemm(x3.data_ptr(), w13.data_ptr(), w23.data_ptr(), out3.data_ptr(), batch, M, N,
                                           K, L, _DTYPE_CODE[x.dtype], wl,
                                           (1 if activation == "relu" else 0) | _VARIANT_BITS[variant], ws_ptr, ws_bytes,
                                           _status_ptr(x.device), stream)
    _lib.check(rc, "ditto_b200_gemm_relu_gemm")
    launch_count += 1
    return out


_ACT_CODE = {"identity": 0, "relu": 1, "gelu": 2}


def ffn(x, w1, b1, w2, b2, out=None, act1="relu", act2="relu", weight_layout="OI"):
    """Position-wise feed-forward block out = act2(act1(x @ W1 + b1) @ W2 + b2), hidden layer on chip.

    Defaults follow the reference's PositionwiseFeedForward (nn/model/transformer.py:21-34): weights
    stored [out, in] like nn/functional/linear.py, ReLU after both linears.  x [M, K] or [batch, M, K];
    w1 [L, K], w2 [N, L] ("OI") or [K, L], [L, N] ("IO"); b1 [L], b2 [N] or None."""
    global launch_count
    _check_tensor(x, "x")
    if x.dtype not in _DTYPE_CODE:
        raise TypeError(f"x dtype {x.dtype} not supported (float16 / bfloat16)")
    squeeze = x.dim() == 2
    x3 = x.unsqueeze(0) if squeeze else x
    w13 = w1.unsqueeze(0) if w1.dim() == 2 else w1
    w23 = w2.unsqueeze(0) if w2.dim() == 2 else w2
    _check_tensor(w13, "w1", x.dtype)
    _check_tensor(w23, "w2", x.dtype)
    batch, M, K = x3.shape
    if weight_layout == "OI":
        (_, L, K1), (_, N, L2) = w13.shape, w23.shape
    elif weight_layout == "IO":
        (_, K1, L), (_, L2, N) = w13.shape, w23.shape
    else:
        raise ValueError("weight_layout must be 'IO' or 'OI'")
    if K1 != K or L2 != L or w13.shape[0] != batch or w23.shape[0] != batch:
        raise ValueError(f"inconsistent shapes: {tuple(x.shape)}, {tuple(w1.shape)}, {tuple(w2.shape)}")
    for bias, n, nm in ((b1, L, "b1"), (b2, N, "b2")):
        if bias is not None:
            _check_tensor(bias, nm, x.dtype)
            if bias.numel() != batch * n:
                raise ValueError(f"{nm} must hold {batch * n} values, got {bias.numel()}")
    if act1 not in _ACT_CODE or act2 not in _ACT_CODE:
        raise ValueError(f"activations must be one of {sorted(_ACT_CODE)}")
    if out is None:
        out3 = torch.empty((batch, M, N), dtype=x.dtype, device=x.device)
        out = out3[0] if squeeze else out3
    else:
        _check_tensor(out, "out", x.dtype)
        out3 = out.unsqueeze(0) if out.dim() == 2 else out
        if tuple(out3.shape) != (batch, M, N):
            raise ValueError(f"out has shape {tuple(out.shape)}, expected {(batch, M, N)}")
    lib = _lib.load()
    with _on_device(x.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.ditto_b200_ffn(x3.data_ptr(), w13.data_ptr(), b1.data_ptr() if b1 is not None else None, w23.data_ptr(),
                                b2.data_ptr() if b2 is not None else None, out3.data_ptr(), batch, M, N, K, L,
                                _DTYPE_CODE[x.dtype], 1 if weight_layout == "OI" else 0, _ACT_CODE[act1], _ACT_CODE[act2],
                                _status_ptr(x.device), stream)
    _lib.check(rc, "ditto_b200_ffn")
    launch_count += 1
    return out
