"""The two fused-chain halves of the reference's transformer block
(python/ditto/auto_compute/nn/model/transformer.py:21-86)."""
from ..module import Linear, Module, MultiHeadAttentionMMA, ReLU


class PositionwiseFeedForward(Module):
    """activation(w_2(activation(w_1(x)))) with biased [out, in] linears and ReLU, as in the reference
    (transformer.py:21-34).  Built as four layers (linear, relu, linear, relu); `chimera.graph_fusion`
    turns them into one feed-forward layer that runs as a single kernel with the hidden layer on chip."""

    def __init__(self, d_model, d_ff, dtype="float32", out_dtype="float32"):
        super().__init__()
        self.w_1 = Linear(d_model, d_ff, bias=True, dtype=dtype, out_dtype=out_dtype)
        self.w_2 = Linear(d_ff, d_model, bias=True, dtype=dtype, out_dtype=out_dtype)
        self.activation = ReLU()

    def forward(self, x):
        return self.activation(self.w_2(self.activation(self.w_1(x))))


class TransformerBlock(Module):
    """Multi-head attention over a packed [batch, M, 3 * hidden] input followed by the feed-forward block.
    The reference's block (transformer.py:37-86) puts a bias-free Linear(hidden, 3 * hidden) in front of the
    attention; a single linear is not a GEMM chain and has no kernel on this path, so the block here starts
    at the packed query/key/value tensor that linear would produce."""

    def __init__(self, hidden, attn_heads, feed_forward_hidden, dtype="float16", mma_in_dtype="float16",
                 mma_acc_dtype="float32", mma_MI=16, mma_NI=16, mma_KI=16):
        super().__init__()
        self.attention = MultiHeadAttentionMMA(num_heads=attn_heads, hidden_size=hidden, in_dtype=mma_in_dtype,
                                               acc_dtype=mma_acc_dtype, mma_MI=mma_MI, mma_NI=mma_NI, mma_KI=mma_KI)
        self.feed_forward = PositionwiseFeedForward(d_model=hidden, d_ff=feed_forward_hidden, dtype=dtype, out_dtype=dtype)

    def forward(self, qkv):
        return self.feed_forward(self.attention(qkv))
