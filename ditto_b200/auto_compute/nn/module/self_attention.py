"""Modules that wrap the fused chains (`ditto.auto_compute.nn.module`)."""
from .... import te
from ...graph import LayerTensor, layer
from ..functional import BatchGemmSoftmaxGemmMMA

MUTI_HEAD_ATTENTION_LAYER = "multi_head_attention_mma_layer"
SELF_ATTENTION_MODULE_REG = {MUTI_HEAD_ATTENTION_LAYER}


def is_self_attention_layer(lay):
    """Dispatch predicate of the reference's task binding
    (python/ditto/auto_compute/nn/module/self_attention.py:11-12)."""
    return lay.name in SELF_ATTENTION_MODULE_REG


class MultiHeadAttentionMMA:
    """Multi-head attention over a packed [batch, M, 3 * hidden] tensor
    (python/ditto/auto_compute/nn/module/self_attention.py:15-82): split into Q, K, V, fold the
    heads into the batch dimension ([batch * heads, M, d]; K pre-transposed to
    [batch * heads, d, M]), run the fused chain, unfold the heads again."""

    def __init__(self, num_heads, hidden_size, in_dtype="float16", acc_dtype="float32", mma_MI=16, mma_NI=16,
                 mma_KI=16):
        assert hidden_size % num_heads == 0
        self.num_heads, self.hidden_size = num_heads, hidden_size
        self.model_k = hidden_size // num_heads
        self.in_dtype, self.acc_dtype = in_dtype, acc_dtype
        self.MI, self.NI, self.KI = mma_MI, mma_NI, mma_KI

    def __call__(self, query_key_value: LayerTensor):
        return self.forward(query_key_value)

    def forward(self, query_key_value: LayerTensor):
        batch, M, K3 = query_key_value.shape
        if K3 != 3 * self.hidden_size:
            raise RuntimeError("Can't prove the self attention inputs conform to the hidden size.")
        bh, d = batch * self.num_heads, self.model_k
        src = query_key_value.tensor
        q = te.compute([bh, M, d], [src], "query_mh", self.in_dtype)
        k = te.compute([bh, d, M], [src], "key_mh", self.in_dtype)
        v = te.compute([bh, M, d], [src], "value_mh", self.in_dtype)
        out_mh = BatchGemmSoftmaxGemmMMA(q, k, v, MI=self.MI, NI=self.NI, KI=self.KI, in_dtype=self.in_dtype,
                                         acc_dtype=self.acc_dtype)
        outputs = te.compute([batch, M, self.hidden_size], [out_mh], "outputs", self.in_dtype)
        attention_layer = layer(outputs.op, inputs=[src], weights=[], name=MUTI_HEAD_ATTENTION_LAYER)
        attention_layer.attention_attrs = {"num_heads": self.num_heads, "head_dim": d}
        return attention_layer(query_key_value)
