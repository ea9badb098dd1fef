"""Op library of the fused-chain path (`ditto.auto_compute.nn.functional`): the chain builders and the
un-fused ops a caller composes them from (activation, linear, softmax)."""
from .activation import GELU, ReLU
from .bmm_chain import BatchGemmGemm, BatchGemmReluGemm, BatchGemmSoftmaxGemm, BatchGemmSoftmaxGemmMMA
from .linear import linear
from .softmax import softmax
