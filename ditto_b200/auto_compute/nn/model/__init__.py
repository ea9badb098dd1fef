"""Model pieces built from the fused-chain modules (`ditto.auto_compute.nn.model`)."""
from .transformer import PositionwiseFeedForward, TransformerBlock
