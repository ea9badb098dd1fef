"""CPU oracle for the fused GEMM chains: test infrastructure, never on the product path."""
