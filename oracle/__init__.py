"""CPU checker for the fused-group kernels (test infrastructure, not part of the product)."""
