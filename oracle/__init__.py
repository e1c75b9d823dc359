"""CPU checker for the CUDA path (test infrastructure, never the product)."""
