"""CPU oracle of the quantized-matmul path: test infrastructure, never imported by the library."""
