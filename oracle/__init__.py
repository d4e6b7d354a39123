"""CPU oracle for the cast / quantise / quantised-GEMM path: test infrastructure only."""
