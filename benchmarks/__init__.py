"""Micro-benchmarks of single kernels and fused paths (run from the repository root: ``python -m benchmarks.<name>``)."""
