"""Micro-benchmarks of the decode step and of single kernels (``python -m glm_tpu_b200.benchmarks.<name>``)."""
