"""Layer-level operations of GLM-MoE-DSA as plain functions over tensors.

Every function states its numerical contract, runs the hand-written CUDA kernel when its operands live on a GPU and the CPU
restatement of the same contract (``glm_tpu_b200.oracle.contract``) otherwise, so the two are interchangeable in tests and in
user code.  The decode and prefill programs in ``models/glm_moe_dsa/model.py`` call the kernels directly (with preallocated
workspaces, fused collectives and a captured launch sequence); these functions are the single-op view of the same kernels.

Parity: reference ``glm_tpu/layers/`` (contracts, embed, norm, rope, linear, mlp, fp8, sampler, attention/*, moe/*).
"""
