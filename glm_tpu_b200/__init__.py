"""glm_tpu_b200: a Blackwell (B200, sm_100a) inference engine for the GLM-5.3 FP8 mixture-of-experts model.

Layering (imports only go downward):

    entrypoints -> executor -> worker -> engine -> runner -> models -> layers -> ops (CUDA) / parallel
    config, utils, envs, exceptions are leaves and import neither torch nor CUDA.
"""

__version__ = "0.1.0"
