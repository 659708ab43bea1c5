"""forge — B200-native GPTQ / SparseGPT solver engine behind the 4Bit-Forge front end.

`from forge.gptq import GPTQ` and `from forge.backend.cuda import kernels` keep the reference's names
(forge/gptq.py, forge/backend/cuda/__init__.py); forge.moe adds the layer-level batched API.
"""
