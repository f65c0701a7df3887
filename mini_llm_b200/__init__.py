"""mini_llm_b200: a small, whole inference engine for one NVIDIA B200.

From a model folder (``config.json`` + ``model.safetensors``) to the next
token: typed configuration and registry, weights by tensor name, layers put
together from parts, a paged cache with block tables and state slots, one
step function for mixed batches, a scheduler, sampling, and hand-written CUDA
kernels for sm_100a.  There is no CPU path.
"""

__version__ = "0.1.0"
