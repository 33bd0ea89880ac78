"""B200-native decode hot path for AdvayMonga/inference-server.

The directory name contains a hyphen, so import it with
``importlib.import_module("inference-server_b200")``.  Sub-modules:

- ``_lib``      ctypes binding of ``libb200decode.so`` (the C-ABI in
                ``include/b200_decode.h``); fails loudly if the library is absent.
- ``ops``       operator wrappers on torch CUDA tensors (paged attention, KV
                append, MoE route/permute/quant/GEMM/combine).
- ``quant``     load-time e4m3 128x128 block quantisation of expert weights.
- ``backend``   ``B200Backend``: the reference ``InferenceBackend`` interface on
                block tables instead of dense caches.
"""

__all__ = ["_lib", "ops", "quant"]
