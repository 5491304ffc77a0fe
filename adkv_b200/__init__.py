"""adkv_b200: the ADKV KV-cache hot path (quantise/append, dequantise-and-attend decode) for B200 (sm_100a).

``gemv``      reference-compatible entry points (``encode_kv``, ``forward_qk``, ``forward_ov``) and the fused,
              checkpointed, variable-length and allocation-free decode steps, over the C ABI of libadkv_b200.so
``cache``     per-layer cache object mirroring the reference's ``KVCacheLayer_ADKV``
``hf_shim``   registers ``gemv`` under the reference's module name
``sharding``  batch x KV-head placement over the GPUs of a node
``synth``     seeded synthetic inputs of the benchmark configurations
``e2e_llama`` random-init Llama-architecture decode harness (tensor-parallel, CUDA-graph replay)
``build``     nvcc build of the shared library
"""
__version__ = "0.1.0"
