"""winnow_b200: the TurboQuant packed-KV decode path of lgoyal6/winnow
(turboquant_kv/) on hand-written sm_100a CUDA kernels behind a C ABI.

Modules keep the reference's names: packing, cache, page_pool,
packed_attention, packed_attention_cuda (in place of packed_attention_triton),
packed_backend, dispatch.  Every operator needs CUDA tensors and the built
libwinnow_tq.so; nothing falls back to the CPU.
"""
__version__ = "0.1.0"
