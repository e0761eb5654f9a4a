"""kch_b200 — B200 (sm_100a) kernels for the forward path of the KDA + CSA + HCA hybrid attention stack
of 183600/kda-csa-hca-fusion, behind the reference's operator interface.

    from kch_b200 import naive_chunk_kda, naive_recurrent_kda, naive_csa, naive_hca
    from kch_b200 import CSADecodingCache, HCADecodingCache, HybridConfig, HybridKCHAttention

All compute runs in hand-written CUDA kernels reached through the C ABI of ``libkch_b200.so``
(``include/kch_b200.h``); there is no Triton, no FLA dispatch and no CPU fallback.
"""
from .kda import kda_forward, naive_chunk_kda, naive_recurrent_kda, validate_kda_backend  # noqa: F401
from .csa import (csa_compress_kv, csa_compress_kv_overlapped, csa_lightning_indexer,  # noqa: F401
                  naive_csa)
from .hca import naive_hca  # noqa: F401
from .decoding_cache import CSADecodingCache, HCADecodingCache  # noqa: F401
from .fused import (CSAHybridLayer, HCAHybridLayer, HybridConfig, HybridDecoding,  # noqa: F401
                    HybridKCHAttention, KDAHybridLayer)
from .backend import install, uninstall  # noqa: F401
from .host_pipeline import HostPipeline  # noqa: F401
from .decoding_modules import CSAAttnDecoding, HCAAttnDecoding, KDAAttnDecoding  # noqa: F401

__all__ = ["HostPipeline", "CSAAttnDecoding", "HCAAttnDecoding", "KDAAttnDecoding", "kda_forward", "naive_chunk_kda", "naive_recurrent_kda", "validate_kda_backend", "csa_compress_kv",
           "csa_compress_kv_overlapped", "csa_lightning_indexer", "naive_csa", "naive_hca", "CSADecodingCache",
           "HCADecodingCache", "HybridConfig", "HybridKCHAttention", "HybridDecoding", "KDAHybridLayer",
           "CSAHybridLayer", "HCAHybridLayer", "install", "uninstall"]
