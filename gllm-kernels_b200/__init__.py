"""gllm-kernels_b200 — B200 (sm_100a) quantized-matmul operators behind the reference's operator API.

Host-side mirror of the quant slice of gllm-kernels' `Kernels<E>` trait (src/traits.rs:473-608),
of `QuantType` metadata (src/quant.rs:375-456) and of `quant_mxfp4` (src/quant_mxfp4.rs), bound to
the C ABI in include/gllmk.h.  All compute happens in libgllmk.so (hand-written CUDA); there is no
CPU fallback and importing the compute classes fails loudly if the library is missing.
"""
from .quant import QuantType, QuantFormatDescriptor, registry, E2M1_LUT_F32, decode_e8m0_scale  # noqa: F401
from ._lib import GllmkError, Status, lib, lib_path, build_library  # noqa: F401
from .kernels import GpuKernels, HostBatch, Weight  # noqa: F401
from .shard import PeerExchange, ShardedLinear, gpu_sharded_linear, shard_rows, slice_blocks  # noqa: F401
from .gguf import GgufFile, GgufError, TensorInfo, write_gguf  # noqa: F401

__all__ = ["GgufFile", "GgufError", "TensorInfo", "write_gguf", "QuantType", "QuantFormatDescriptor", "registry", "E2M1_LUT_F32", "decode_e8m0_scale", "GllmkError", "Status", "lib", "lib_path",
           "build_library", "GpuKernels", "HostBatch", "Weight", "PeerExchange", "ShardedLinear", "gpu_sharded_linear", "shard_rows", "slice_blocks"]
