"""helix_b200 -- B200-native NVFP4 quantizer and decode/prefill loop behind Helix's boundary.

The product is the C-ABI shared library ``libhelix_b200.so`` (declared in ``include/helix_b200.h``)
and the kernel-entry image ``helix_b200_kernels.fatbin``; this package is the ctypes binding used by
the tests and the benchmark.  There is no CPU fallback: every call fails with ``HxError`` when the
library or a GPU is missing.
"""
from .lib import (HxError, HxConfig, Model, lib, lib_path, fatbin_path, quantize_host, roundtrip_host,
                  DeviceBuffer, PinnedArray, KernelImage, launch_count, QWEN3_8B, QWEN3_32B, GPT2_124M,
                  HX_LOAD_KEEP_COMMITTED, HX_LOAD_VERIFY_SHA, HX_LOAD_FILE_EPS, pld_draft, pack_qwen3, probe_mxf4_rate, Sampler, worker_path, Tokenizer)

__all__ = ["HxError", "HxConfig", "Model", "lib", "lib_path", "fatbin_path", "quantize_host",
           "roundtrip_host", "DeviceBuffer", "PinnedArray", "KernelImage", "launch_count", "QWEN3_8B", "QWEN3_32B", "GPT2_124M",
           "HX_LOAD_KEEP_COMMITTED", "HX_LOAD_VERIFY_SHA", "HX_LOAD_FILE_EPS", "pld_draft", "pack_qwen3", "probe_mxf4_rate", "Sampler", "worker_path", "Tokenizer"]
