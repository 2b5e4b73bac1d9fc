"""webllm_b200 — B200 (sm_100a) implementation of webllm's GPTQ-int4 quantized-linear path.

The product is the C-ABI library ``lib/libwebllm_b200.so`` (sources in ``csrc/``, interface in
``include/webllm_b200.h``). This package is the thin host layer over it, mirroring the reference's
TypeScript operator surface (``dequantizeGptqInt4``, ``Arena``/``Tensor``, ``QwenGpt.gemm`` and the
``upload*`` family, ``planGemvSplit``, ``generateQwen``).
"""
from ._lib import WebllmError, LIB_PATH  # noqa: F401
from .buffer import ALIGN, Tensor, align_to  # noqa: F401
from .device import Arena, Gpu  # noqa: F401
from .quant import GptqInt4Params, dequantize_gptq_int4  # noqa: F401
from .qwen import QwenGpt, concat_gptq  # noqa: F401,E402
from .generate import SamplerOptions, generate_qwen, sample_token  # noqa: F401,E402
from .plan import plan_gemv_split  # noqa: F401,E402
from .qwen_loader import QwenLoadResult, load_qwen_weights  # noqa: F401,E402
