"""B200-native quantized matrix products for go-pherence (MLX 4-bit, GPTQ INT4, GGUF Q8_0/Q4_K/Q5_K/Q6_K, FP8 E4M3).

`runtime` mirrors the operator API of the reference's backends/nvidia/runtime package over
the C ABI of libgoph_b200.so; `build` compiles that library in-tree; `checkpoint` reads safetensors
and GGUF files into the uploads.
"""
from . import build  # noqa: F401
from . import checkpoint  # noqa: F401
from . import runtime  # noqa: F401
from . import decode  # noqa: F401
from . import sharding  # noqa: F401
from . import synth  # noqa: F401
