"""mnemocuda_b200: sm_100a kernels for MnemoCUDA's quantized-weight hot path.

`kernels` mirrors the reference's extern "C" kernel ABI over torch tensors;
`synth` generates the seeded synthetic GGUF blocks the benchmark runs on.
The compute lives in libmnemo_b200.so (csrc/, built by `build`); importing
`kernels` without it raises.
"""
from . import synth  # noqa: F401

__all__ = ["synth"]
