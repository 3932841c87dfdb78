"""infurnace_b200: a single-GPU inference engine for the Qwen3 dense decoder on B200.

Importing the package loads no CUDA code; kernels are compiled and loaded on first use
(``infurnace_b200.kernels``)."""
__version__ = "0.1.0"
