"""qwenforge_b200: a small model library with generation of its own for NVIDIA B200 (sm_100a).

Everything between a request's tokens and its next token for the dense grouped-query Qwen2
decoder: typed configuration and registry, safetensors weights by name, layers put together from
parts, a paged sequence cache, one step function, a generation loop, sampling, and hand-written
CUDA kernels. Importing the package touches no GPU and compiles nothing.
"""
__version__ = "0.1.0"
