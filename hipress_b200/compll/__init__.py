"""CompLL: a small DSL for gradient-compression algorithms and a generator that
turns it into sm_100a CUDA kernels with PyTorch bindings."""
from .emit_cuda import Emitter, generate  # noqa: F401
from .frontend import CompileError, parse, tokenize  # noqa: F401
from .generator import compile_generated, generate_files  # noqa: F401
