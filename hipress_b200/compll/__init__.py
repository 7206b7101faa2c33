"""CompLL: a small DSL for gradient-compression algorithms and a generator that
turns it into sm_100a CUDA kernels (and plain C++ for CPU tensors) with PyTorch
bindings; ``load_op`` gives the shipped operators, built on first use."""
from .emit_cuda import Emitter, generate  # noqa: F401
from .frontend import CompileError, parse, tokenize  # noqa: F401
from .generator import compile_generated, generate_files  # noqa: F401
from .library import available, build_all, build_op, load_op  # noqa: F401
