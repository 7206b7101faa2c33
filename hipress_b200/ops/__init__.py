"""Compression operators: algorithm table and tensor-level encode/decode."""
from .algorithms import AlgSpec, algorithm_names, get_algorithm  # noqa: F401
from .compressor import Compressor, PayloadError, sparse_pairs  # noqa: F401
from .custom import CustomCompressor, register_algorithm, unregister_algorithm  # noqa: F401
