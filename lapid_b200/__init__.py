"""B200 (sm_100a) backend for lapid's quantized-matmul path.

The product is the C-ABI library ``liblapid_b200.so`` (``include/lapid_b200.h``); this package
is the Python binding over it, shaped like the reference's operator surface so that tests read
like the reference's own:

* :class:`Backend` -- ``lapid_compiler::Backend`` (crates/lapid-compiler/src/backend.rs:8-63)
* :class:`Launch`, :class:`MatMulSpec`, :class:`MatMulDims`, :class:`MatView`, :class:`View`
  -- crates/lapid-compiler/src/ir.rs:226-282, :483-488
* :mod:`lapid_b200.quant` -- ``lapid_quant::{Format, layout, quantize, dequantize,
  from_ggml_blocks}`` (crates/lapid-quant/src/lib.rs:27-160)
* :mod:`lapid_b200.gguf` -- the GGUF tensor table and its "keep the blocks" import
  (crates/lapid-convert/src/gguf.rs:1-12, :177-215)

There is no CPU fallback anywhere: importing works without a GPU (so the library and its symbols
can be checked), but every device call fails with ``device_unavailable`` / ``cuda_unavailable``.
"""
from ._lib import LapidError, abi_version, lib, library_path  # noqa: F401
from .backend import (Backend, Buffer, DType, Epilogue, Launch, MatMulDims, MatMulSpec, MatView, View,  # noqa: F401
                      gather_launch, matmul_id_launch, matmul_launch)
from . import quant  # noqa: F401
from . import gguf  # noqa: F401
