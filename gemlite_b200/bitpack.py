"""Weight bit-packing front end (same function names and results as gemlite/bitpack.py).

All four directions run as CUDA kernels through the C ABI (``gl_pack_over_cols`` & co.), bit
for bit equal to the reference's torch loops (gemlite/bitpack.py:10-60, 146-163, 320-336).
The ``*_torch`` and ``*_triton`` names of the reference are kept as aliases of the one CUDA
implementation: there is no second code path.
"""
import torch

from . import _lib
from .dtypes import PACKING_BITWIDTH_TO_TORCH_DTYPE, TORCH_TO_DTYPE


def _check_bits(W_nbits, packing_bitwidth):
    assert packing_bitwidth in [8, 16, 32, 64], "Unsuported bitpacking width"
    assert W_nbits in [8, 4, 2, 1], "Unsuported nbits"


def pack_weights_over_cols(W_q: torch.Tensor, W_nbits: int, packing_bitwidth: int, transpose: bool):
    """Pack ``W_q`` [rows, cols] (one value per element, uint8 range) along its columns.

    Returns ``(packed [rows, cols // e], e)`` with ``e = packing_bitwidth // W_nbits``; with
    ``transpose`` the ``.t()`` view is returned, as the reference does (bitpack.py:58, 141).
    """
    _check_bits(W_nbits, packing_bitwidth)
    _lib.require_cuda(W_q, "W_q")
    e = packing_bitwidth // W_nbits
    src = W_q.to(torch.uint8).contiguous()
    rows, cols = src.shape
    out = torch.empty((rows, cols // e), dtype=PACKING_BITWIDTH_TO_TORCH_DTYPE[packing_bitwidth], device=W_q.device)
    with torch.cuda.device(W_q.device):
        _lib.check(_lib.lib().gl_pack_over_cols(src.data_ptr(), out.data_ptr(), rows, cols, W_nbits, packing_bitwidth,
                                                _lib.current_stream_ptr(W_q.device)))
    if transpose:
        out = out.t()
    return out, e


def pack_weights_over_rows(W_q: torch.Tensor, W_nbits: int, packing_bitwidth: int, transpose: bool):
    """Pack ``W_q`` [rows, cols] along its rows: ``(packed [rows // e, cols], e)``."""
    _check_bits(W_nbits, packing_bitwidth)
    _lib.require_cuda(W_q, "W_q")
    e = packing_bitwidth // W_nbits
    src = W_q.to(torch.uint8).contiguous()
    rows, cols = src.shape
    out = torch.empty((rows // e, cols), dtype=PACKING_BITWIDTH_TO_TORCH_DTYPE[packing_bitwidth], device=W_q.device)
    with torch.cuda.device(W_q.device):
        _lib.check(_lib.lib().gl_pack_over_rows(src.data_ptr(), out.data_ptr(), rows, cols, W_nbits, packing_bitwidth,
                                                _lib.current_stream_ptr(W_q.device)))
    if transpose:
        out = out.t()
    return out, e


def _packing_bitwidth_of(t):
    return t.element_size() * 8


def _unpack_over_cols_impl(W_q_packed: torch.Tensor, W_nbits: int, num_output_cols: int,
                           dtype: torch.dtype = torch.uint8) -> torch.Tensor:
    """Inverse of :func:`pack_weights_over_cols`: [rows, cols_packed] -> [rows, num_output_cols].

    ``num_output_cols // cols_packed`` fields are taken from every word (bitpack.py:154-155)."""
    _lib.require_cuda(W_q_packed, "W_q_packed")
    src = W_q_packed.contiguous()
    pb = _packing_bitwidth_of(src)
    rows, cols_packed = src.shape
    e = num_output_cols // cols_packed
    out = torch.empty((rows, cols_packed * e), dtype=dtype, device=src.device)
    with torch.cuda.device(src.device):
        _lib.check(_lib.lib().gl_unpack_over_cols(src.data_ptr(), out.data_ptr(), rows, cols_packed, W_nbits, pb, e,
                                                  TORCH_TO_DTYPE[dtype].value, _lib.current_stream_ptr(src.device)))
    return out.view(rows, num_output_cols)


def _unpack_over_cols_fake(W_q_packed, W_nbits, num_output_cols, dtype=torch.uint8):
    return torch.empty((W_q_packed.shape[0], num_output_cols), dtype=dtype, device=W_q_packed.device)


def _unpack_over_rows_impl(W_q_packed: torch.Tensor, W_nbits: int, num_output_rows: int,
                           dtype: torch.dtype = torch.uint8) -> torch.Tensor:
    """Inverse of :func:`pack_weights_over_rows`: [rows_packed, cols] -> [num_output_rows, cols]."""
    _lib.require_cuda(W_q_packed, "W_q_packed")
    src = W_q_packed.contiguous()
    pb = _packing_bitwidth_of(src)
    rows_packed, cols = src.shape
    e = num_output_rows // rows_packed
    out = torch.empty((rows_packed * e, cols), dtype=dtype, device=src.device)
    with torch.cuda.device(src.device):
        _lib.check(_lib.lib().gl_unpack_over_rows(src.data_ptr(), out.data_ptr(), rows_packed, cols, W_nbits, pb, e,
                                                  TORCH_TO_DTYPE[dtype].value, _lib.current_stream_ptr(src.device)))
    return out.view(num_output_rows, cols)


def _unpack_over_rows_fake(W_q_packed, W_nbits, num_output_rows, dtype=torch.uint8):
    return torch.empty((num_output_rows, W_q_packed.shape[1]), dtype=dtype, device=W_q_packed.device)


def _register_op(name, impl, fake):
    op = torch.library.custom_op("gemlite::" + name, mutates_args=())(impl)
    torch.library.register_fake("gemlite::" + name)(fake)
    return op


# Operator names: the reference registers gemlite::unpack_over_{cols,rows}_{torch,triton} (gemlite/bitpack.py:146, 207,
# 320, 383) and graphs traced against it carry those names; all of them are the one CUDA kernel here.
unpack_over_cols_torch = _register_op("unpack_over_cols_torch", _unpack_over_cols_impl, _unpack_over_cols_fake)
unpack_over_cols_triton = _register_op("unpack_over_cols_triton", _unpack_over_cols_impl, _unpack_over_cols_fake)
unpack_over_rows_torch = _register_op("unpack_over_rows_torch", _unpack_over_rows_impl, _unpack_over_rows_fake)
unpack_over_rows_triton = _register_op("unpack_over_rows_triton", _unpack_over_rows_impl, _unpack_over_rows_fake)
unpack_over_cols = unpack_over_cols_triton
unpack_over_rows = unpack_over_rows_triton

# Names the reference exports (gemlite/bitpack.py:430-433 and the *_torch / *_triton pairs).
pack_weights_over_cols_torch = pack_weights_over_cols
pack_weights_over_cols_triton = pack_weights_over_cols
pack_weights_over_rows_torch = pack_weights_over_rows
pack_weights_over_rows_triton = pack_weights_over_rows
