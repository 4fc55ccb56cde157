"""Operator API of the paged NVFP4 decode kernel (drop-in for ``nvfp4_decode_kernel``)."""

from .interface import RESIDUAL_ROW_TILE, KernelNotAvailableError, fp4_decode, host_io_step

__all__ = ["RESIDUAL_ROW_TILE", "KernelNotAvailableError", "fp4_decode", "host_io_step"]
