"""ctypes bindings of the CUDA kernel library.

The library is hand-written CUDA for sm_100a with a C interface; it is compiled on first use
and loaded from the source tree. There is no fallback: if it cannot be built or loaded,
:func:`kernels` raises.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p
from functools import lru_cache

import torch

from . import build

DTYPE_CODES = {torch.float32: 0, torch.bfloat16: 1}

ERROR_BITS = {
    1: "a block-table entry was negative or past the cache arena",
    2: "a token id was outside the embedding table",
    4: "a position did not fit the block table",
    8: "a kernel gave up waiting on one of its own barriers",
}


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODES[dtype]
    except KeyError:
        raise KernelError(f"kernels take float32 or bfloat16, not {dtype}") from None


def ptr(tensor: torch.Tensor | None) -> int | None:
    """A tensor's device address as ctypes takes it for a declared ``c_void_p`` parameter: a plain
    int (None for a null pointer). No ctypes object is built per argument: a step makes some two
    thousand of these calls."""
    return None if tensor is None else tensor.data_ptr()


def stream_handle() -> c_void_p:
    return c_void_p(torch.cuda.current_stream().cuda_stream)


_SIGNATURES: dict[str, list] = {
    "b200_embedding_gather": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_void_p],
    "b200_rmsnorm": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_float, c_int, c_void_p],
    "b200_silu_mul": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "b200_rope_kv_write": [c_void_p] * 7 + [c_int, c_int] + [c_void_p] * 3 + [c_int] * 8 + [c_void_p, c_void_p],
    "b200_paged_attention_plain": [c_void_p] * 6
    + [c_int, c_int, c_void_p]
    + [c_int] * 6
    + [c_float, c_int, c_void_p, c_void_p],
    "b200_gemm_f32": [c_void_p] * 4 + [c_int] * 6 + [c_void_p],
    "b200_paged_flash_attention": [c_void_p] * 8 + [c_int] * 11 + [c_float, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "b200_paged_decode_attention_tma": [c_void_p] * 8 + [c_int] * 8 + [c_float, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "b200_flash_prefill_tcgen05": [c_void_p] * 8 + [c_int] * 11 + [c_float, c_void_p, c_void_p],
    "b200_skinny_gemm": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int64, c_void_p, c_int, c_void_p],
    "b200_stream_gemm": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "b200_skinny_gemm_fold": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_int64, c_void_p, c_int,
                              c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "b200_stream_gemm_fold": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p,
                              c_void_p, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "b200_argmax_rows": [c_void_p, c_int, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p],
    "b200_sample_rows": [c_void_p, c_int, c_int, c_int64] + [c_void_p] * 7 + [c_void_p, c_int64, c_void_p],
}


class KernelLibrary:
    def __init__(self, path: str) -> None:
        self.path = path
        self.lib = ctypes.CDLL(path)
        self.lib.b200_last_error.restype = ctypes.c_char_p
        self.lib.b200_abi_version.restype = c_int
        self.lib.b200_flash_attention_supported.argtypes = [c_int] * 5
        self.lib.b200_flash_attention_supported.restype = c_int
        self.lib.b200_decode_attention_tma_supported.argtypes = [c_int] * 4
        self.lib.b200_decode_attention_tma_supported.restype = c_int
        self.lib.b200_flash_prefill_tcgen05_supported.argtypes = [c_int] * 5
        self.lib.b200_flash_prefill_tcgen05_supported.restype = c_int
        self.lib.b200_skinny_gemm_supported.argtypes = [c_int] * 4
        self.lib.b200_skinny_gemm_supported.restype = c_int
        self.lib.b200_skinny_gemm_scratch.argtypes = [c_int, c_int, c_int, ctypes.POINTER(c_int64), ctypes.POINTER(c_int)]
        self.lib.b200_skinny_gemm_scratch.restype = None
        self.lib.b200_stream_gemm_supported.argtypes = [c_int] * 4
        self.lib.b200_stream_gemm_supported.restype = c_int
        self.lib.b200_stream_gemm_plan_override.argtypes = [c_int] * 3
        self.lib.b200_stream_gemm_plan_override.restype = None
        self.lib.b200_stream_gemm_trace.argtypes = [c_void_p, c_int, c_int]
        self.lib.b200_stream_gemm_trace.restype = None
        self.lib.b200_stream_gemm_trace_stamps.argtypes = []
        self.lib.b200_stream_gemm_trace_stamps.restype = c_int
        self.lib.b200_sm_count.restype = c_int
        self.lib.b200_skinny_gemm_fold_parts.argtypes = [c_int, c_int]
        self.lib.b200_skinny_gemm_fold_parts.restype = c_int
        self.lib.b200_stream_gemm_fold_parts.argtypes = [c_int, c_int, c_int]
        self.lib.b200_stream_gemm_fold_parts.restype = c_int
        self._functions = {}
        self.calls = 0  # kernel launches issued through this library
        for name, argtypes in _SIGNATURES.items():
            self.bind(name, argtypes)

    def bind(self, name: str, argtypes: list) -> None:
        try:
            fn = getattr(self.lib, name)
        except AttributeError:
            raise KernelError(f"{self.path} does not export {name}") from None
        fn.argtypes = argtypes
        fn.restype = c_int
        self._functions[name] = fn

    def has(self, name: str) -> bool:
        return hasattr(self.lib, name)

    def call(self, name: str, *args) -> None:
        status = self._functions[name](*args)
        self.calls += 1
        if status != 0:
            raise KernelError(self.lib.b200_last_error().decode(errors="replace"))


@lru_cache(maxsize=1)
def kernels() -> KernelLibrary:
    """The loaded kernel library; builds it first if the sources changed."""
    if not torch.cuda.is_available():
        raise KernelError(
            "the engine's kernels are CUDA code for sm_100a and no CUDA device is visible; "
            "there is no CPU path"
        )
    return KernelLibrary(str(build.build_kernels()))


def check_error_word(word: torch.Tensor, where: str) -> None:
    """Raise if a kernel set a bit in the device error word (this synchronises)."""
    value = int(word.item())
    if value:
        reasons = [text for bit, text in ERROR_BITS.items() if value & bit]
        word.zero_()
        raise KernelError(f"{where}: " + "; ".join(reasons or [f"error bits {value}"]))
