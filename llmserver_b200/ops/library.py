"""Loads the compiled kernel library and declares the C launchers' signatures.

There is no fallback: if the library cannot be built or loaded, or the device is not a B200-class
GPU, the engine refuses to run.
"""
from __future__ import annotations

import ctypes
import threading

import torch

from ..csrc.build import KernelBuildError, ensure_built

_P, _I, _F, _S = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_void_p

# name -> argument types (every launcher returns an int status; the stream comes last)
SIGNATURES = {
    "llm_embedding_gather": [_P, _P, _P, _I, _I, _I, _I, _S],
    "llm_add_rmsnorm": [_P, _P, _P, _P, _P, _I, _I, _F, _I, _I, _I, _P, _S],
    "llm_rmsnorm": [_P, _P, _P, _I, _I, _F, _I, _I, _S],
    "llm_silu_mul": [_P, _P, _I, _I, _I, _I, _S],
    "llm_sample": [_P, _P, _P, _P, _P, _I, _I, _P, _P, _S],
    "llm_sample_slices": [_I, _I],
    "llm_qk_norm_rope_kv_write": [_P, _P, _P, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _I, _I, _I, _I, _S],
    "llm_attention_generic": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _P, _I, _S],
    "llm_gemm_f32": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _S],
    "llm_attention_mma_supports": [_I, _I, _I],
    "llm_attention_prefill_tcgen05_supports": [_I, _I, _I, _I],
    "llm_attention_prefill_tcgen05": [_P, _I, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _I, _I, _P, _S],
    "llm_attention_prefill_wide_supports": [_I, _I, _I, _I],
    "llm_attention_prefill_wide": [_P, _I, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _I, _I, _P, _S],
    "llm_gemm_small_m_supports": [_I, _I, _I],
    "llm_gemm_small_m": [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _I, _I, _F, _P, _S],
    "llm_gemm_into_stream_parts": [_I],
    "llm_gemm_into_stream": [_P, _P, _P, _I, _I, _I, _I, _P, _I, _P, _P, _I, _P, _S],
    "llm_gemm_gate_up_silu": [_P, _P, _P, _I, _I, _I, _I, _I, _P, _I, _I, _F, _P, _S],
    "llm_gemm_qkv_rope_supports": [_I, _I, _I, _I, _I],
    "llm_gemm_qkv_rope": [_P, _P, _P, _I, _I, _I, _I, _P, _P, _I, _P, _P, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _F, _I, _P,
                          _P, _I, _I, _F, _P, _S],
    "llm_attention_mma": [_P, _I, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _I, _I, _I, _I, _P, _P, _I, _P, _S],
}

_lock = threading.Lock()
_library = None
_arch_checked = False


class KernelError(RuntimeError):
    """A launcher refused its arguments or CUDA reported an error."""


def library() -> ctypes.CDLL:
    global _library
    if _library is None:
        with _lock:
            if _library is None:
                path = ensure_built()
                try:
                    loaded = ctypes.CDLL(path)
                except OSError as error:
                    raise KernelBuildError(f"the kernel library {path} could not be loaded: {error}") from error
                loaded.llm_last_error.restype = ctypes.c_char_p
                loaded.llm_last_error.argtypes = []
                for name, argtypes in SIGNATURES.items():
                    function = getattr(loaded, name)
                    function.argtypes = argtypes
                    function.restype = ctypes.c_int
                _library = loaded
    return _library


def declare(name: str, argtypes) -> None:
    """Adds a launcher's signature (used by modules that own further kernels)."""
    SIGNATURES[name] = argtypes
    if _library is not None:
        function = getattr(_library, name)
        function.argtypes = argtypes
        function.restype = ctypes.c_int


def require_device() -> None:
    """Raises unless CUDA is usable and the current device is compute capability 10.x."""
    global _arch_checked
    if _arch_checked:
        return
    if not torch.cuda.is_available():
        raise KernelError("llmserver_b200 runs on a CUDA device only (no CPU path); torch.cuda.is_available() is False")
    arch = library().llm_device_arch()
    if arch < 0:
        raise KernelError(f"device query failed: {library().llm_last_error().decode()}")
    if arch // 10 != 10:
        raise KernelError(f"the kernels are built for sm_100a (B200); the current device is sm_{arch}")
    _arch_checked = True


_launches = 0


def launch_count() -> int:
    """How many of this package's kernel launchers have been called in this process."""
    return _launches


def call(name: str, *args) -> None:
    global _launches
    _launches += 1
    status = getattr(library(), name)(*args)
    if status != 0:
        raise KernelError(f"{name} failed ({status}): {library().llm_last_error().decode()}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream_handle() -> int:
    """The raw handle of PyTorch's current stream on the current device (asked for at every launch: it is
    another stream while a CUDA graph is being captured)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return 0
    if dtype == torch.bfloat16:
        return 1
    raise KernelError(f"the kernels take float32 or bfloat16, not {dtype}")


def pointer(tensor) -> int:
    return 0 if tensor is None else tensor.data_ptr()


def check(tensor: torch.Tensor, name: str, dtype=None, last_dim=None) -> torch.Tensor:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must live on a CUDA device (there is no CPU path); it is on {tensor.device}")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous; strides {tensor.stride()} for shape {tuple(tensor.shape)}")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
    if last_dim is not None and tensor.shape[-1] != last_dim:
        raise KernelError(f"{name}: last dimension {tensor.shape[-1]} != {last_dim}")
    return tensor


_wait_error_flags = {}


def wait_error_flag(device) -> torch.Tensor:
    """Device word that a kernel sets when one of its bounded waits (on an mbarrier: a TMA copy or an MMA
    that never reported completion) ran out.  Never expected; checked after steps by ``check_wait_errors``."""
    device = torch.device(device)
    if device.index is None and device.type == "cuda":
        device = torch.device("cuda", torch.cuda.current_device())
    if device not in _wait_error_flags:
        _wait_error_flags[device] = torch.zeros(1, dtype=torch.int32, device=device)
    return _wait_error_flags[device]


def check_wait_errors() -> None:
    for flag in _wait_error_flags.values():
        code = int(flag.item())
        if code != 0:
            flag.zero_()
            raise KernelError(f"a kernel gave up waiting on one of its barriers (code {code}: 2 matrix product, "
                              "3 decode attention, 4 prompt attention), or attention met a block-table entry that names no "
                              "page of the pool (5) or a context that needs more splits than it was given (6); the step's "
                              "result is invalid")
