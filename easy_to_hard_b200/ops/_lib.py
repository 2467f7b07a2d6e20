"""ctypes binding of the native sm_100a library.

The library is plain C entry points over raw device pointers and a CUDA stream, so the
binding needs no torch headers; tensors are passed as ``tensor.data_ptr()`` and kernels
run on ``torch.cuda.current_stream()`` (which is what makes them capturable in CUDA graphs
together with the surrounding torch code).

On a machine with a GPU the library is mandatory: ``lib()`` raises if it cannot be loaded,
so a missing build can never turn into a silent PyTorch fallback.
"""
from __future__ import annotations

import ctypes as C
from functools import lru_cache

import torch

from . import build as _build


class GemmParams(C.Structure):
    """Mirror of ``E2hGemmParams`` (csrc/gemm_umma.cuh)."""

    _fields_ = [
        ("F", C.c_int), ("T", C.c_int), ("K", C.c_int),
        ("splitk", C.c_int), ("epi", C.c_int), ("stages", C.c_int),
        ("a_mn_major", C.c_int), ("b_mn_major", C.c_int),
        ("bn", C.c_int), ("dual", C.c_int), ("accumulate", C.c_int), ("pdl", C.c_int),
        ("lda", C.c_longlong), ("lda2", C.c_longlong), ("ldb", C.c_longlong),
        ("a", C.c_void_p), ("a2", C.c_void_p), ("b", C.c_void_p),
        ("out", C.c_void_p), ("ldo", C.c_longlong),
        ("out2", C.c_void_p), ("ldo2", C.c_longlong),
        ("aux", C.c_void_p), ("scale", C.c_void_p),
        ("freqs", C.c_void_p), ("pos_base", C.c_void_p),
        ("sq", C.c_int), ("n_head", C.c_int), ("n_kv", C.c_int), ("head_dim", C.c_int),
        ("smax", C.c_int),
        ("kcache", C.c_void_p), ("vcache", C.c_void_p),
        ("status", C.c_void_p),
        ("tf", C.c_int),
        ("th", C.c_int),
        ("stage_epi", C.c_int),
        ("kps", C.c_int),
        ("n_signal", C.c_int),
        ("signal", C.c_void_p * 8),
        ("ticket", C.c_void_p),
        ("a_tiled", C.c_int),
        ("groupsize", C.c_int), ("qsz", C.c_void_p), ("qsz2", C.c_void_p),
        ("phase_clock", C.c_void_p),
    ]


EPI_STORE_BF16 = 0
EPI_STORE_F32 = 1
EPI_SWIGLU = 2
EPI_ROPE_KV = 3
EPI_RESIDUAL = 4
EPI_ROWMAJOR_F32_ACC = 5
EPI_ROWMAJOR_BF16 = 6
EPI_DUAL_STORE = 7

_vp, _i, _ll, _f, _ull = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_ulonglong

_SIGNATURES = {
    "e2h_gemm_umma": [C.POINTER(GemmParams), _vp],
    "e2h_gemm_persistent": [C.POINTER(GemmParams), _vp],
    "e2h_gemm_w8": [C.POINTER(GemmParams), _vp],
    "e2h_gemm_w4": [C.POINTER(GemmParams), _vp],
    "e2h_rmsnorm_fwd": [_vp, _vp, _vp, _i, C.POINTER(C.c_void_p), _i, _vp, _vp, _vp, _vp, _i, _i, _f,
                        _vp, _vp, _vp, _vp, _vp],
    "e2h_reduce_residual_norm_bf16": [_vp, C.POINTER(C.c_void_p), _i, _vp, _vp, _vp, _i, _i, _f,
                                      _vp, _vp, _vp, _vp, _vp],
    "e2h_rmsnorm_bwd": [_vp, _vp, _vp, _vp, _vp, _i, _i, _f, _vp],
    "e2h_embedding": [_vp, _vp, _i, _vp, _i, _i, _vp, _vp],
    "e2h_swiglu_fwd": [_vp, _vp, _vp, _ll, _vp],
    "e2h_swiglu_bwd": [_vp, _vp, _vp, _vp, _vp, _ll, _vp],
    "e2h_rope": [_vp, _vp, _vp, _vp, _i, _i, _i, _ll, _i, _vp],
    "e2h_attn_decode": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _f, _i, _vp, _vp,
                        _vp],
    "e2h_adamw": [_vp, _vp, _vp, _vp, _ll, _i, _i, _i, _f, _f, _f, _f, _f, _f, _f, _vp, _vp, _vp],
    "e2h_sqnorm": [_vp, _ll, _i, _vp, _vp],
    "e2h_clip_coef": [_vp, _f, _vp, _vp, _vp],
    "e2h_reward_head": [_vp, _ll, _vp, _vp, _ll, _i, _i, _i, _f, _vp, _i, _ll, _vp, _vp, _i, _vp, _vp,
                        _vp, _vp],
    "e2h_gae": [_vp, _vp, _vp, _vp, _i, _i, _f, _f, _vp],
    "e2h_flash_fwd": [_vp, _ll, _ll, _ll, _vp, _vp, _ll, _ll, _ll, _vp, _ll, _ll, _ll, _vp, _vp,
                      _i, _i, _i, _i, _i, _i, _f, _vp, _vp],
    "e2h_signal_peers": [C.POINTER(C.c_void_p), _i, _vp],
    "e2h_reduce_scatter_accum": [C.POINTER(C.c_void_p), _i, _vp, _ll, _f, _i, _vp, _vp, _vp, _i,
                                 _vp, _vp],
    "e2h_wait_flags": [_vp, _i, _vp, _i, _i, _vp, _vp],
    "e2h_p2p_all_gather": [C.POINTER(C.c_void_p), _i, _vp, _ll, _vp, _vp, _vp, _i, _vp, _vp],
    "e2h_p2p_reduce_bf16": [C.POINTER(C.c_void_p), _i, _vp, _ll, _f, _vp, _vp, _vp, _i, _vp, _vp],
    "e2h_tp_reduce_norm": [_vp, _vp, _vp, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                           C.POINTER(C.c_void_p), _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _i, _i,
                           _i, _i, _vp, _vp],
    "e2h_tp_rows": [_i, _vp, _vp, _vp, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                    C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), _vp, _vp, _vp, _vp, _i, _i, _i,
                    _i, _f, _i, _i, _i, _vp, _vp],
    "e2h_tp_embed_partial": [_vp, _vp, _i, _i, _vp, _i, _i, C.POINTER(C.c_void_p), _i, _vp, _vp],
    "e2h_tp_gather_logits": [C.POINTER(C.c_void_p), _i, _i, _i, _vp, _ll, _vp, _vp, _vp, _i, _vp,
                             _vp],
    "e2h_relayout_pull": [C.POINTER(C.c_void_p), _i, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _ll, _vp,
                          _vp],
    "e2h_set_pdl": [_i],
    "e2h_set_flag_wait_ms": [_i],
    "e2h_flash_bwd": [_vp, _ll, _ll, _ll, _vp, _vp, _ll, _ll, _ll, _vp, _ll, _ll, _ll, _vp, _ll,
                      _ll, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _vp,
                      _vp],
    "e2h_ce_stats": [_vp, _ll, _i, _i, _vp, _i, _f, _vp, _vp],
    "e2h_ce_grad": [_vp, _ll, _i, _i, _vp, _i, _f, _vp, _vp, _vp, _vp, _vp, _ll, _vp],
    "e2h_sample": [_vp, _ll, _i, _i, _f, _i, _ull, _vp, _i, _vp, _vp, _ll, _i, _i, _vp, _vp,
                   _vp, _vp, _vp],
}


class NativeLibraryError(RuntimeError):
    pass


@lru_cache(maxsize=1)
def lib() -> C.CDLL:
    """Load (building first if the sources changed and nvcc is present) the native library."""
    path = _build.lib_path()
    try:
        if _build.needs_build():
            path = _build.build()
    except Exception as e:  # no nvcc on this machine: use the shipped binary if there is one
        if not path.exists():
            raise NativeLibraryError(f"native library missing and cannot be built: {e}") from e
    try:
        cdll = C.CDLL(str(path))
    except OSError as e:
        raise NativeLibraryError(f"cannot load {path}: {e}") from e
    for name, argtypes in _SIGNATURES.items():
        try:
            fn = getattr(cdll, name)
        except AttributeError:
            continue  # optional entry point of a newer / older build
        fn.argtypes = argtypes
        fn.restype = C.c_int
    return cdll


def available() -> bool:
    """True when CUDA kernels can run here (a GPU is visible and the library loads)."""
    if not torch.cuda.is_available():
        return False
    lib()  # raises loudly on a GPU machine without the library
    return True


def ptr(t) -> int | None:
    if t is None:
        return None
    return t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeLibraryError(f"{what} failed with code {rc}")


_status_words: dict = {}


def status_word(device=None) -> torch.Tensor:
    """Per-device int32 status word that kernels write a code to when a bounded wait expires."""
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    if dev.type != "cuda":
        dev = torch.device("cuda", torch.cuda.current_device())
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    w = _status_words.get(dev.index)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=dev)
        _status_words[dev.index] = w
    return w


def read_status(device=None, reset: bool = True) -> int:
    w = status_word(device)
    v = int(w.item())
    if reset and v != 0:
        w.zero_()
    return v
