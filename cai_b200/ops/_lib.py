"""ctypes binding of ``libcai_kernels.so`` (the sm_100a kernel library).

The library is built in-tree by :mod:`cai_b200._build`. Loading it never needs a GPU; launching
does. If the library is missing the import of this module fails loudly rather than falling back
to PyTorch ops: on a GPU box the CUDA path is the only path.
"""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_void_p
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent.parent / "lib" / "libcai_kernels.so"
_lib = None


class KernelError(RuntimeError):
    pass


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise KernelError(
                f"{_LIB_PATH} is missing: run `python -m cai_b200._build` (or __graft_entry__.build()) first")
        _lib = ctypes.CDLL(str(_LIB_PATH), mode=ctypes.RTLD_GLOBAL)
        _declare(_lib)
    return _lib


def _declare(L):
    P, I, F, LL = c_void_p, c_int, c_float, c_longlong
    L.cai_last_error.restype = c_char_p
    L.cai_status_read.argtypes = [I]
    L.cai_sm_count.argtypes = []
    L.cai_gemm_bf16.argtypes = [P, P, P, P, I, I, I, LL, LL, LL, LL, I, I, I, F, I, P]
    L.cai_gemm_bf16_seg.argtypes = [P, P, P, P, I, I, I, LL, LL, LL, LL, I, I, I, F, P, I, I, I, P]
    if hasattr(L, "cai_gemm_fp8_blockscaled"):
        L.cai_gemm_fp8_blockscaled.argtypes = [P, P, P, P, P, P, I, I, I, LL, LL, LL, LL, I, P]
        L.cai_quant_rows_1x128.argtypes = [P, LL, P, LL, P, I, I, P]
        L.cai_quant_blocks_128x128.argtypes = [P, LL, P, LL, P, LL, P, P, I, I, P]
    if hasattr(L, "cai_gemm_bf16_grouped"):
        L.cai_gemm_bf16_grouped.argtypes = [P, P, P, I, I, I, LL, LL, LL, I, I, I, P, I, I, I, LL, LL, LL, I, P]
    L.cai_moe_route_fwd.argtypes = [P, P, P, P, P, I, I, I, I, P]
    L.cai_moe_route_bwd.argtypes = [P, P, P, P, P, I, I, I, P]
    ULL = ctypes.c_ulonglong
    L.cai_signal_block_bytes.restype = ULL
    L.cai_signal_block_bytes.argtypes = []
    L.cai_moe_dispatch_c.argtypes = [P, I, I, ULL, P, P, P, P, P, ULL, ULL, I, I, I, I, I, P, ctypes.c_uint32, P, P]
    L.cai_moe_combine_c.argtypes = [P, I, I, ULL, P, P, P, P, P, ULL, P, P, I, I, I, I, I, I, P, ctypes.c_uint32, P]
    L.cai_rmsnorm_fwd.argtypes = [P, P, P, P, I, I, F, P]
    L.cai_rmsnorm_bwd_parts.argtypes = [I]
    L.cai_rmsnorm_bwd.argtypes = [P, P, P, P, P, P, P, I, I, I, I, P]
    L.cai_rope_table.argtypes = [P, I, I, F, P]
    L.cai_rope_apply.argtypes = [P, P, I, I, I, I, I, LL, I, P]
    L.cai_swiglu_fwd.argtypes = [P, P, I, I, P]
    L.cai_swiglu_bwd.argtypes = [P, P, P, I, I, P]
    L.cai_embed_fwd.argtypes = [P, P, P, I, I, I, I, P]
    L.cai_embed_bwd.argtypes = [P, P, P, I, I, I, I, P]
    L.cai_cross_entropy.argtypes = [P, P, P, P, I, I, LL, F, F, P]
    L.cai_adamw.argtypes = [P, P, P, P, P, LL, F, F, F, F, F, F, I, P]
    L.cai_cast_f32_to_bf16.argtypes = [P, P, LL, P]
    L.cai_cast_bf16_to_f32.argtypes = [P, P, LL, P]
    L.cai_fill_f32.argtypes = [P, F, LL, P]
    L.cai_add_bf16.argtypes = [P, P, P, LL, P]
    L.cai_l2_flush.argtypes = [P, LL, P]
    if hasattr(L, "cai_flash_attn_fwd"):
        L.cai_flash_attn_fwd.argtypes = [P, P, P, I, I, I, I, I, F, P]
        L.cai_flash_attn_fwd_variant.argtypes = [P, P, P, I, I, I, I, I, F, I, P]
    if hasattr(L, "cai_flash_attn_bwd"):
        L.cai_flash_attn_bwd.argtypes = [P, P, P, P, P, P, I, I, I, I, I, F, P]
        L.cai_flash_attn_bwd_parts.argtypes = [P, P, P, P, P, P, I, I, I, I, I, F, I, P]


def check(rc: int, what: str):
    if rc != 0:
        msg = lib().cai_last_error()
        raise KernelError(f"{what} failed (rc={rc}): {msg.decode() if msg else ''}")


def device_status(clear: bool = True) -> int:
    """Status word of the current device: 0, or the code of the first bounded wait that ran out."""
    return lib().cai_status_read(1 if clear else 0)


def set_wait_limit_us(us: int) -> None:
    """Time limit of every in-kernel wait on another GPU's flag on the current device (0 = the default, ~2 s)."""
    check(lib().cai_set_wait_limit_us(ctypes.c_uint(int(us))), "set_wait_limit_us")


def status_abort() -> None:
    """Make every kernel of the current device that sits in a bounded wait give up now (status 108)."""
    check(lib().cai_status_abort(), "status_abort")
