"""ctypes binding of libbsa_b200.so (declarations mirror include/bsa.h).

The library is the only compute path of this package: if it is missing the
import fails with a clear error instead of falling back to anything else.
"""
from __future__ import annotations

import ctypes as C
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("BSA_B200_LIB") or os.path.join(_HERE, "libbsa_b200.so")

BSA_F16, BSA_BF16, BSA_F32, BSA_F8E4M3 = 0, 1, 2, 3
IMPL_AUTO, IMPL_GENERIC, IMPL_SM100 = 0, 1, 2
ROWS_BY_TILE, ROWS_BY_POSITION = 0, 1

_i32, _i64, _f32, _vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p


class LocalStrideParams(C.Structure):
    _fields_ = [(n, _i32) for n in (
        "num_heads", "num_kv_heads", "num_dense_heads", "q_blocks", "kv_blocks", "q_start_block",
        "kv_start_block", "trim_q_blocks", "local_left", "local_right", "vert_stride",
        "head_sliding_step", "head_sliding_offset", "causal", "absolute_vert")]


class FwdParams(C.Structure):
    _fields_ = (
        [(n, _vp) for n in ("q", "k", "v", "o", "lse")]
        + [(n, _i64) for n in ("q_sb", "q_ss", "q_sh", "k_sb", "k_ss", "k_sh", "v_sb", "v_ss", "v_sh",
                               "o_sb", "o_ss", "o_sh", "lse_sb", "lse_sh")]
        + [(n, _i32) for n in ("batch", "hq", "hkv", "d", "sq", "sk", "total_q")]
        + [(n, _vp) for n in ("q_start", "q_end", "k_start", "k_end", "crow", "col")]
        + [(n, _i64) for n in ("crow_sh", "col_sh")]
        + [(n, _i32) for n in ("h_pat", "n_rows", "block_size", "causal", "row_mode", "dtype", "impl")]
        + [("sm_scale", _f32), ("col_bits", _vp), ("col_bits_sh", _i64), ("fine_block", _i32),
           ("tile_counter", _vp)]
    )


class BwdParams(C.Structure):
    _fields_ = (
        [("f", FwdParams), ("d_o", _vp), ("d_lse", _vp)]
        + [(n, _i64) for n in ("do_sb", "do_ss", "do_sh")]
        + [(n, _vp) for n in ("dq", "dk", "dv")]
        + [(n, _i64) for n in ("dq_sb", "dq_ss", "dq_sh", "dk_sb", "dk_ss", "dk_sh",
                               "dv_sb", "dv_ss", "dv_sh")]
        + [("ccol", _vp), ("row", _vp), ("ccol_sh", _i64), ("row_sh", _i64), ("n_cols", _i32),
           ("delta", _vp), ("kv_pairs", _vp), ("kv_pairs_sh", _i64), ("n_pairs", _i32),
           ("ds_ws", _vp), ("ds_tiles_per_head", _i64), ("csc_csr", _vp)]
    )


class DecodeParams(C.Structure):
    _fields_ = (
        [(n, _vp) for n in ("q", "k", "v", "o", "lse")]
        + [(n, _i64) for n in ("q_sb", "q_sh", "k_sb", "k_ss", "k_sh", "v_sb", "v_ss", "v_sh",
                               "o_sb", "o_sh", "lse_sb", "lse_sh")]
        + [(n, _i32) for n in ("batch", "hq", "hkv", "d", "sk")]
        + [(n, _vp) for n in ("k_start", "k_end", "k_pos0", "k_total", "crow", "col")]
        + [(n, _i64) for n in ("crow_sh", "col_sh")]
        + [(n, _i32) for n in ("h_pat", "n_rows", "block_size", "heads_per_cta", "blocks_per_split",
                               "max_row_nnz", "dtype")]
        + [("sm_scale", _f32), ("ws", _vp), ("k_blk_mod", _i32), ("k_blk_rem", _i32),
           ("kv_dtype", _i32), ("k_scale", _f32), ("v_scale", _f32)]
    )


class XchgParams(C.Structure):
    _fields_ = ([(n, _vp) for n in ("stage_o", "stage_lse", "out", "out_lse")]
                + [("xbuf", _vp * 8), ("rows", _i64)]
                + [(n, _i32) for n in ("world", "rank", "d", "dtype")]
                + [("part_o", _vp), ("part_lse", _vp), ("nsplit", _i32)])


EXPORTS = {
    # name: (restype, argtypes)
    "bsa_abi_version": (_i32, []),
    "bsa_last_error": (C.c_char_p, []),
    "bsa_local_stride_mask": (_i32, [C.POINTER(LocalStrideParams), _vp, _vp]),
    "bsa_csr_row_ptr": (_i32, [_vp, _i32, _i32, _i32, _i64, _i64, _i64, _vp, _vp, _vp]),
    "bsa_csr_fill_cols": (_i32, [_vp, _i32, _i32, _i32, _i64, _i64, _i64, _vp, _vp, _i32, _i32, _vp]),
    "bsa_fwd": (_i32, [C.POINTER(FwdParams), _vp]),
    "bsa_fwd_uses_sm100": (_i32, [C.POINTER(FwdParams)]),
    "bsa_bwd": (_i32, [C.POINTER(BwdParams), _vp]),
    "bsa_decode_workspace_bytes": (C.c_size_t, [C.POINTER(DecodeParams)]),
    "bsa_decode": (_i32, [C.POINTER(DecodeParams), _vp]),
    "bsa_decode_static": (_i32, [C.POINTER(DecodeParams), _vp]),
    "bsa_decode_static_capacity": (C.c_size_t, []),
    "bsa_merge_partials": (_i32, [_vp, _vp, _i32, _i64, _i32, _i64, _i64, _i64, _i64, _vp, _i64, _vp,
                                  _i32, _vp]),
    "bsa_xchg_buffer_bytes": (C.c_size_t, [_i32, _i64, _i32]),
    "bsa_xchg_merge": (_i32, [C.POINTER(XchgParams), _vp]),
    "bsa_wait_status": (_i32, [C.POINTER(_i32), _i32]),
    "bsa_set_wait_status_mirror": (_i32, [_vp]),
    "bsa_selftest_wait_timeout": (_i32, [C.c_uint32, _vp]),
    "bsa_fwd_why_not_sm100": (C.c_char_p, [C.POINTER(FwdParams)]),
}

_lib = None


class BsaError(RuntimeError):
    """An entry point of libbsa_b200.so returned a non-zero code."""


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m dkernel_b200._build` "
                "(nvcc, sm_100a). There is no other compute path in this package.")
        l = C.CDLL(LIB_PATH)
        for name, (res, args) in EXPORTS.items():
            fn = getattr(l, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
        if l.bsa_abi_version() != 3:
            raise RuntimeError("libbsa_b200.so has an unexpected ABI version; rebuild it")
        _lib = l
    return _lib


# Host-visible copy of the device wait-status word (one pinned int32 shared by all devices):
# the kernels store the code of the first bounded wait that gave up there, so every later
# call can raise without synchronising with the device.
_mirror = None          # the pinned tensor (kept alive here)
_mirror_addr = None     # its address; tests may point this at any int32
_armed = set()          # device indices whose status block knows the mirror


def _arm_mirror(device_index: int) -> None:
    global _mirror, _mirror_addr
    if device_index in _armed:
        return
    if _mirror is None:
        _mirror = torch.zeros(1, dtype=torch.int32).pin_memory()
        _mirror_addr = _mirror.data_ptr()
    with torch.cuda.device(device_index):
        rc = lib().bsa_set_wait_status_mirror(_mirror.data_ptr())
    if rc != 0:
        msg = lib().bsa_last_error()
        raise BsaError(f"bsa_set_wait_status_mirror failed ({rc}): {msg.decode() if msg else ''}")
    _armed.add(device_index)


def check_rc(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().bsa_last_error()
        raise BsaError(f"{what} failed ({rc}): {msg.decode() if msg else ''}")


def check(rc: int, what: str) -> None:
    """Raise on a failed call, or when a device-side wait has given up since the last
    ``wait_status()``: from then on the kernels are no-ops and outputs are undefined."""
    check_rc(rc, what)
    if _mirror_addr is not None:
        code = C.c_int32.from_address(_mirror_addr).value
        if code != 0:
            raise BsaError(
                f"{what}: a bounded device-side wait gave up earlier (code {code}); kernels launched "
                "since then did nothing and their outputs are undefined. Call "
                "dkernel_b200._lib.wait_status() to read and clear the status.")


def dtype_code(dt: torch.dtype) -> int:
    if dt == torch.float16:
        return BSA_F16
    if dt == torch.bfloat16:
        return BSA_BF16
    if dt == torch.float32:
        return BSA_F32
    raise TypeError(f"unsupported dtype {dt}: expected float16, bfloat16 or float32")


def ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def stream_of(t: torch.Tensor) -> int:
    _arm_mirror(t.device.index if t.device.index is not None else torch.cuda.current_device())
    return torch.cuda.current_stream(t.device).cuda_stream


def require_cuda(t: torch.Tensor, name: str) -> None:
    if not t.is_cuda:
        raise RuntimeError(
            f"{name} is on {t.device}: this package only computes on CUDA devices (sm_100a); "
            "there is no CPU path.")


def wait_status(reset: bool = True) -> int:
    """Synchronise and return the device wait-status word (0 = healthy)."""
    s = _i32(0)
    check_rc(lib().bsa_wait_status(C.byref(s), 1 if reset else 0), "bsa_wait_status")
    return s.value
