"""The C-ABI library loads on a machine without a GPU and exports every symbol
that include/bsa.h declares; argument validation works without a device."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    src = open(os.path.join(ROOT, "include", "bsa.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(bsa_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_are_exported_and_bound():
    from dkernel_b200 import _lib
    names = declared_symbols()
    assert "bsa_fwd" in names and "bsa_decode" in names and len(names) >= 12
    lib = C.CDLL(_lib.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/bsa.h but not exported"
    assert set(names) == set(_lib.EXPORTS), "ctypes binding table and header differ"
    assert _lib.lib().bsa_abi_version() == 3


def test_struct_layouts_match_the_header(tmp_path):
    """sizeof of every parameter struct as seen by a C compiler == ctypes layout."""
    import subprocess
    from dkernel_b200 import _lib
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include "bsa.h"\nint main(void){printf("%zu %zu %zu %zu %zu\\n",'
                   'sizeof(bsa_local_stride_params),sizeof(bsa_fwd_params),sizeof(bsa_bwd_params),'
                   'sizeof(bsa_decode_params),sizeof(bsa_xchg_params));return 0;}\n')
    exe = tmp_path / "sz"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    sizes = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    assert sizes == [C.sizeof(_lib.LocalStrideParams), C.sizeof(_lib.FwdParams), C.sizeof(_lib.BwdParams),
                     C.sizeof(_lib.DecodeParams), C.sizeof(_lib.XchgParams)]


def test_argument_validation_needs_no_device():
    from dkernel_b200 import _lib
    lib = _lib.lib()
    p = _lib.FwdParams()
    assert lib.bsa_fwd(C.byref(p), None) == -1          # null tensors
    assert b"null" in lib.bsa_last_error()
    p.q = p.k = p.v = p.o = p.crow = p.col = 16
    p.batch, p.hq, p.hkv, p.d, p.sq, p.sk = 1, 3, 2, 64, 8, 8
    assert lib.bsa_fwd(C.byref(p), None) == -1          # hq not a multiple of hkv
    assert b"multiple" in lib.bsa_last_error()
    p.hq, p.h_pat, p.block_size = 4, 3, 64
    assert lib.bsa_fwd(C.byref(p), None) == -1          # pattern heads
    p.h_pat, p.block_size = 1, 48
    assert lib.bsa_fwd(C.byref(p), None) == -1          # block size
    assert b"power of two" in lib.bsa_last_error()
    d = _lib.DecodeParams()
    assert lib.bsa_decode(C.byref(d), None) == -1
    assert lib.bsa_merge_partials(None, None, 2, 4, 8, 0, 0, 0, 0, None, 0, None, 1, None) == -1
    with pytest.raises(_lib.BsaError):
        _lib.check(-1, "x")


def test_decode_split_choice_needs_no_device():
    """bsa_decode_workspace_bytes reflects the blocks-per-CTA choice: the caller's value, or
    (<= 0) the library's: as many blocks per CTA as keep the grid about two waves deep."""
    import ctypes as C
    from dkernel_b200 import _lib
    lib = _lib.lib()
    p = _lib.DecodeParams()
    p.batch, p.hq, p.hkv, p.d, p.sk = 64, 32, 8, 128, 8192
    p.block_size, p.heads_per_cta, p.max_row_nnz = 64, 4, 30
    p.o = 16                                   # an output tensor is given (NULL = leave the partials unmerged)

    def splits():
        return lib.bsa_decode_workspace_bytes(C.byref(p)) // (4 * p.batch * p.hq * (p.d + 1))

    p.blocks_per_split = 8
    assert splits() == 4                      # ceil(30 / 8)
    p.blocks_per_split = 0
    assert splits() == 2                      # 512 (sequence, kv head) items -> 16 blocks per CTA
    p.batch = 1
    assert splits() == 8                      # few items: 4 blocks per CTA (the minimum)
    p.batch, p.max_row_nnz = 4096, 30
    assert lib.bsa_decode_workspace_bytes(C.byref(p)) // (4 * p.batch * p.hq * (p.d + 1)) == 2
    p.max_row_nnz = 12
    assert lib.bsa_decode_workspace_bytes(C.byref(p)) == 0   # one split: no workspace
    p.o = 0                                    # partials only: even one split goes to the workspace
    assert lib.bsa_decode_workspace_bytes(C.byref(p)) == 4 * p.batch * p.hq * (p.d + 1)


def test_zeroed_decode_params_are_rejected_not_divided_by():
    """The split planning divides by the head counts: a zeroed struct must come back as
    BSA_E_BADARG (0 bytes from the size query), never as a host arithmetic fault."""
    from dkernel_b200 import _lib
    lib = _lib.lib()
    d = _lib.DecodeParams()
    assert lib.bsa_decode_workspace_bytes(C.byref(d)) == 0
    assert lib.bsa_decode_workspace_bytes(None) == 0
    assert lib.bsa_decode(C.byref(d), None) == -1
    assert lib.bsa_decode_static(C.byref(d), None) == -1
    assert b"head counts" in lib.bsa_last_error()
    assert lib.bsa_decode_static(None, None) == -1
    d.hq, d.hkv, d.d = 8, 2, 128
    assert lib.bsa_decode_static(C.byref(d), None) == -1       # heads_per_cta = 0
    assert b"heads_per_cta" in lib.bsa_last_error()
    d.heads_per_cta = 3                                        # does not divide the group size 4
    assert lib.bsa_decode_workspace_bytes(C.byref(d)) == 0
    assert lib.bsa_decode(C.byref(d), None) == -1


def test_a_recorded_wait_failure_raises_on_the_next_call():
    """The kernels mirror the code of a bounded wait that gave up into a host-visible word;
    every later checked call raises until the status is cleared."""
    from dkernel_b200 import _lib
    word = C.c_int32(0)
    old = _lib._mirror_addr
    try:
        _lib._mirror_addr = C.addressof(word)
        _lib.check(0, "bsa_fwd")                               # healthy
        word.value = 423
        with pytest.raises(_lib.BsaError, match="423"):
            _lib.check(0, "bsa_fwd")
    finally:
        _lib._mirror_addr = old


def test_exchange_buffer_geometry_and_validation_need_no_device():
    """bsa_xchg_buffer_bytes: two parities x world slots of (rows, d) 16-bit rows and fp32 LSEs, every
    4 payload bytes paired with a 4-byte step word, plus a control block; 256-byte aligned regions;
    bad geometry gives 0 / BADARG."""
    from dkernel_b200 import _lib
    lib = _lib.lib()
    n = lib.bsa_xchg_buffer_bytes(8, 2048, 128)
    assert n >= 2 * 8 * 2 * (2048 * 128 * 2 + 2048 * 4) and n % 256 == 0 and n < 20 << 20
    assert lib.bsa_xchg_buffer_bytes(2, 2048, 128) < n
    assert lib.bsa_xchg_buffer_bytes(9, 16, 128) == 0          # more ranks than one node has
    assert lib.bsa_xchg_buffer_bytes(2, 16, 12) == 0           # rows must be whole 16-byte chunks
    p = _lib.XchgParams()
    assert lib.bsa_xchg_merge(C.byref(p), None) == -1
    p.world, p.rank, p.rows, p.d, p.dtype = 2, 2, 16, 128, _lib.BSA_BF16
    assert lib.bsa_xchg_merge(C.byref(p), None) == -1 and b"world/rank" in lib.bsa_last_error()
    p.rank = 1
    assert lib.bsa_xchg_merge(C.byref(p), None) == -1 and b"null" in lib.bsa_last_error()
    p.stage_o = p.stage_lse = p.out = 4096
    p.xbuf[0] = 4096
    assert lib.bsa_xchg_merge(C.byref(p), None) == -1 and b"exchange buffer 1" in lib.bsa_last_error()


def test_graft_entry_build_compiles_and_checks_the_abi():
    """The driver's build hook: both libraries compile (cached objects make this quick) and the
    ABI version it asserts is the header's."""
    import re
    import __graft_entry__
    from dkernel_b200 import _lib
    __graft_entry__.build()
    hdr = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "bsa.h")).read()
    assert int(re.search(r"#define BSA_ABI_VERSION (\d+)", hdr).group(1)) == _lib.lib().bsa_abi_version()
    from dkernel_b200 import _build
    assert os.path.exists(_build.LIB_DEBUG)
