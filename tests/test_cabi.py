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
    assert _lib.lib().bsa_abi_version() == 1


def test_struct_layouts_match_the_header(tmp_path):
    """sizeof of every parameter struct as seen by a C compiler == ctypes layout."""
    import subprocess
    from dkernel_b200 import _lib
    src = tmp_path / "sz.c"
    src.write_text('#include <stdio.h>\n#include "bsa.h"\nint main(void){printf("%zu %zu %zu %zu\\n",'
                   'sizeof(bsa_local_stride_params),sizeof(bsa_fwd_params),sizeof(bsa_bwd_params),'
                   'sizeof(bsa_decode_params));return 0;}\n')
    exe = tmp_path / "sz"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    sizes = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    assert sizes == [C.sizeof(_lib.LocalStrideParams), C.sizeof(_lib.FwdParams), C.sizeof(_lib.BwdParams),
                     C.sizeof(_lib.DecodeParams)]


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
