"""The C-ABI library loads on a machine without a GPU and exports every symbol include/rswa.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "rswa.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rswa_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported_and_bound():
    from ring_swa import _C
    lib = _C.lib()
    declared = _declared_symbols()
    assert "rswa_fwd" in declared and "rswa_bwd" in declared and "rswa_merge" in declared
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in rswa.h but not exported"
        assert name in _C.SYMBOLS, f"{name} has no ctypes signature in ring_swa/_C.py"
    assert sorted(_C.SYMBOLS) == declared
    assert lib.rswa_abi_version() == 1


def test_struct_sizes_match_the_header():
    """ctypes mirrors must have the C layout: compile a tiny program against the header and compare."""
    import subprocess
    import tempfile
    from ring_swa import _C
    src = r'''
#include <stdio.h>
#include "rswa.h"
int main(void) {
  printf("%zu %zu %zu %zu %zu %zu\n", sizeof(rswa_span_t), sizeof(rswa_geom_t), sizeof(rswa_fwd_params_t),
         sizeof(rswa_bwd_params_t), sizeof(rswa_merge_params_t), sizeof(rswa_merge_acc_params_t));
  return 0;
}
'''
    with tempfile.TemporaryDirectory() as tmp:
        c = os.path.join(tmp, "s.c")
        open(c, "w").write(src)
        exe = os.path.join(tmp, "s")
        subprocess.run(["gcc", "-I", os.path.join(ROOT, "include"), c, "-o", exe], check=True)
        sizes = [int(x) for x in subprocess.run([exe], capture_output=True, text=True, check=True).stdout.split()]
    assert sizes == [ctypes.sizeof(_C.Span), ctypes.sizeof(_C.Geom), ctypes.sizeof(_C.FwdParams),
                     ctypes.sizeof(_C.BwdParams), ctypes.sizeof(_C.MergeParams), ctypes.sizeof(_C.MergeAccParams)]


def test_argument_rejection_without_a_gpu():
    from ring_swa import _C
    lib = _C.lib()
    assert lib.rswa_fwd(None, None) == -1
    assert b"null" in lib.rswa_last_error()
    p = _C.FwdParams()
    p.g.dtype, p.g.head_dim = 0, 64
    assert lib.rswa_fwd(ctypes.byref(p), None) == -2          # unsupported head_dim
    assert b"head_dim" in lib.rswa_last_error()
    # two fp32 rows (delta, scaled lse) per batch row and head, padded to whole 128-query tiles
    assert lib.rswa_bwd_workspace_bytes(1, 130, 2, 128) == 2 * (2 * 256 * 4) + 256     # + the dQ work counter
    assert lib.rswa_bwd_workspace_bytes(1, 128, 2, 64) == -1
    assert lib.rswa_merge_acc(None, None) == -1
    m = _C.MergeAccParams()
    m.acc_o = m.new_o = m.acc_lse = m.new_lse = 16
    m.new_dtype = 7
    assert lib.rswa_merge_acc(ctypes.byref(m), None) == -2      # unknown dtype of the incoming output
    with pytest.raises(ValueError):
        _C.check(-1, "x")
    with pytest.raises(RuntimeError):
        _C.check(-3, "x")


def test_product_has_no_cpu_path():
    import torch
    import ring_swa
    q = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ring_swa.ring_sliding_window_attn(q, q, q, 10)
