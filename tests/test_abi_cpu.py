"""The C-ABI library loads without a GPU, exports every symbol the header declares, agrees
with the ctypes mirror on struct layout, and rejects bad arguments before touching the device."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

from pope_pytorch_b200 import _native as N
from pope_pytorch_b200 import build as B

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "pope_b200.h")


@pytest.fixture(scope="module")
def lib():
    B.build()
    return N.load_library()


def declared_symbols():
    text = open(HEADER).read()
    return re.findall(r"POPE_API\s+[\w\s\*]+?\b(pope_b200_\w+)\s*\(", text)


def test_exports_match_header(lib):
    names = declared_symbols()
    assert set(N.EXPORTS) <= set(names) and len(names) >= 8
    for name in names:
        assert hasattr(lib, name), f"{name} declared in the header but not exported"
    assert lib.pope_b200_abi_version() == N.ABI_VERSION
    assert lib.pope_b200_status_str(0) == b"ok"
    assert b"workspace" in lib.pope_b200_status_str(-4)


def test_struct_layout_matches_c(tmp_path):
    fields = {
        "PopeSimArgs": (N.SimArgs, ["shape", "embed", "q", "sim", "ss", "workspace", "workspace_bytes"]),
        "PopeSimBwdArgs": (N.SimBwdArgs, ["dsim", "dq", "dfreqs", "dbias_stride_h", "workspace", "workspace_bytes"]),
        "PopeAttnArgs": (N.AttnArgs, ["softmax_scale", "shape", "embed", "v", "lse", "mask", "workspace_bytes"]),
        "PopeAttnBwdArgs": (N.AttnBwdArgs, ["dout", "lse", "mask_stride_n", "dq", "dv", "dfreqs", "dbias", "workspace"]),
        "PopeApplyArgs": (N.ApplyArgs, ["shape", "embed", "q", "k", "q_out", "sqo", "k_out", "sko"]),
        "PopeApplyBwdArgs": (N.ApplyBwdArgs, ["dq_out", "dk_out", "dq", "dk", "dfreqs", "dbias", "dbias_stride_h"]),
        "PopePagedKV": (N.PagedKV, ["k_pages", "v_pages", "page_table", "seq_lens", "num_pages", "page_size", "max_pages_per_seq"]),
        "PopeKvAppendArgs": (N.KvAppendArgs, ["dtype", "B", "n_new", "advance", "kv", "k", "sk", "v", "sv"]),
        "PopePagedDecodeArgs": (N.PagedDecodeArgs, ["softmax_scale", "shape", "embed", "kv", "q", "out", "so", "lse", "workspace_bytes"]),
    }
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void){"]
    for cname, (_, fl) in fields.items():
        lines.append(f'printf("{cname} %zu\\n", sizeof({cname}));')
        for f in fl:
            lines.append(f'printf("{cname}.{f} %zu\\n", offsetof({cname}, {f}));')
    lines.append("return 0;}")
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", str(src), "-o", str(exe)], check=True)
    got = dict(l.split() for l in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.splitlines())
    for cname, (ct, fl) in fields.items():
        assert int(got[cname]) == C.sizeof(ct), cname
        for f in fl:
            assert int(got[f"{cname}.{f}"]) == getattr(ct, f).offset, f"{cname}.{f}"


def _attn_args(**over):
    shape = dict(B=1, H=2, Hk=2, Nq=4, Nk=4, d=32, r=16, dtype=1)
    shape.update(over)
    a = N.AttnArgs()
    a.struct_bytes = C.sizeof(N.AttnArgs)
    a.shape = N.Shape(*[shape[k] for k in ("B", "H", "Hk", "Nq", "Nk", "d", "r", "dtype")])
    return a


def test_bad_arguments_are_rejected_without_a_device(lib):
    bad = -1
    assert lib.pope_b200_attn_fwd(None, None) == bad
    a = _attn_args()
    a.struct_bytes = 8
    assert lib.pope_b200_attn_fwd(C.addressof(a), None) == bad          # wrong struct size
    for over in (dict(Nq=8), dict(r=64), dict(H=3), dict(B=0), dict(dtype=7)):
        a = _attn_args(**over)
        assert lib.pope_b200_attn_fwd(C.addressof(a), None) == bad, over
    a = _attn_args()                                                     # valid shape, null tensors
    assert lib.pope_b200_attn_fwd(C.addressof(a), None) == bad
    s = N.SimArgs()
    s.struct_bytes = C.sizeof(N.SimArgs)
    s.shape = N.Shape(1, 2, 2, 4, 4, 32, 16, 0)
    assert lib.pope_b200_sim_fwd(C.addressof(s), None) == bad            # r > 0 without freqs
    assert lib.pope_b200_sim_bwd(None, None) == bad and lib.pope_b200_attn_bwd(None, None) == bad


def test_paged_cache_arguments_are_checked_without_a_device(lib):
    bad, unsupported = -1, -2
    assert lib.pope_b200_kv_append(None, None) == bad and lib.pope_b200_attn_decode_paged(None, None) == bad
    k = N.KvAppendArgs()
    k.struct_bytes = C.sizeof(N.KvAppendArgs)
    k.dtype, k.B, k.Hk, k.d, k.n_new = 1, 2, 2, 64, 4
    assert lib.pope_b200_kv_append(C.addressof(k), None) == bad            # null tensors
    buf = (C.c_char * 4096)()
    ptr = (C.addressof(buf) + 255) & ~255
    k.k, k.v = ptr, ptr
    k.sk = k.sv = N.Stride3(512, 256, 64)
    assert lib.pope_b200_kv_append(C.addressof(k), None) == bad            # no cache
    k.kv = N.PagedKV(ptr, ptr, ptr, ptr, 4, 100, 2, 0)
    assert lib.pope_b200_kv_append(C.addressof(k), None) == unsupported    # page size not a multiple of 64
    k.kv = N.PagedKV(ptr, ptr, ptr, ptr, 4, 128, 2, 0)
    k.dtype = 0
    assert lib.pope_b200_kv_append(C.addressof(k), None) == unsupported    # fp32 cache
    k.dtype, k.sk = 1, N.Stride3(512, 256, 60)
    assert lib.pope_b200_kv_append(C.addressof(k), None) == -3             # rows off 16-byte boundaries
    d = N.PagedDecodeArgs()
    d.struct_bytes = C.sizeof(N.PagedDecodeArgs)
    d.shape = N.Shape(2, 4, 2, 1, 4096, 128, 0, 1)
    d.kv = N.PagedKV(ptr, ptr, ptr, ptr, 64, 256, 16, 0)
    assert lib.pope_b200_workspace_bytes(N.OP_DECODE_PAGED, C.addressof(d)) > 0
    assert lib.pope_b200_attn_decode_paged(C.addressof(d), None) == bad    # no q / out
    d.q, d.out = ptr, ptr
    assert lib.pope_b200_attn_decode_paged(C.addressof(d), None) == -4     # no workspace
    d.shape = N.Shape(2, 4, 2, 1, 4096, 80, 0, 1)
    assert lib.pope_b200_attn_decode_paged(C.addressof(d), None) == unsupported


def test_workspace_query_needs_no_device(lib):
    a = _attn_args(B=1, H=1, Hk=1, Nq=1, Nk=32768, d=128, r=64)
    assert lib.pope_b200_workspace_bytes(N.OP_ATTN_FWD, C.addressof(a)) > 0    # decode splits the keys
    b = N.AttnBwdArgs()
    b.struct_bytes = C.sizeof(N.AttnBwdArgs)
    b.shape = N.Shape(2, 4, 4, 64, 64, 64, 32, 1)
    assert lib.pope_b200_workspace_bytes(N.OP_ATTN_BWD, C.addressof(b)) >= 2 * 4 * 64 * 4
    assert lib.pope_b200_workspace_bytes(99, C.addressof(a)) == 0


def test_cuda_call_without_library_or_device_raises():
    import torch
    from pope_pytorch_b200 import flash_attn_with_pope
    q = torch.randn(1, 2, 4, 32)
    with pytest.raises(RuntimeError):
        flash_attn_with_pope(q, q, q, pos_emb=(torch.rand(4, 16), torch.zeros(2, 16)), fused=True)
