"""The C-ABI library loads without a GPU and exports every symbol include/*.h declares."""
import ctypes
import glob
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    for path in sorted(glob.glob(os.path.join(ROOT, "include", "*.h"))):
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        text = re.sub(r"typedef struct.*?\}\s*\w+;", "", text, flags=re.S)
        names += re.findall(r"\b(arc_\w+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for must in ("arc_sdpa_prefill", "arc_sdpa_decode", "arc_sdpa_merge", "arc_sdpa_prefill_workspace_bytes",
                 "arc_sdpa_decode_workspace_bytes", "arc_mul_sigmoid_inplace", "arc_fill_causal_mask"):
        assert must in names


def test_library_loads_and_exports_every_declared_symbol():
    from arcaine_b200 import _lib
    lib = _lib.load()
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    for name in _lib.EXPORTS:
        assert name in declared_functions(), f"{name} bound in Python but not declared in include/"
    assert lib.arc_sdpa_status_string(0) == b"ok"
    assert b"128 or 256" in lib.arc_sdpa_status_string(_lib.ARC_ERR_UNSUPPORTED_HEAD_DIM)


def test_struct_layouts_match_the_header():
    """ctypes mirrors of the parameter structs have the field order of the C declarations."""
    from arcaine_b200 import _lib
    text = open(os.path.join(ROOT, "include", "arc_sdpa.h")).read()
    for cname, cls in (("arc_sdpa_prefill_params", _lib.PrefillParams), ("arc_sdpa_decode_params", _lib.DecodeParams),
                       ("arc_qkv_prepare_params", _lib.QkvPrepareParams)):
        body = re.search(r"typedef struct " + cname + r" \{(.*?)\} " + cname + ";", text, flags=re.S).group(1)
        body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
        fields = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            names = decl.replace("*", " ").split(",")
            first = names[0].split()[-1]
            fields.append(first)
            fields += [n.strip() for n in names[1:]]
        fields = [re.sub(r"\[\d+\]$", "", f) for f in fields]  # fixed-size array members
        assert fields == [f[0] for f in cls._fields_], cname


def test_no_cpu_fallback():
    """The operators refuse CPU tensors instead of computing somewhere else."""
    from arcaine_b200 import ops
    q = torch.zeros(4, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="no CPU path"):
        ops.sdpa_prefill(q, q, q, scale=1.0)
    with pytest.raises(ValueError, match="no CPU path"):
        ops.sdpa_decode(q, q, q, scale=1.0)
    with pytest.raises(ValueError, match="no CPU path"):
        ops.qkv_prepare(q, None, None)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from arcaine_b200 import _lib
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "libarc_sdpa.so"))
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _lib.load()


def test_qkv_prepare_argument_validation_needs_no_gpu():
    """Statuses that are decided before any CUDA call: an in-place K with V taken from it, parts with no
    heads, negative or too small token strides."""
    from arcaine_b200 import _lib
    lib = _lib.load()
    buf = (ctypes.c_uint16 * 4096)()
    base = ctypes.addressof(buf)
    base += (-base) % 16

    def params(**kw):
        p = _lib.QkvPrepareParams()
        p.batch, p.seq, p.nq, p.nkv, p.hd = 1, 2, 2, 1, 128
        p.q_stride_t, p.q_stride_b = 256, 512
        for name in ("k_src", "v_src", "k_dst", "v_dst"):
            setattr(p, name + "_stride_t", 128)
            setattr(p, name + "_stride_b", 256)
        p.eps, p.theta = 1e-6, 10000.0
        for k, v in kw.items():
            setattr(p, k, v)
        return p

    # V from the raw K projection while K is rewritten in place
    p = params(k_src=base, k_dst=base, v_dst=base + 2048)
    assert lib.arc_qkv_prepare(ctypes.byref(p), None) == _lib.ARC_ERR_BAD_SHAPE
    # pointers given but no heads at all: nothing to do, and no division by zero
    p = params(q=base, nq=0, nkv=0)
    assert lib.arc_qkv_prepare(ctypes.byref(p), None) == _lib.ARC_OK
    # a negative stride, and a token stride smaller than the token's heads
    p = params(q=base, q_stride_t=-256)
    assert lib.arc_qkv_prepare(ctypes.byref(p), None) == _lib.ARC_ERR_ALIGNMENT
    p = params(q=base, q_stride_t=128)
    assert lib.arc_qkv_prepare(ctypes.byref(p), None) == _lib.ARC_ERR_BAD_SHAPE


def test_ctypes_mirrors_have_the_layout_the_header_declares(tmp_path):
    """The Python mirrors of the parameter structs against the C compiler's view of include/arc_sdpa.h:
    same size, same offset for every field (a field added to one side only would shift everything behind
    it without any error at the call)."""
    import ctypes as C
    import shutil
    import subprocess
    from arcaine_b200 import _lib
    cc = shutil.which("gcc") or shutil.which("cc")
    if cc is None:
        pytest.skip("no C compiler")
    pairs = [("arc_sdpa_prefill_params", _lib.PrefillParams), ("arc_sdpa_decode_params", _lib.DecodeParams),
             ("arc_qkv_prepare_params", _lib.QkvPrepareParams), ("arc_head_shard", _lib.HeadShard)]
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "arc_sdpa.h"', 'int main(void) {']
    for cname, mirror in pairs:
        lines.append(f'  printf("{cname} %zu\\n", sizeof({cname}));')
        for fname, _ in mirror._fields_:
            lines.append(f'  printf("{cname}.{fname} %zu\\n", offsetof({cname}, {fname}));')
    lines += ['  return 0;', '}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    include = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include")
    subprocess.run([cc, "-I", include, "-o", str(exe), str(src)], check=True)
    seen = dict(line.split() for line in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.splitlines())
    for cname, mirror in pairs:
        assert int(seen[cname]) == C.sizeof(mirror), cname
        for fname, _ in mirror._fields_:
            assert int(seen[f"{cname}.{fname}"]) == getattr(mirror, fname).offset, f"{cname}.{fname}"
