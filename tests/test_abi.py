"""CPU-only checks of the drop-in boundary: the library loads, exports every symbol the header
declares, the ctypes structs match the C layout, and it fails loudly without a GPU."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def native():
    from ctox_llm_b200 import _native
    _native.load()
    return _native


def declared_functions():
    text = open(os.path.join(ROOT, "include", "ctox_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ctox_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(native):
    lib = native.load()
    names = declared_functions()
    assert len(names) >= 15
    for name in names:
        assert hasattr(lib, name), f"{name} declared in ctox_b200.h but not exported"
        assert name in native.SIGNATURES, f"{name} has no ctypes signature"
    for name in native.SIGNATURES:
        assert name in names, f"{name} bound but not declared in the header"


def test_struct_layouts_match_the_header(native, tmp_path):
    """Offsets as the C compiler sees them (gcc on include/ctox_b200.h) equal the ctypes ones."""
    import subprocess
    fields = [f[0] for f in native.FusedMatVecOp._fields_]
    seg_fields = [f[0] for f in native.Segment._fields_]
    src = ['#include <stdio.h>', '#include <stddef.h>', '#include "ctox_b200.h"', 'int main(void){',
           'printf("%zu\\n", sizeof(ctox_fused_matvec_op));']
    src += [f'printf("%zu\\n", offsetof(ctox_fused_matvec_op, {f}));' for f in fields]
    src += ['printf("%zu\\n", sizeof(ctox_segment));']
    src += [f'printf("%zu\\n", offsetof(ctox_segment, {f}));' for f in seg_fields]
    src += ['return 0;}']
    c = tmp_path / "layout.c"
    c.write_text("\n".join(src))
    exe = tmp_path / "layout"
    subprocess.check_call(["gcc", "-I", os.path.join(ROOT, "include"), str(c), "-o", str(exe)])
    out = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    assert out[0] == C.sizeof(native.FusedMatVecOp)
    assert out[1:1 + len(fields)] == [getattr(native.FusedMatVecOp, f).offset for f in fields]
    rest = out[1 + len(fields):]
    assert rest[0] == C.sizeof(native.Segment) == 40
    assert rest[1:] == [getattr(native.Segment, f).offset for f in seg_fields]


def test_abi_identity(native):
    lib = native.load()
    assert lib.ctox_abi_version() == 1
    assert lib.ctox_backend_profile() == b"cuda-sm100a-b200"


def test_no_cpu_fallback_without_a_device(native):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    import ctox_llm_b200 as ctox
    with pytest.raises(ctox.CtoxError) as e:
        ctox.B200Backend()
    assert e.value.kind == "UnsupportedOperation"
    assert "no CPU fallback" in str(e.value)


def test_product_package_does_not_import_the_oracle():
    import subprocess
    import sys
    code = ("import sys; sys.path.insert(0, %r); import ctox_llm_b200; "
            "assert not any(m == 'oracle' or m.startswith('oracle.') for m in sys.modules)" % ROOT)
    subprocess.check_call([sys.executable, "-c", code])
    for dirpath, _, files in os.walk(os.path.join(ROOT, "ctox_llm_b200")):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp")):
                text = open(os.path.join(dirpath, f)).read()
                assert "import oracle" not in text and "from oracle" not in text, f
                assert "ctox_oracle" not in text, f
