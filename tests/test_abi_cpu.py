"""The C-ABI library loads without a GPU and exports exactly what
include/backend_cuda.h declares; without a device it fails loudly."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    src = open(os.path.join(ROOT, "include", "backend_cuda.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    names = set(re.findall(r"\b(apus_(?:cuda|synth)_\w+)\s*\(", src))
    names |= set(re.findall(r"extern\s+\w+\s+(apus_cuda_\w+)\s*;", src))
    return names


def test_every_declared_symbol_is_exported(be, pkg):
    import apus_b200.backend as b
    hs = header_symbols()
    assert hs == set(b.SYMBOLS), hs ^ set(b.SYMBOLS)
    for s in hs:
        assert hasattr(be.lib, s), s


def test_header_is_c11(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "backend_cuda.h"\nint main(void){'
                   'ApusCudaMoeCfg c = {0}; (void)c; return 0;}\n')
    import subprocess
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Wextra", "-Werror",
                    "-pedantic", "-I", os.path.join(ROOT, "include"), "-c",
                    str(src), "-o", str(tmp_path / "t.o")], check=True)


def test_no_device_fails_loudly(be):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    import numpy as np
    with pytest.raises(Exception):
        be.enable()
    assert not be.is_enabled()
    w = np.zeros((4, 8), np.uint16)
    with pytest.raises(Exception):
        be.bf16_gemv(w, np.zeros(8, np.uint16))
    # zero dimensions are "unsupported" (c/backend_metal.mm:323)
    assert be.lib.apus_cuda_bf16_gemv(None, None, None, 0, 8) != 0


def test_product_does_not_reach_for_the_oracle():
    """The package never imports or links anything under oracle/."""
    pk = os.path.join(ROOT, "apus-qwen3.6-35b-a3b_b200")
    for dp, _, fs in os.walk(pk):
        for f in fs:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                s = open(os.path.join(dp, f)).read()
                assert "oracle" not in s.lower().replace("numpy oracle", ""), f
