"""The C-ABI library loads and exports every symbol its header declares (no GPU needed)."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from doppler_b200 import _lib as L
from doppler_b200 import synthetic
from doppler_b200.ops import Device, DopplerError, rope_tables

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _has_gpu():
    return os.path.exists("/dev/nvidia0")


def test_header_symbols_are_exported_and_bound():
    hdr = open(os.path.join(ROOT, "include", "doppler_b200.h")).read()
    declared = set(re.findall(r"\b(dp_[a-z0-9_]+)\s*\(", hdr))
    assert len(declared) > 60
    lib = L.load()
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"
    assert declared == set(L.SIGNATURES), (declared ^ set(L.SIGNATURES))
    assert b"sm_100a" in lib.dp_version()


def test_bucket_rule():  # src/memory/buffer-pool.js:73-118
    b = L.load().dp_pool_bucket_size
    assert b(1) == 256 and b(256) == 256 and b(257) == 512 and b(1000) == 1024
    assert b(3 * 2**20 + 1) == 4 * 2**20
    assert b(64 * 2**20) == 64 * 2**20
    assert b(600 * 2**20 + 5) == 608 * 2**20  # linear 16 MiB steps above 64 MiB, not doubled


def test_no_cpu_fallback_without_device():
    if _has_gpu():
        pytest.skip("a GPU is present")
    with pytest.raises(DopplerError):
        Device(0)


def test_synthetic_streams_are_counter_based():
    k = synthetic.key(7, 3)
    whole = synthetic.q4k_blocks(k, 10)
    part = synthetic.q4k_blocks(k, 4, first_block=6)
    assert np.array_equal(whole[6 * 144:], part)
    a = synthetic.normal_f16(k, 1000)
    assert np.array_equal(a[300:400].view(np.uint16), synthetic.normal_f16(k, 100, first=300).view(np.uint16))
    x = synthetic.normal_f32(k, 200000)
    assert abs(float(x.mean())) < 0.01 and abs(float(x.std()) - 1) < 0.01
    # block statistics of the generator: 6-bit codes and nibbles uniform, d ~ |N(0,0.02)|
    blocks = synthetic.q4k_blocks(k, 4096).reshape(-1, 144)
    d = blocks[:, :2].copy().view(np.float16).astype(np.float32)
    assert 0.012 < float(d.mean()) < 0.020
    assert abs(float((blocks[:, 16:] & 15).mean()) - 7.5) < 0.05
    t = synthetic.tokens(k, 1000, 151936)
    assert t.min() >= 0 and t.max() < 151936


def test_rope_tables_match_oracle():
    from oracle import oracle as O
    c, s = rope_tables(1e6, 128, 64)
    oc, os_ = O.rope_tables(1e6, 128, 64)
    assert np.array_equal(c, oc) and np.array_equal(s, os_)


def test_header_is_plain_c_and_links(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 and as C++ without CUDA headers, and a C
    program must link against the library (it only asks for the version string: no GPU needed)."""
    import shutil
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    inc = os.path.join(root, "include")
    lib_dir = os.path.join(root, "doppler_b200")
    gcc = shutil.which("gcc", path="/usr/bin") or shutil.which("gcc")
    gxx = shutil.which("g++", path="/usr/bin") or shutil.which("g++")
    src = tmp_path / "use_abi.c"
    src.write_text('#include "doppler_b200.h"\n#include <stdio.h>\n'
                   'int main(void) { dp_matmul_opts o; dp_matmul_opts_default(&o);\n'
                   '  printf("%s %d\\n", dp_version(), (int)(o.alpha == 1.0f)); return 0; }\n')
    subprocess.run([gcc, "-std=c99", "-Wall", "-Werror", "-pedantic", "-fsyntax-only", "-I", inc, str(src)], check=True)
    cpp = tmp_path / "use_abi.cc"
    cpp.write_text('#include "doppler_b200.h"\nint main() { return dp_version() ? 0 : 1; }\n')
    subprocess.run([gxx, "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-I", inc, str(cpp)], check=True)
    exe = tmp_path / "use_abi"
    subprocess.run([gcc, "-std=c99", "-I", inc, str(src), "-o", str(exe), "-L", lib_dir, "-ldoppler_b200",
                    f"-Wl,-rpath,{lib_dir}"], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()
    assert len(out) >= 2 and out[-1] == "1"
