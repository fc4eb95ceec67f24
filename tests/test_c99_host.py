"""The boundary is a C ABI for C99 hosts: the header compiles as strict C99, and a plain C
program linked against the library reproduces the golden Q4 matvec cases bit for bit."""
import os
import struct
import subprocess

import numpy as np
import pytest

from conftest import ROOT, golden, load_package

HDR_DIR = os.path.join(ROOT, "include")
SRC = os.path.join(ROOT, "tests", "c", "host_q4_matvec.c")


def test_header_is_strict_c99(tmp_path):
    src = tmp_path / "t.c"
    src.write_text('#include "salt_gpu_b200.h"\nint main(void) { return 0; }\n')
    subprocess.run(["gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-fsyntax-only",
                    "-I", HDR_DIR, str(src)], check=True)


def test_c_host_program_compiles_and_links(tmp_path):
    lib = load_package().library_path()
    exe = tmp_path / "host_q4"
    subprocess.run(["gcc", "-std=c99", "-pedantic", "-Wall", "-Wextra", "-Werror", "-I", HDR_DIR, SRC, "-o", str(exe),
                    lib, "-Wl,-rpath," + os.path.dirname(lib)], check=True)


@pytest.mark.gpu
def test_c_host_program_matches_golden(tmp_path):
    lib = load_package().library_path()
    exe = tmp_path / "host_q4"
    subprocess.run(["gcc", "-std=c99", "-I", HDR_DIR, SRC, "-o", str(exe), lib,
                    "-Wl,-rpath," + os.path.dirname(lib)], check=True)
    fx = golden("q4_matvec.npz")
    blob = bytearray()
    cases = []
    for i in range(int(fx["n_cases"])):
        R, Cc, B = (int(v) for v in fx[f"c{i}_shape"])
        vals = np.ascontiguousarray(fx[f"c{i}_vals"])
        if Cc % 8 or vals.dtype != np.uint32:      # the flat file carries whole 32-bit words only
            continue
        for t in range(B):
            cases.append((R, Cc, vals, fx[f"c{i}_scales"], fx[f"c{i}_biases"], fx[f"c{i}_x"][t], fx[f"c{i}_y"][t]))
    assert cases
    blob += struct.pack("<i", len(cases))
    for R, Cc, vals, s, b, x, y in cases:
        blob += struct.pack("<ii", R, Cc)
        for arr, dt in ((vals, np.uint32), (s, np.uint16), (b, np.uint16), (x, np.float32), (y, np.float32)):
            blob += np.ascontiguousarray(arr, dtype=dt).tobytes()
    data = tmp_path / "cases.bin"
    data.write_bytes(bytes(blob))
    out = subprocess.run([str(exe), str(data)], capture_output=True, text=True)
    assert out.returncode == 0, out.stdout + out.stderr
    assert f"{len(cases)} cases, 0 mismatches" in out.stdout
