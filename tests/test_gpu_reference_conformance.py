"""The reference's OWN GPU conformance programs (tools/test/gpu-trunk-mapped-test.c,
gpu-moe-shared-mapped-test.c, gpu-resource-binding-test.c), compiled from the reference checkout
with the reference host sources they need and linked against libsalt_gpu_b200.so in place of the
reference's backend object (recipe: oracle/Makefile, target `conformance`).  Their assertions --
CPU-vs-backend memcmp of projections and MoE steps, mapped-only accounting, stats deltas, guard
bands, defer / sync behaviour -- are the reference's, not ours."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


@pytest.mark.parametrize("program,expect", [
    ("conf-gpu-resource-binding", "gpu-resource: PASS"),
    ("conf-gpu-trunk-mapped", "gpu-trunk mapped projection: PASS"),
    ("conf-gpu-moe-shared-mapped", "gpu-moe shared mapped: PASS"),
])
def test_reference_conformance_program(program, expect):
    path = os.path.join(REF_DIR, program)
    if not os.path.exists(path):
        pytest.skip("reference conformance programs were not built (no reference checkout at build time)")
    env = dict(os.environ, SALT_REQUIRE_GPU="1")
    res = subprocess.run([path], capture_output=True, text=True, timeout=600, env=env, cwd=REF_DIR)
    out = res.stdout + res.stderr
    assert res.returncode == 0, out[-4000:]
    assert "SKIP" not in out, out[-4000:]
    assert expect in out, out[-4000:]
