"""Affine-Q4 projections through the reference operator surface, on the GPU,
bit-exact against the CPU oracle and the golden fixtures."""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_bits_equal, golden
from gpu_util import backend_mod, gpu

pytestmark = pytest.mark.gpu


def _ids(n, base=0x5000):
    return [base + 64 * i for i in range(n)]


def test_q4_matvec_golden_small_cases_arena_path():
    g, fx = gpu(), golden("q4_matvec.npz")
    g.set_mapped_only(0)
    for i in range(int(fx["n_cases"])):
        R, Cc, B = (int(v) for v in fx[f"c{i}_shape"])
        vals, s, b, x = fx[f"c{i}_vals"], fx[f"c{i}_scales"], fx[f"c{i}_biases"], fx[f"c{i}_x"]
        for t in range(B):
            y = np.zeros(R, np.float32)
            assert g.q4_matvec(vals, s, b, R, Cc, x[t], y) == 0
            assert_bits_equal(y, fx[f"c{i}_y"][t], f"case {i} {R}x{Cc} token {t}")
        ys = np.zeros((B, R), np.float32)
        assert g.proj_batch(vals, s, b, R, Cc, np.ascontiguousarray(x), ys, 0x9000 + i) == 0
        assert_bits_equal(ys, fx[f"c{i}_y"], f"case {i} proj_batch")


def test_q4_matvec_benchmark_shapes(orc, synth):
    g, fx = gpu(), golden("q4_matvec_seeded.npz")
    for name in ("cfg1_4096x4096", "gate_704x2816", "down_2816x704", "odd_705x2816"):
        R, Cc, seed = (int(v) for v in fx[name + "_meta"])
        rng = np.random.default_rng(seed)
        vals, s, b = synth.make_q4(rng, R, Cc)
        x = rng.standard_normal(Cc).astype(np.float32)
        y = np.zeros(R, np.float32)
        assert g.q4_matvec(vals, s, b, R, Cc, x, y) == 0
        assert_bits_equal(y, fx[name + "_y"], name)


@pytest.mark.parametrize("B", [1, 2, 3, 4, 5, 17, 64])
def test_q4_token_batches_match_single_vector_form(orc, synth, B):
    # reference tools/test/gemma4-bit-identity-test.c: batch == single, memcmp
    g = gpu()
    rng = np.random.default_rng(1000 + B)
    R, Cc = 705, 2816
    vals, s, b = synth.make_q4(rng, R, Cc)
    xs = rng.standard_normal((B, Cc)).astype(np.float32)
    ys = np.zeros((B, R), np.float32)
    assert g.proj_batch(vals, s, b, R, Cc, xs, ys, 0xA000 + B) == 0
    assert_bits_equal(ys, orc.q4_matvec_batch(vals, s, b, R, Cc, xs, threads=8), f"B={B}")


def test_q4_registered_resource_offsets_and_mapped_only(orc, synth):
    # tensors at odd offsets inside one described resource, as in the reference's
    # gpu-trunk-mapped-test.c (layer payloads at byte 100 and 40000 of the source)
    g = gpu()
    bm = backend_mod()
    rng = np.random.default_rng(5)
    R, Cc = 64, 64
    vb, gb = R * Cc // 2, R * Cc // 64 * 2
    src = np.zeros(70000, np.uint8)
    keys = []
    for off in (100, 40000):
        v, s, b = synth.make_q4(rng, R, Cc)
        src[off:off + vb] = v.view(np.uint8)
        src[off + vb:off + vb + gb] = s.view(np.uint8)
        src[off + vb + gb:off + vb + 2 * gb] = b.view(np.uint8)
        keys.append(off)
    assert g.weight_resource_bind(bm.RESOURCE_TRUNK, 7, src) == 0
    g.set_mapped_only(1)
    x = rng.standard_normal(Cc).astype(np.float32)
    before = g.batch_stats()
    for off in keys:
        v = src[off:off + vb].view(np.uint32)
        s = src[off + vb:off + vb + gb].view(np.uint16)
        b = src[off + vb + gb:off + vb + 2 * gb].view(np.uint16)
        assert g.weight_resource_slot(bm.RESOURCE_TRUNK, 7, 0x100 + off, v, s, b, 4, R, Cc) == 0
        y = np.zeros(R, np.float32)
        ys = [y]
        assert g.q4_batch([v], [s], [b], [x], ys, [0x100 + off], [R], Cc) == 0
        assert_bits_equal(y, orc.q4_matvec(v, s, b, R, Cc, x), f"offset {off}")
    after = g.batch_stats()
    assert after.trunk_batches == before.trunk_batches + 2
    assert after.arena_batches == before.arena_batches
    # an unregistered tensor outside every resource is a miss in mapped-only mode
    v, s, b = synth.make_q4(rng, R, Cc)
    y = np.zeros(R, np.float32)
    assert g.q4_batch([v], [s], [b], [x], [y], [0xdead0], [R], Cc) == -1
    assert g.batch_stats().mapped_only_misses == after.mapped_only_misses + 1
    g.set_mapped_only(0)
    rc, usage = g.weight_resource_usage()
    assert rc == 0 and usage.device_copied_weight_bytes >= src.nbytes and usage.active_resources >= 1
    assert g.weight_resource_unbind(bm.RESOURCE_TRUNK, 7) == 0


def test_q4_heterogeneous_batch(orc, synth):
    g = gpu()
    rng = np.random.default_rng(77)
    Cc = 704
    tensors = [synth.make_q4(rng, R, Cc) for R in (2816, 64, 100, 2816)]
    Rj = [2816, 64, 100, 2816]
    xs = [rng.standard_normal(Cc).astype(np.float32) for _ in Rj]
    ys = [np.zeros(R, np.float32) for R in Rj]
    ids = _ids(4, 0xB000)
    assert g.q4_batch([t[0] for t in tensors], [t[1] for t in tensors], [t[2] for t in tensors], xs, ys, ids,
                      Rj, Cc) == 0
    for j in range(4):
        assert_bits_equal(ys[j], orc.q4_matvec(*tensors[j], Rj[j], Cc, xs[j]), f"job {j}")


def test_q4_invalid_arguments_fail_closed(synth):
    g = gpu()
    rng = np.random.default_rng(3)
    v, s, b = synth.make_q4(rng, 64, 64)
    y = np.zeros(64, np.float32)
    x = np.zeros(64, np.float32)
    assert g.q4_matvec(v, s, b, 0, 64, x, y) == -1
    assert g.q4_matvec(v, s, b, 64, -1, x, y) == -1
    assert g.lib.salt_gpu_q4_matvec(None, None, None, 64, 64, None, None) == -1


def test_q4_results_are_bit_identical_run_to_run(synth):
    g = gpu()
    rng = np.random.default_rng(9)
    R, Cc = 704, 2816
    v, s, b = synth.make_q4(rng, R, Cc)
    xs = rng.standard_normal((6, Cc)).astype(np.float32)
    first = None
    for _ in range(3):
        ys = np.zeros((6, R), np.float32)
        assert g.proj_batch(v, s, b, R, Cc, xs, ys, 0xC000) == 0
        if first is None:
            first = ys.copy()
        assert_bits_equal(ys, first, "repeat")


def test_q8_matvec_golden_and_batch(orc):
    """Affine 8-bit router projections (reference src/kernels.c:343-369) through salt_gpu_q8_matvec and
    salt_gpu_q8_batch: golden vectors, then a two-token batch on one weight against the oracle."""
    g, fx = gpu(), golden("q8_matvec.npz")
    g.set_mapped_only(0)
    for i, (R, Cc) in enumerate(fx["shapes"]):
        R, Cc = int(R), int(Cc)
        vals, s, b, x = (np.ascontiguousarray(fx[f"c{i}_{k}"]) for k in ("vals", "scales", "biases", "x"))
        y = np.zeros(R, np.float32)
        assert g.q8_matvec(vals, s, b, R, Cc, x, y) == 0
        assert_bits_equal(y, fx[f"c{i}_y"], f"q8 matvec {R}x{Cc}")
    R, Cc = (int(v) for v in fx["shapes"][0])
    vals, s, b = (np.ascontiguousarray(fx[f"c0_{k}"]) for k in ("vals", "scales", "biases"))
    rng = np.random.default_rng(5)
    xs = [rng.standard_normal(Cc).astype(np.float32) for _ in range(2)]
    ys = [np.zeros(R, np.float32) for _ in range(2)]
    key = vals.ctypes.data
    assert g.q8_batch([vals, vals], [s, s], [b, b], xs, ys, [key, key], [R, R], Cc) == 0
    for t in range(2):
        assert_bits_equal(ys[t], orc.q8_matvec(vals, s, b, R, Cc, xs[t]), f"q8 batch token {t}")
    # router-sized (128 experts x 2816) seeded case against the oracle
    R, Cc = 128, 2816
    vals = rng.integers(0, 256, R * Cc, dtype=np.uint8)
    groups = R * Cc // 64
    s = (rng.uniform(0.001, 0.02, groups).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    b = ((-128.0 * rng.uniform(0.001, 0.02, groups)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    x = rng.standard_normal(Cc).astype(np.float32)
    y = np.zeros(R, np.float32)
    assert g.q8_matvec(vals, s, b, R, Cc, x, y) == 0
    assert_bits_equal(y, orc.q8_matvec(vals, s, b, R, Cc, x), "q8 router-sized")

