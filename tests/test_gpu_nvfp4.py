"""NVFP4 activation Q/DQ and W4A4 projections through the reference operator
surface, bit/byte-exact against the CPU oracle, the golden fixtures and the
reference's own known-answer vectors."""
import numpy as np
import pytest

from conftest import assert_bits_equal, golden
from gpu_util import backend_mod, gpu

pytestmark = pytest.mark.gpu


def _resource(packed, scales, divisor, input_global):
    """One host range holding codes | scales | divisor | input scale, as a tensor
    package lays an NVFP4 tensor out (reference src/tensorops.c:104-119)."""
    pb, sb = packed.nbytes, scales.nbytes
    off_s = (pb + 15) & ~15
    off_w = (off_s + sb + 15) & ~15
    buf = np.zeros(off_w + 16, np.uint8)
    buf[:pb] = packed.ravel()
    buf[off_s:off_s + sb] = scales.ravel()
    buf[off_w:off_w + 4] = np.array([divisor], np.float32).view(np.uint8)
    buf[off_w + 4:off_w + 8] = np.array([input_global], np.float32).view(np.uint8)
    views = (buf[:pb], buf[off_s:off_s + sb], buf[off_w:off_w + 4].view(np.float32),
             buf[off_w + 4:off_w + 8].view(np.float32))
    return buf, views


def test_nvfp4_qdq_golden_and_reference_kat():
    g, fx = gpu(), golden("nvfp4.npz")
    C = fx["x"].shape[1]
    for t in range(fx["x"].shape[0]):
        packed, scales, dq = np.zeros(C // 2, np.uint8), np.zeros(C // 16, np.uint8), np.zeros(C, np.float32)
        assert g.nvfp4_qdq(fx["x"][t], float(fx["input_global"]), packed, scales, dq) == 0
        assert_bits_equal(packed, fx["qdq_packed"][t], "codes")
        assert_bits_equal(scales, fx["qdq_scales"][t], "scales")
        assert_bits_equal(dq, fx["qdq_dequant"][t], "dequant")
    # reference tests/test_nvfp4.c:56-91
    x = np.array([-6, -5, -4, -3, -2, -1.5, -1, -0.5, 0, 0.25, 0.5, 0.75, 1, 2, 4, 6,
                  -3, -2.5, -2, -1.5, -1, -0.5, 0, 0.25, 0.5, 0.75, 1, 1.5, 2, 2.5, 3, 0], np.float32)
    packed, scales, dq = np.zeros(16, np.uint8), np.zeros(2, np.uint8), np.zeros(32, np.float32)
    assert g.nvfp4_qdq(x, 64.0, packed, scales, dq) == 0
    assert packed.tolist() == [239, 222, 188, 154, 0, 33, 66, 118, 239, 222, 172, 16, 50, 84, 102, 7]
    assert scales.tolist() == [104, 96]
    # non-finite activations are rejected
    x[3] = np.inf
    assert g.nvfp4_qdq(x, 64.0, packed, scales, dq) == -1
    assert g.nvfp4_qdq(x[:8], 64.0, packed, scales, dq) == -1          # C < 16


def test_nvfp4_qdq_many_blocks_vs_oracle(orc):
    g = gpu()
    rng = np.random.default_rng(12)
    C = 5120
    x = (rng.standard_normal(C) * rng.choice([1e-3, 0.1, 1.0, 30.0], C)).astype(np.float32)
    x[100:116] = 0.0
    x[200] = 1e6
    packed, scales, dq = np.zeros(C // 2, np.uint8), np.zeros(C // 16, np.uint8), np.zeros(C, np.float32)
    assert g.nvfp4_qdq(x, 64.0, packed, scales, dq) == 0
    rc, p, s, d = orc.nvfp4_qdq(x, 64.0)
    assert rc == 0
    assert_bits_equal(packed, p, "codes")
    assert_bits_equal(scales, s, "scales")
    assert_bits_equal(dq, d, "dequant")


def test_nvfp4_qdq_every_rounding_boundary_vs_oracle(orc):
    """The device encoders are arithmetic (round to nearest even in the target format) where the reference
    searches for the nearest code (src/nvfp4.c:41-80).  Sweep every decision boundary of both: block maxima
    that put the scale on, just below and just above each midpoint of consecutive E4M3 codes (and on the codes
    themselves, the sub-normal grid, the clamp at 448), and block elements on, below and above every E2M1 tie
    point of the block's scale, both signs."""
    g = gpu()
    dec = np.array([orc.e4m3fn(c) for c in range(0x7f)], np.float64)          # the finite non-negative codes
    targets = np.concatenate([(dec[:-1] + dec[1:]) / 2, dec, [448.0, 460.0, 2.0 ** -10, 2.0 ** -11, 3e-4]])
    ties = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float64)
    blocks = []
    for ig in (1.0, 64.0):
        for tv in targets:
            base = np.float32(tv * 6.0 / ig)                                  # amax that lands the scale near tv
            for step in range(-3, 4):
                amax = base
                for _ in range(abs(step)):
                    amax = np.nextafter(amax, np.float32(np.inf if step > 0 else 0), dtype=np.float32)
                blk = np.zeros(16, np.float32)
                blk[0] = amax
                frac = (ties[(np.arange(15) + step) % ties.size] / 6.0) * np.float64(amax)
                blk[1:] = frac.astype(np.float32)
                for i in range(1, 16, 3):                                     # one ulp to either side of a tie
                    blk[i] = np.nextafter(blk[i], np.float32(0), dtype=np.float32)
                for i in range(2, 16, 3):
                    blk[i] = np.nextafter(blk[i], np.float32(np.inf), dtype=np.float32)
                blk[1::2] *= np.float32(-1.0)
                blocks.append((ig, blk))
    for ig in (1.0, 64.0):
        x = np.concatenate([b for i, b in blocks if i == ig])
        x = np.ascontiguousarray(np.concatenate([x, np.zeros((-x.size) % 256, np.float32)]))
        packed, scales, dq = np.zeros(x.size // 2, np.uint8), np.zeros(x.size // 16, np.uint8), np.zeros(x.size, np.float32)
        assert g.nvfp4_qdq(x, ig, packed, scales, dq) == 0
        rc, p, sc, d = orc.nvfp4_qdq(x, ig)
        assert rc == 0
        assert len(set(sc.tolist())) > 120                                    # the sweep reaches (nearly) every scale code
        assert_bits_equal(scales, sc, f"scales, input global {ig}")
        assert_bits_equal(packed, p, f"codes, input global {ig}")
        assert_bits_equal(dq, d, f"dequant, input global {ig}")


def test_nvfp4_matvec_golden_and_reference_kat(orc):
    g, bm, fx = gpu(), backend_mod(), golden("nvfp4.npz")
    R, C = fx["wpacked"].shape[0], fx["wpacked"].shape[1] * 2
    buf, (p, s, wg, ig) = _resource(fx["wpacked"], fx["wscale"], float(fx["divisor"]), float(fx["input_global"]))
    assert g.weight_resource_bind(bm.RESOURCE_EXPERT_LAYER, 90, buf) == 0
    assert g.nvfp4_resource_slot(bm.RESOURCE_EXPERT_LAYER, 90, 0xF4000, p, s, wg, ig, R, C) == 0
    for t in range(fx["x"].shape[0]):
        y = np.zeros(R, np.float32)
        assert g.nvfp4_matvec(0xF4000, R, C, fx["x"][t], y) == 0
        assert_bits_equal(y, fx["y"][t], f"matvec token {t}")
    ys = np.zeros((fx["x"].shape[0], R), np.float32)
    assert g.nvfp4_matvec_batch(0xF4000, R, C, np.ascontiguousarray(fx["x"]), ys) == 0
    assert_bits_equal(ys, fx["y"], "matvec batch")
    assert g.nvfp4_matvec(0xF4001, R, C, fx["x"][0], ys[0]) == -1      # unknown key
    assert g.weight_resource_unbind(bm.RESOURCE_EXPERT_LAYER, 90) == 0
    # reference tests/test_nvfp4.c:92-118: weights 0x22 / 0xa2, unit scales, golden output bits
    x = np.array([-6, -5, -4, -3, -2, -1.5, -1, -0.5, 0, 0.25, 0.5, 0.75, 1, 2, 4, 6,
                  -3, -2.5, -2, -1.5, -1, -0.5, 0, 0.25, 0.5, 0.75, 1, 1.5, 2, 2.5, 3, 0], np.float32)
    w = np.array([[0x22] * 16, [0xa2] * 16], np.uint8)
    buf, (p, s, wg, ig) = _resource(w, np.full((2, 2), 0x38, np.uint8), 1.0, 64.0)
    assert g.weight_resource_bind(bm.RESOURCE_EXPERT_LAYER, 91, buf) == 0
    assert g.nvfp4_resource_slot(bm.RESOURCE_EXPERT_LAYER, 91, 0xF4100, p, s, wg, ig, 2, 32) == 0
    y = np.zeros(2, np.float32)
    assert g.nvfp4_matvec(0xF4100, 2, 32, x, y) == 0
    assert y.view(np.uint32).tolist() == [0xc0d00000, 0xc0f00000]
    assert g.weight_resource_unbind(bm.RESOURCE_EXPERT_LAYER, 91) == 0


@pytest.mark.parametrize("shape", [(1536, 5120), (5120, 1536), (40, 256), (17, 48)])
def test_nvfp4_expert_shapes_vs_oracle(orc, synth, shape):
    g, bm = gpu(), backend_mod()
    R, C = shape
    rng = np.random.default_rng(R * 7 + C)
    packed, scales, divisor = synth.make_nvfp4(rng, R, C)
    packed[0, :4] = 0x88                                   # negative-zero codes
    buf, (p, s, wg, ig) = _resource(packed, scales, float(divisor), 64.0)
    assert g.weight_resource_bind(bm.RESOURCE_EXPERT_LAYER, 92, buf) == 0
    assert g.nvfp4_resource_slot(bm.RESOURCE_EXPERT_LAYER, 92, 0xF4200, p, s, wg, ig, R, C) == 0
    xs = rng.standard_normal((5, C)).astype(np.float32)
    ys = np.zeros((5, R), np.float32)
    assert g.nvfp4_matvec_batch(0xF4200, R, C, xs, ys) == 0
    for t in range(5):
        rc, want = orc.nvfp4_matvec(p.reshape(R, C // 2), s.reshape(R, C // 16), float(divisor), 64.0, R, C,
                                    xs[t], threads=8)
        assert rc == 0
        assert_bits_equal(ys[t], want, f"{R}x{C} token {t}")
    assert g.weight_resource_unbind(bm.RESOURCE_EXPERT_LAYER, 92) == 0
