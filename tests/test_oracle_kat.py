"""Known-answer vectors held by the reference project's own unit tests,
restated here as data and applied to the CPU oracle."""
import numpy as np

from conftest import assert_bits_equal


def test_q4_decode_known_vector_and_group_boundary(orc):
    # reference tests/test_kernels.c:357-392 (test 12)
    vals = np.zeros(8, np.uint32)
    for i in range(8):
        v = 0
        for j in range(8):
            v |= ((i * 8 + j) % 16) << (4 * j)
        vals[i] = v
    out = orc.q4_decode(vals, np.array([0x3F80], np.uint16), np.array([0], np.uint16), 64)
    assert (out == (np.arange(64) % 16).astype(np.float32)).all()
    v2 = np.zeros(9, np.uint32)
    v2[8] = 5
    out2 = orc.q4_decode(v2, np.array([0x3F80, 0x4000], np.uint16), np.zeros(2, np.uint16), 72)
    assert out2[64] == 10.0


def test_q4_matvec_vs_naive_ragged_columns(orc):
    # reference tests/test_kernels.c:394-451 (test 13): C=200 is a multiple of 8
    # but not of 64, so rows straddle quantisation groups.  Tolerance as there.
    R, C = 8, 200
    rng = np.random.default_rng(13)
    n = R * C
    q = rng.integers(0, 16, n)
    vals = np.zeros((n + 7) // 8, np.uint32)
    for i in range(n):
        vals[i >> 3] |= np.uint32(int(q[i]) << (4 * (i & 7)))
    ng = (n + 63) // 64
    scales = rng.integers(0, 20000, ng).astype(np.uint16)
    biases = rng.integers(0, 20000, ng).astype(np.uint16)
    x = (rng.integers(0, 200, C) / 100.0 - 1.0).astype(np.float32)
    s = (scales.astype(np.uint32) << 16).view(np.float32)
    b = (biases.astype(np.uint32) << 16).view(np.float32)
    want = np.zeros(R, np.float32)
    for r in range(R):
        acc = np.float32(0)
        for c in range(C):
            k = r * C + c
            acc = np.float32(acc + np.float32(np.float32(np.float32(q[k]) * s[k // 64]) + b[k // 64]) * x[c])
        want[r] = acc
    got = orc.q4_matvec(vals, scales, biases, R, C, x)
    assert (np.abs(got - want) <= 1e-3 * (1 + np.abs(want))).all()


def test_q4_word_map_from_unaligned_source(orc):
    # reference tests/test_kernels.c:453-478 (test 14): y == 120 exactly, the
    # four packed words sit on a 4-byte but not 16-byte boundary.
    raw = np.zeros(64, np.uint8)
    base = raw.ctypes.data
    off = (4 - (base & 15)) & 15
    if off == 0:
        off = 4
    words = raw[off:off + 16].view(np.uint32)
    words[:] = [0x11111111, 0x22222222, 0x44444444, 0x88888888]
    y = orc.q4_matvec(words, np.array([0x3F80], np.uint16), np.array([0], np.uint16), 1, 32,
                      np.ones(32, np.float32))
    assert y[0] == 120.0


def test_q4_byte_unaligned_payloads(orc):
    # reference tests/test_kernels.c:480-521 (test 15): payloads at odd addresses
    import ctypes as C
    vs = np.zeros(48, np.uint8); ss = np.zeros(8, np.uint8); bs = np.zeros(8, np.uint8)
    voff = (1 - (vs.ctypes.data & 3)) & 3
    soff = (1 - (ss.ctypes.data & 1)) & 1
    boff = (1 - (bs.ctypes.data & 1)) & 1
    vs[voff:voff + 32] = 0x11
    ss[soff:soff + 2] = np.array([0x3f80], np.uint16).view(np.uint8)
    x = np.ones(64, np.float32)
    y = np.zeros(1, np.float32)
    rc = orc.lib.orc_q4_matvec(C.c_void_p(vs.ctypes.data + voff), C.c_void_p(ss.ctypes.data + soff),
                               C.c_void_p(bs.ctypes.data + boff), 1, 64,
                               x.ctypes.data_as(C.c_void_p), y.ctypes.data_as(C.c_void_p), 1)
    assert rc == 0 and y[0] == 64.0


def test_q4_c8192_group_boundary(orc):
    # reference tests/test_kernels.c:523-558 (test 16): 128 groups per row
    R, C = 2, 8192
    vals = np.full(R * C // 8, 0x11111111, np.uint32)
    scales = np.full(R * C // 64, 0x3f80, np.uint16)
    biases = np.zeros(R * C // 64, np.uint16)
    x = (((np.arange(C) * 11) % 29 - 14).astype(np.float32) * np.float32(0.001))
    y = orc.q4_matvec(vals, scales, biases, R, C, x)
    want = np.float32(0)
    acc = np.zeros(32, np.float32)
    for c in range(C):
        acc[c & 31] = np.float32(acc[c & 31] + x[c])
    lane = np.zeros(4, np.float32)
    for a in range(8):
        for j in range(4):
            lane[j] = np.float32(lane[j] + acc[4 * a + j])
    want = np.float32(np.float32(lane[0] + lane[2]) + np.float32(lane[1] + lane[3]))
    assert_bits_equal(y, np.array([want, want], np.float32), "C=8192")


def test_router_scores_vs_naive(orc):
    # reference tests/test_kernels.c:139-161 (test 5)
    E, H = 5, 12
    W = (((np.arange(E * H) * 3 + 1) % 50 - 25).astype(np.float32) * np.float32(0.1)).reshape(E, H)
    bias = np.arange(E, dtype=np.float32) * np.float32(0.5)
    x = ((np.arange(H) % 5 - 2).astype(np.float32) * np.float32(0.25))
    got = orc.router_scores(W, bias, x)
    want = bias + (W.astype(np.float64) @ x.astype(np.float64))
    assert np.abs(got - want).max() <= 1e-4


def test_route_group_golden(orc):
    # reference tests/test_text_verify.c:1234-1312
    selected = np.array([2, 0, 2, 1, 0, 2], np.int32)
    rows = np.array([[1, 2, 3], [4, 5, 6], [7, 8, 9]], np.float32)
    rc, offs, g2c, c2g, routed = orc.route_group(selected, 3, 2, 4, rows)
    assert rc == 0
    assert g2c.tolist() == [1, 4, 3, 0, 2, 5]
    assert c2g.tolist() == [3, 0, 4, 2, 1, 5]
    assert routed.tolist() == [[1, 2, 3], [7, 8, 9], [4, 5, 6], [1, 2, 3], [4, 5, 6], [7, 8, 9]]
    weights = np.array([0.6, 0.4, 0.25, 0.75, 0.3, 0.7], np.float32)
    gout = (np.arange(6)[:, None] * 10 + 10 + np.arange(3)[None, :]).astype(np.float32)
    rc, red = orc.weighted_reduce(weights, c2g, gout, 3, 2)
    assert rc == 0
    want = np.zeros((3, 3), np.float32)
    for r in range(3):
        for k in range(2):
            want[r] = want[r] + weights[r * 2 + k] * gout[c2g[r * 2 + k]]
    assert_bits_equal(red, want, "weighted reduce")


def test_nvfp4_known_answers(orc):
    # reference tests/test_nvfp4.c:28-118
    pos = [0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]
    for i, v in enumerate(pos):
        assert orc.e2m1(i) == v and orc.e2m1(i | 8) == -v
    assert orc.e4m3fn(0x38) == 1.0 and orc.e4m3fn(0x68) == 64.0
    assert orc.e4m3fn(0x7e) == 448.0 and orc.e4m3fn(0xfe) == -448.0
    assert np.isnan(orc.e4m3fn(0x7f))
    assert orc.e4m3fn_encode(64.0) == (0, 0x68)
    assert orc.e4m3fn_encode(448.0) == (0, 0x7e)
    assert orc.e4m3fn_encode(-448.0) == (0, 0xfe)
    x = np.array([-6, -5, -4, -3, -2, -1.5, -1, -0.5, 0, 0.25, 0.5, 0.75, 1, 2, 4, 6,
                  -3, -2.5, -2, -1.5, -1, -0.5, 0, 0.25, 0.5, 0.75, 1, 1.5, 2, 2.5, 3, 0], np.float32)
    rc, packed, scales, dq = orc.nvfp4_qdq(x, 64.0)
    assert rc == 0
    assert packed.tolist() == [239, 222, 188, 154, 0, 33, 66, 118, 239, 222, 172, 16, 50, 84, 102, 7]
    assert scales.tolist() == [104, 96]
    want_bits = [0xc0c00000, 0xc0800000, 0xc0800000, 0xc0400000, 0xc0000000, 0xbfc00000, 0xbf800000,
                 0xbf000000, 0, 0, 0x3f000000, 0x3f800000, 0x3f800000, 0x40000000, 0x40800000,
                 0x40c00000, 0xc0400000, 0xc0000000, 0xc0000000, 0xbfc00000, 0xbf800000, 0xbf000000,
                 0, 0x3e800000, 0x3f000000, 0x3f400000, 0x3f800000, 0x3fc00000, 0x40000000,
                 0x40000000, 0x40400000, 0]
    assert dq.view(np.uint32).tolist() == want_bits
    weights = np.array([0x22] * 16 + [0xa2] * 16, np.uint8)
    rc, y = orc.nvfp4_matvec(weights, np.array([0x38] * 4, np.uint8), 1.0, 64.0, 2, 32, x)
    assert rc == 0
    assert y.view(np.uint32).tolist() == [0xc0d00000, 0xc0f00000]


def test_synthetic_nvfp4_encoders_agree_with_the_search_based_reference_form(orc, synth):
    """synth's arithmetic E4M3 / E2M1 encoders (also used inside the CUDA kernels)
    against the oracle's nearest-code searches, including every midpoint."""
    dec = [orc.e4m3fn(c) for c in range(0x7f)]
    vals = [np.float32(0), np.float32(448), np.float32(1000), np.float32(1e-10)]
    for c in range(0x7e):
        m = np.float32((np.float64(dec[c]) + np.float64(dec[c + 1])) / 2)
        vals += [m, np.nextafter(m, np.float32(0)), np.nextafter(m, np.float32(1e9)), np.float32(dec[c])]
    vals = np.array(vals, np.float32)
    want = np.array([orc.e4m3fn_encode(float(v))[1] for v in vals], np.uint8)
    assert (synth.e4m3fn_encode(vals) == want).all()
    assert (synth.e4m3fn_decode(np.arange(0x7f, dtype=np.uint8)) == np.array(dec, np.float32)).all()
    # E2M1: drive the oracle's encoder through the activation Q/DQ with scale exactly 1
    t = np.array([0, 0.25, 0.26, 0.5, 0.75, 1.0, 1.25, 1.3, 1.75, 2.0, 2.5, 2.6, 3.5, 4.0, 5.0, 6.0], np.float32)
    for sign in (1.0, -1.0):
        x = (t * np.float32(sign)).astype(np.float32)
        rc, packed, scales, _ = orc.nvfp4_qdq(x, 1.0)       # amax 6 -> scale code 0x38 (1.0)
        assert rc == 0 and scales[0] == 0x38
        codes = np.stack([packed & 15, packed >> 4], axis=1).ravel()
        assert (synth.e2m1_encode(x) == codes).all()
