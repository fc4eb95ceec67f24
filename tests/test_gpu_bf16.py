"""BF16 router / head projections behind salt_gpu_bf16_resource_slot, salt_gpu_bf16_matvec and
salt_gpu_bf16_matvec_batch (reference include/salt/gpu.h:60-66), bit for bit against the golden
vectors of the reference CPU functions and, at a router-sized shape, against the oracle."""
import numpy as np
import pytest

from conftest import assert_bits_equal, golden
from gpu_util import backend_mod, gpu

pytestmark = pytest.mark.gpu


def _bound(g, bm, rid, W):
    assert g.weight_resource_bind(bm.RESOURCE_TRUNK, rid, W) == 0
    R, Cc = W.shape
    return g.bf16_resource_slot(bm.RESOURCE_TRUNK, rid, 0x9000 + rid, W, R, Cc)


def test_bf16_matvec_and_batch_golden():
    g, bm, fx = gpu(), backend_mod(), golden("bf16_matvec.npz")
    for i, (R, Cc, B) in enumerate(fx["shapes"]):
        R, Cc, B = int(R), int(Cc), int(B)
        W = np.ascontiguousarray(fx[f"c{i}_W"])
        rc = _bound(g, bm, 40 + i, W)
        if Cc % 8 != 0:
            # the operator surface only admits column counts that are multiples of 8
            assert rc == -1
            assert g.weight_resource_unbind(bm.RESOURCE_TRUNK, 40 + i) == 0
            continue
        assert rc == 0
        xs = np.ascontiguousarray(fx[f"c{i}_xs"])
        for t in range(B):
            y = np.zeros(R, np.float32)
            assert g.bf16_matvec(0x9000 + 40 + i, R, Cc, xs[t], y) == 0
            assert_bits_equal(y, fx[f"c{i}_y"][t], f"bf16 matvec {R}x{Cc} token {t}")
        ys = np.zeros((B, R), np.float32)
        assert g.bf16_matvec_batch(0x9000 + 40 + i, R, Cc, B, xs, ys) == 0
        assert_bits_equal(ys, fx[f"c{i}_y_serial"], f"bf16 batch (serial order) {R}x{Cc}")
        # wrong geometry or an unknown key is refused
        assert g.bf16_matvec(0x9000 + 40 + i, R + 1, Cc, xs[0], np.zeros(R + 1, np.float32)) == -1
        assert g.bf16_matvec(0x7777, R, Cc, xs[0], np.zeros(R, np.float32)) == -1
        assert g.weight_resource_unbind(bm.RESOURCE_TRUNK, 40 + i) == 0
        assert g.bf16_matvec(0x9000 + 40 + i, R, Cc, xs[0], np.zeros(R, np.float32)) == -1


def test_bf16_router_sized_vs_oracle(orc):
    g, bm = gpu(), backend_mod()
    rng = np.random.default_rng(61)
    R, Cc, B = 128, 2816, 9
    W = (rng.normal(0.0, 0.02, (R, Cc)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    assert _bound(g, bm, 60, W) == 0
    xs = rng.standard_normal((B, Cc)).astype(np.float32)
    y = np.zeros(R, np.float32)
    assert g.bf16_matvec(0x9000 + 60, R, Cc, xs[0], y) == 0
    assert_bits_equal(y, orc.bf16_matvec(W, R, Cc, xs[0]), "router-sized bf16 matvec")
    ys = np.zeros((B, R), np.float32)
    assert g.bf16_matvec_batch(0x9000 + 60, R, Cc, B, xs, ys) == 0
    assert_bits_equal(ys, orc.bf16_matvec_serial(W, R, Cc, xs), "router-sized bf16 batch")
    assert g.weight_resource_unbind(bm.RESOURCE_TRUNK, 60) == 0
