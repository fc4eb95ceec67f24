"""Prefill expert GEMMs on the tensor cores (tcgen05/TMEM), tolerance path.

Stated tolerances against the fp32 CPU oracle (the router - selected experts, weights - stays
bit-exact in both):
  split  (hi + lo fp16 operands): max |y - y_ref| / max(|y_ref|, rms(y_ref row)) <= 1e-3
  single (operands rounded once): max |y - y_ref| / max|y_ref row|               <= 1e-3"""
import numpy as np
import pytest

from conftest import assert_bits_equal
from gpu_util import d2h, stack_mod

pytestmark = pytest.mark.gpu

TOL = 1e-3


def _run_tc_layer(st, x, B, H, mode=True):
    import torch
    d_x = torch.from_numpy(x).cuda()
    d_y = torch.zeros(B, H, dtype=torch.float32, device="cuda")
    assert st.layer_experts(0, d_x.data_ptr(), B, tensor_core=mode) == 0
    assert st.layer_combine(0, B, d_y.data_ptr(), apply_norm=False) == 0
    assert st.status() == 0
    return d_y.cpu().numpy()


def _rel_err(y, ref):
    rms = np.sqrt((ref.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
    return float((np.abs(y.astype(np.float64) - ref) / np.maximum(np.abs(ref), rms)).max())


def _rel_err_rowmax(y, ref):
    top = np.abs(ref).max(axis=1, keepdims=True).astype(np.float64)
    return float((np.abs(y.astype(np.float64) - ref) / top).max())


# (hidden, inter, experts, top-k, tokens).  The fourth case: column counts that are no multiple of 256 (the
# scale tables of a tile are copied whole, an odd number of chunks per pass), tail tiles (192 = 128 + 64 fused
# rows, 320 = 256 + 64 down rows) and about 200 tokens per expert (two passes per tile).
@pytest.mark.parametrize("geom", [(256, 128, 8, 2, 64), (512, 256, 16, 4, 200), (2816, 704, 128, 8, 512),
                                  (320, 192, 4, 2, 400)])
def test_tensor_core_prefill_within_tolerance(orc, synth, geom):
    H, M, E, K, B = geom
    make = synth.make_q4_moe_layer_bulk if H == 2816 else synth.make_q4_moe_layer
    layer = make(70 + B, hidden=H, inter=M, n_experts=E, topk=K)
    x = synth.make_tokens(71 + B, B, H)
    st = stack_mod().MoeStack(B, H, M, E, K)
    st.add_layer(layer)
    y = _run_tc_layer(st, x, B, H, "split")
    want, sel, w = orc.moe_layer_q4(layer, x, threads=16)
    ws = st.workspace()
    assert_bits_equal(d2h(ws.selected, B * K, np.int32).reshape(B, K), sel, "selected (exact)")
    assert_bits_equal(d2h(ws.weights, B * K, np.float32).reshape(B, K), w, "weights (exact)")
    err = _rel_err(y, want)
    print(f"tensor-core prefill H={H} B={B}: max relative error {err:.3e}")
    assert err <= TOL, err
    y1 = _run_tc_layer(st, x, B, H, "single")
    err1, err1_rms = _rel_err_rowmax(y1, want), _rel_err(y1, want)
    print(f"  single-pass fp16: {err1:.3e} of the row maximum, {err1_rms:.3e} of max(|ref|, row rms)")
    assert err1 <= TOL, err1
    assert st.status() == 0
    st.close()


def test_tensor_core_prefill_one_table_buffer_and_refusal(orc, synth):
    """hidden = 2112 is no multiple of 256: the gate/up tables of a tile stay in shared memory, where only one
    buffer fits (33 chunks, an odd count); inter = 64 gives the down projection a single chunk per unit and
    nine row tiles (8 x 256 + 64).  The hi + lo form does not fit this hidden size and must refuse the call."""
    import torch
    H, M, E, K, B = 2112, 64, 2, 1, 40
    layer = synth.make_q4_moe_layer(91, hidden=H, inter=M, n_experts=E, topk=K)
    x = synth.make_tokens(92, B, H)
    st = stack_mod().MoeStack(B, H, M, E, K)
    st.add_layer(layer)
    d_x = torch.from_numpy(x).cuda()
    assert st.layer_experts(0, d_x.data_ptr(), B, tensor_core="split") == -1
    y1 = _run_tc_layer(st, x, B, H, "single")
    want, sel, w = orc.moe_layer_q4(layer, x, threads=16)
    ws = st.workspace()
    assert_bits_equal(d2h(ws.selected, B * K, np.int32).reshape(B, K), sel, "selected (exact)")
    err1 = _rel_err_rowmax(y1, want)
    print(f"tensor-core prefill H={H} M={M}: single-pass fp16 {err1:.3e} of the row maximum")
    assert err1 <= TOL, err1
    assert st.status() == 0
    st.close()
