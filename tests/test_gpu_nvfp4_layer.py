"""MoE layers with NVFP4 experts as a device sequence (salt_b200_stack_add_nvfp4_layer): router, grouping,
activation quantise-dequantise, W4A4 gate / up, GeGLU, W4A4 down, ordered reduce -- bit for bit against
the golden vectors of the reference's own functions and against the oracle composition."""
import numpy as np
import pytest

import oracle
from conftest import assert_bits_equal, golden
from gpu_util import d2h, stack_mod

pytestmark = pytest.mark.gpu


def test_nvfp4_layer_small_golden(synth):
    fx = golden("moe_layer_nvfp4_small.npz")
    lseed, xseed, B, H, M, E, K = (int(v) for v in fx["meta"])
    layer = synth.make_nvfp4_moe_layer(lseed, hidden=H, inter=M, n_experts=E, topk=K)
    x = synth.make_tokens(xseed, B, H)
    st = stack_mod().MoeStack(8, H, M, E, K)
    st.add_nvfp4_layer(layer)
    y = st.forward_host(x)
    ws = st.workspace()
    assert_bits_equal(d2h(ws.selected, B * K, np.int32).reshape(B, K), fx["sel"], "selected")
    assert_bits_equal(d2h(ws.weights, B * K, np.float32).reshape(B, K), fx["w"], "weights")
    assert_bits_equal(y, fx["y"], "nvfp4 layer output")
    assert_bits_equal(st.forward_host(x), y, "run to run")
    st.close()


@pytest.mark.parametrize("B", [1, 5])
def test_nvfp4_cfg4_layer_vs_oracle(orc, synth, B):
    """Config 4 of the baseline: 64 experts, hidden 5120, intermediate 1536, top-4."""
    layer = synth.make_nvfp4_moe_layer(4410)
    x = synth.make_tokens(4411 + B, B, layer.hidden)
    st = stack_mod().MoeStack(8, layer.hidden, layer.inter, layer.n_experts, layer.topk)
    st.add_nvfp4_layer(layer)
    y = st.forward_host(x)
    want, sel, w = oracle.moe_layer_nvfp4(orc, layer, x, threads=8)
    ws = st.workspace()
    assert_bits_equal(d2h(ws.selected, B * 4, np.int32).reshape(B, 4), sel, "selected")
    assert_bits_equal(d2h(ws.weights, B * 4, np.float32).reshape(B, 4), w, "weights")
    assert_bits_equal(y, want, f"cfg4 nvfp4 layer B={B}")
    st.close()


def test_nvfp4_two_layers_with_rmsnorm_and_expert_ranges(orc, synth):
    """Two stacked NVFP4 layers (RMSNorm between them), and the same first layer cut into two expert
    ranges over one shared grouped buffer."""
    import torch
    H, M, E, K, B = 512, 256, 8, 2, 6
    layers = [synth.make_nvfp4_moe_layer(4420 + i, hidden=H, inter=M, n_experts=E, topk=K) for i in range(2)]
    x = synth.make_tokens(4423, B, H)
    sm = stack_mod()
    st = sm.MoeStack(8, H, M, E, K)
    for layer in layers:
        st.add_nvfp4_layer(layer)
    y = st.forward_host(x)
    y0, _, _ = oracle.moe_layer_nvfp4(orc, layers[0], x)
    mid = np.stack([orc.rmsnorm(y0[t], layers[0].norm_weight, layers[0].eps, True)[1] for t in range(B)])
    want, _, _ = oracle.moe_layer_nvfp4(orc, layers[1], mid)
    assert_bits_equal(y, want, "two nvfp4 layers")
    st.close()
    d_x = torch.from_numpy(x).cuda()
    shared = torch.zeros(8 * K * H, dtype=torch.float32, device="cuda")
    halves = []
    for lo, hi in ((0, 4), (4, 8)):
        h = sm.MoeStack(8, H, M, E, K, expert_begin=lo, expert_end=hi)
        h.add_nvfp4_layer(layers[0])
        assert h.set_grouped_out(shared.data_ptr(), shared.numel() * 4) == 0
        assert h.layer_experts(0, d_x.data_ptr(), B) == 0
        halves.append(h)
    d_y = torch.zeros(B, H, dtype=torch.float32, device="cuda")
    assert halves[0].layer_combine(0, B, d_y.data_ptr(), apply_norm=False) == 0
    assert all(h.status() == 0 for h in halves)
    assert_bits_equal(d_y.cpu().numpy(), y0, "two expert ranges, nvfp4")
    for h in halves:
        h.close()
