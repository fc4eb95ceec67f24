"""The one-launch decode expert kernel (gate | up -> GeGLU -> down for all selected experts)
against the two-launch form and the CPU oracle, bit for bit, through the C ABI."""
import numpy as np
import pytest

from conftest import assert_bits_equal
from gpu_util import oracle_stack, stack_mod

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("geom", [
    # (hidden, inter, experts, topk): the bench layer; a layer whose rows need no padding; one
    # with many small experts (all 32 groups in one round); odd multiples of 64
    (2816, 704, 128, 8), (256, 128, 32, 8), (512, 128, 32, 4), (1344, 320, 16, 2)])
@pytest.mark.parametrize("B", [1, 2, 3, 4])
def test_fused_decode_equals_two_launch_form_and_oracle(orc, synth, geom, B):
    H, M, E, K = geom
    make = synth.make_q4_moe_layer_bulk if H == 2816 else synth.make_q4_moe_layer
    layers = [make(300 + i, hidden=H, inter=M, n_experts=E, topk=K) for i in range(2)]
    x = synth.make_tokens(310 + B, B, H)
    st = stack_mod().MoeStack(4, H, M, E, K)
    for layer in layers:
        st.add_layer(layer)
    y_fused = st.forward_host(x)
    y_again = st.forward_host(x)
    assert st.set_fused_decode(False) == 0
    y_two = st.forward_host(x)
    assert st.set_fused_decode(True) == 0
    y_back = st.forward_host(x)
    want, _ = oracle_stack(orc, layers, x, threads=8)
    assert_bits_equal(y_two, want, "two-launch form vs oracle")
    assert_bits_equal(y_fused, want, "fused decode vs oracle")
    assert_bits_equal(y_again, y_fused, "fused decode, run to run")
    assert_bits_equal(y_back, y_fused, "fused decode after switching back")
    st.close()


def test_fused_decode_repeated_tokens_share_groups(orc, synth):
    """Four identical tokens select the same experts: every group holds four tokens."""
    H, M, E, K = 2816, 704, 128, 8
    layer = synth.make_q4_moe_layer_bulk(320)
    x = np.repeat(synth.make_tokens(321, 1, H), 4, axis=0)
    st = stack_mod().MoeStack(4, H, M, E, K)
    st.add_layer(layer)
    y = st.forward_host(x)
    want, _, _ = orc.moe_layer_q4(layer, x, threads=8)
    assert_bits_equal(y, want, "four tokens per group")
    st.close()


def test_fused_decode_sharded_expert_ranges(orc, synth):
    """Expert-parallel ranges: each stack runs the fused kernel on its own groups only (some
    ranges get none); the union over one shared grouped buffer equals the unsharded layer."""
    import torch
    H, M, E, K, B = 2816, 704, 128, 8, 2
    layer = synth.make_q4_moe_layer_bulk(330)
    x = synth.make_tokens(331, B, H)
    want, _, _ = orc.moe_layer_q4(layer, x, threads=8)
    sm = stack_mod()
    d_x = torch.from_numpy(x).cuda()
    shared = torch.zeros(4 * K * H, dtype=torch.float32, device="cuda")
    parts = []
    for r in range(8):
        st = sm.MoeStack(4, H, M, E, K, expert_begin=r * 16, expert_end=(r + 1) * 16)
        st.add_layer(layer)
        assert st.set_grouped_out(shared.data_ptr(), shared.numel() * 4) == 0
        assert st.layer_experts(0, d_x.data_ptr(), B) == 0
        parts.append(st)
    d_y = torch.zeros(B, H, dtype=torch.float32, device="cuda")
    assert parts[0].layer_combine(0, B, d_y.data_ptr(), apply_norm=False) == 0
    assert all(st.status() == 0 for st in parts)
    assert_bits_equal(d_y.cpu().numpy(), want, "eight ranges, fused kernel")
    for st in parts:
        st.close()


@pytest.mark.parametrize("geom", [(2816, 704, 128, 8, 5), (256, 128, 32, 8, 7), (1344, 320, 16, 2, 4)])
def test_whole_pass_in_one_launch_equals_per_layer_launches_and_oracle(orc, synth, geom):
    """One token through several layers: all layers in one launch (level 2: resident blocks, a layer ends
    with an arrival counter), one launch per layer (level 1), the phase kernels (level 0) and the CPU oracle
    agree bit for bit; so do CUDA-graph replays of the one-launch pass, and sub-ranges of the layers."""
    import torch
    H, M, E, K, L = geom
    make = synth.make_q4_moe_layer_bulk if H == 2816 else synth.make_q4_moe_layer
    layers = [make(340 + i, hidden=H, inter=M, n_experts=E, topk=K) for i in range(L)]
    x = synth.make_tokens(350, 1, H)
    st = stack_mod().MoeStack(4, H, M, E, K)
    for layer in layers:
        st.add_layer(layer)
    want, _ = oracle_stack(orc, layers, x, threads=8)
    out = {}
    for level in (2, 1, 0, 2):
        assert st.set_fused_decode(level) == 0
        out[level] = st.forward_host(x)
        assert st.status() == 0
        assert_bits_equal(out[level], want, f"level {level} vs oracle")
    # graph replays of the whole-pass launch
    stream = torch.cuda.Stream()
    sp = stream.cuda_stream
    d_x = torch.from_numpy(x).cuda()
    d_y = torch.zeros_like(d_x)
    with torch.cuda.stream(stream):
        assert st.graph_capture(d_x.data_ptr(), 1, d_y.data_ptr(), sp) == 0
        for rep in range(4):
            d_y.zero_()
            assert st.graph_launch(sp) == 0
            stream.synchronize()
            assert st.status(sp) == 0
            assert_bits_equal(d_y.cpu().numpy(), want, f"graph replay {rep}")
    # a sub-range of the layers (first = 1): the pass starts from a given row
    mid, _ = oracle_stack(orc, layers[:1], x, threads=8)
    rc, mid_n = orc.rmsnorm(mid[0], layers[0].norm_weight, layers[0].eps, True)
    assert rc == 0
    got = st.forward_host(mid_n.reshape(1, H), first=1)
    assert_bits_equal(got, want, "layers 1.. from the normalised output of layer 0")
    st.close()
