"""NVFP4 expert projections on the tensor cores (block-scaled tcgen05.mma.kind::mxf4nvf4), tolerance path.

Stated tolerance against the exact path (the CPU oracle composition at the small sizes, the bit-exact GPU
kernels - themselves pinned to the oracle - at config-4 size): max |y - y_ref| / max(|y_ref|, rms(y_ref row))
<= 1e-3.  Router, top-k and grouping stay bit-exact; the activation codes and block scales are the
bit-exact quantiser's, so only the order of the fp32 additions differs."""
import numpy as np
import pytest

import oracle
from conftest import assert_bits_equal
from gpu_util import d2h, stack_mod

pytestmark = pytest.mark.gpu

TOL = 1e-3


def _run(st, x, B, H, tensor_core):
    import torch
    d_x = torch.from_numpy(x).cuda()
    d_y = torch.zeros(B, H, dtype=torch.float32, device="cuda")
    assert st.layer_experts(0, d_x.data_ptr(), B, tensor_core=tensor_core) == 0
    assert st.layer_combine(0, B, d_y.data_ptr(), apply_norm=False) == 0
    assert st.status() == 0
    return d_y.cpu().numpy()


def _rel_err(y, ref):
    rms = np.sqrt((ref.astype(np.float64) ** 2).mean(axis=1, keepdims=True))
    return float((np.abs(y.astype(np.float64) - ref) / np.maximum(np.abs(ref), rms)).max())


# (hidden, inter, experts, top-k, tokens): groups of about 10, 75 (two token passes) and 1-3 tokens
@pytest.mark.parametrize("geom", [(512, 256, 8, 2, 40), (1024, 512, 4, 2, 150), (768, 256, 16, 2, 9)])
def test_nvfp4_tensor_core_layer_vs_oracle(orc, synth, geom):
    H, M, E, K, B = geom
    layer = synth.make_nvfp4_moe_layer(4500 + B, hidden=H, inter=M, n_experts=E, topk=K)
    x = synth.make_tokens(4501 + B, B, H)
    st = stack_mod().MoeStack(B, H, M, E, K)
    st.add_nvfp4_layer(layer)
    y = _run(st, x, B, H, True)
    want, sel, w = oracle.moe_layer_nvfp4(orc, layer, x, threads=16)
    ws = st.workspace()
    assert_bits_equal(d2h(ws.selected, B * K, np.int32).reshape(B, K), sel, "selected (exact)")
    assert_bits_equal(d2h(ws.weights, B * K, np.float32).reshape(B, K), w, "weights (exact)")
    err = _rel_err(y, want)
    print(f"nvfp4 tensor-core layer H={H} M={M} B={B}: max relative error {err:.3e}")
    assert err <= TOL, err
    assert_bits_equal(_run(st, x, B, H, False), want, "exact path on the same stack")
    st.close()


@pytest.mark.parametrize("B", [64, 256])
def test_nvfp4_tensor_core_cfg4_vs_exact_kernels(synth, B):
    """Config 4 (64 experts, hidden 5120, intermediate 1536, top-4) against the bit-exact GPU path."""
    layer = synth.make_nvfp4_moe_layer(4410)
    x = synth.make_tokens(4600 + B, B, layer.hidden)
    st = stack_mod().MoeStack(B, layer.hidden, layer.inter, layer.n_experts, layer.topk)
    st.add_nvfp4_layer(layer)
    y = _run(st, x, B, layer.hidden, True)
    want = _run(st, x, B, layer.hidden, False)
    err = _rel_err(y, want)
    print(f"nvfp4 tensor-core cfg 4 B={B}: max relative error {err:.3e}")
    assert err <= TOL, err
    assert_bits_equal(_run(st, x, B, layer.hidden, True), y, "run to run")
    st.close()
