"""The allocation-free expert chain (salt_b200_q4_expert_chain_static).

Some hosts of this library cannot call cudaMalloc once they are running: the
engine's own allocator has taken the whole device, or a fixed memory budget was
agreed when the plugin was loaded.  For them the library offers one entry point whose
intermediate rows live in a fixed array inside the library image.  This test
calls it through the C ABI twice in a row -- the second call smaller than the
first, so stale rows of the first are still lying in the shared array -- and
requires the same bits as the ordinary, allocating entry point
(salt_gpu_q4_moe_chain).  It also checks that an oversized call is refused.

Collected last on purpose (file name), so a run that stops at the first failure
has already exercised everything else.
"""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_bits_equal
from gpu_util import backend_mod, gpu

pytestmark = pytest.mark.gpu


def test_static_scratch_chain_matches_allocating_entry_point(synth, orc):
    import torch
    g, bm = gpu(), backend_mod()
    H, M = 256, 128
    layer = synth.make_q4_moe_layer(314, hidden=H, inter=M, n_experts=2, topk=1)
    e = 1
    # ordinary path: host pointers, weights registered as an expert-layer resource
    assert g.expert_resource_bind(71, layer.pool) == 0
    keys = [0x31400 + i for i in range(3)]
    tensors = [layer.tensor(e, which) for which in range(3)]
    for which, (v, s, b) in enumerate(tensors):
        R, Cc = (M, H) if which < 2 else (H, M)
        assert g.expert_resource_slot(71, keys[which], v, s, b, R, Cc) == 0
    # allocation-free path: the same bytes in device memory owned by the caller
    dev = [[torch.from_numpy(np.ascontiguousarray(a).view(np.uint8).copy()).cuda() for a in t] for t in tensors]
    for t in dev:
        for a in t:
            assert a.data_ptr() % 16 == 0
    fn = g.lib.salt_b200_q4_expert_chain_static
    for call, ntok in enumerate((9, 4)):
        x = synth.make_tokens(500 + call, ntok, H)
        want = np.zeros((ntok, H), np.float32)
        def addr(a):
            return a.ctypes.data
        ex = bm.MoeExpert(addr(tensors[0][0]), addr(tensors[0][1]), addr(tensors[0][2]), keys[0],
                          addr(tensors[1][0]), addr(tensors[1][1]), addr(tensors[1][2]), keys[1],
                          addr(tensors[2][0]), addr(tensors[2][1]), addr(tensors[2][2]), keys[2], ntok, -1, 0)
        assert g.q4_moe_chain([ex], H, M, x, want) == 0
        d_x = torch.from_numpy(x).cuda()
        d_y = torch.zeros(ntok, H, dtype=torch.float32, device="cuda")
        ptrs = [C.c_void_p(a.data_ptr()) for t in dev for a in t]
        rc = fn(*ptrs, H, M, C.c_void_p(d_x.data_ptr()), ntok, C.c_void_p(d_y.data_ptr()), None)
        assert rc == 0
        torch.cuda.synchronize()
        assert_bits_equal(d_y.cpu().numpy(), want, f"call {call} (ntok={ntok})")
        # and against the CPU oracle directly (first and last token of the call)
        for t in (0, ntok - 1):
            gate = orc.q4_matvec(*tensors[0], M, H, x[t])
            up = orc.q4_matvec(*tensors[1], M, H, x[t])
            ref = orc.q4_matvec(*tensors[2], H, M, orc.map_f32("gelu_tanh", gate) * up)
            assert_bits_equal(d_y[t].cpu().numpy(), ref, f"call {call} token {t} vs oracle")
    # beyond the fixed capacity (ntok*inter > 65536 floats) the call is refused, nothing runs
    big = 65536 // M + 1
    d_x = torch.zeros(big, H, dtype=torch.float32, device="cuda")
    d_y = torch.zeros(big, H, dtype=torch.float32, device="cuda")
    ptrs = [C.c_void_p(a.data_ptr()) for t in dev for a in t]
    assert fn(*ptrs, H, M, C.c_void_p(d_x.data_ptr()), big, C.c_void_p(d_y.data_ptr()), None) == -1
    assert g.expert_resource_unbind(71) == 0
