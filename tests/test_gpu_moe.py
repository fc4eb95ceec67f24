"""Router, grouping, expert chain and the device-resident MoE stack on the GPU,
against the CPU oracle and the golden fixtures (bit exact)."""
import ctypes as C

import numpy as np
import pytest

from conftest import assert_bits_equal, golden
from gpu_util import backend_mod, d2h, gpu, oracle_stack, stack_mod

pytestmark = pytest.mark.gpu


def test_exact_cells_router_chain_golden():
    g, bm, fx = gpu(), backend_mod(), golden("router.npz")
    H, E, K = fx["x"].shape[1], fx["W"].shape[0], int(fx["topk"])
    rc, buf = g.shared_buffer_alloc(4 * (4 * H + 2 * E + 2 * K + 16))
    assert rc == 0
    f = buf.array(np.float32)
    o_x, o_w, o_out, o_log, o_pes, o_sel, o_wts = 0, H, 2 * H, 3 * H, 3 * H + E, 3 * H + 2 * E, 3 * H + 2 * E + K
    for t in range(fx["x"].shape[0]):
        f[o_x:o_x + H] = fx["x"][t]
        f[o_w:o_w + H] = fx["scale"]
        cell = bm.exact_cell(bm.EXACT_ROUTER_INPUT, [buf] * 3, [o_x, o_w, o_out], H, eps=float(fx["eps"]))
        assert g.exact_cells([cell]) == 0
        assert_bits_equal(f[o_out:o_out + H].copy(), fx["rin"][t], "router input cell")
        f[o_w:o_w + H] = fx["nw"]
        cell = bm.exact_cell(bm.EXACT_RMSNORM, [buf] * 3, [o_x, o_w, o_out], H, aux=1, eps=float(fx["eps"]))
        assert g.exact_cells([cell]) == 0
        assert_bits_equal(f[o_out:o_out + H].copy(), fx["norm"][t], "rmsnorm cell")
        f[o_log:o_log + E] = fx["logits"][t]
        f[o_pes:o_pes + E] = fx["pes"]
        cell = bm.exact_cell(bm.EXACT_TOPK, [buf] * 4, [o_log, o_pes, o_sel, o_wts], E, aux=K)
        assert g.exact_cells([cell]) == 0
        assert_bits_equal(f[o_sel:o_sel + K].view(np.int32).copy(), fx["sel"][t], "topk selected")
        assert_bits_equal(f[o_wts:o_wts + K].copy(), fx["wts"][t], "topk weights")
    # non-finite input is rejected, as the reference functions return -1
    f[o_log] = np.inf
    cell = bm.exact_cell(bm.EXACT_TOPK, [buf] * 4, [o_log, o_pes, o_sel, o_wts], E, aux=K)
    assert g.exact_cells([cell]) == -1
    assert g.shared_buffer_free(buf) == 0


@pytest.mark.parametrize("kind", ["normal", "wide_range", "ties", "subnormal_squares", "sparse", "powers_of_two"])
def test_ordered_sum_of_squares_adversarial_rows(orc, kind):
    """RMSNorm and router-input cells on rows built to stress the in-order sum of squares:
    half-way cases, subnormal squares, zeros and terms spread over many binades."""
    g, bm = gpu(), backend_mod()
    rng = np.random.default_rng(abs(hash(kind)) % (1 << 31))
    nmax = 5000
    rc, buf = g.shared_buffer_alloc(4 * (3 * nmax + 16))
    assert rc == 0
    f = buf.array(np.float32)
    for n in (1, 2, 63, 64, 65, 257, 1024, 1025, 2816, 5000):
        if kind == "normal":
            x = rng.standard_normal(n)
        elif kind == "wide_range":
            x = rng.standard_normal(n) * 10.0 ** rng.uniform(-18, 12, n)
        elif kind == "ties":
            x = rng.integers(0, 64, n) * 2.0 ** -10
        elif kind == "subnormal_squares":
            x = rng.standard_normal(n) * 1e-20
        elif kind == "sparse":
            x = np.where(rng.random(n) < 0.6, 0.0, rng.standard_normal(n))
        else:
            x = np.sign(rng.standard_normal(n)) * 2.0 ** rng.integers(-8, 8, n)
        x = x.astype(np.float32)
        w = (1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32)
        f[0:n] = x
        f[nmax:nmax + n] = w
        for cell_kind, name in ((bm.EXACT_RMSNORM, "rmsnorm"), (bm.EXACT_ROUTER_INPUT, "router input")):
            cell = bm.exact_cell(cell_kind, [buf] * 3, [0, nmax, 2 * nmax], n, aux=1, eps=1e-6)
            assert g.exact_cells([cell]) == 0, (kind, n, name)
            want = orc.rmsnorm(x, w, 1e-6)[1] if cell_kind == bm.EXACT_RMSNORM else orc.router_input(x, w, 1e-6)[1]
            assert_bits_equal(f[2 * nmax:2 * nmax + n].copy(), want, f"{name} {kind} n={n}")
    assert g.shared_buffer_free(buf) == 0


def test_exact_cells_residual_combine_softcap_golden(orc):
    """The consumers of the routed-expert output (reference gemma4.c:188-286) through
    salt_gpu_exact_cells, against the golden vectors and, at larger sizes, the oracle."""
    g, bm, fx = gpu(), backend_mod(), golden("cells.npz")
    eps, scalar = float(fx["eps"]), float(fx["scalar"])
    nmax = 5120
    rc, buf = g.shared_buffer_alloc(4 * (9 * nmax + 16))
    assert rc == 0
    f = buf.array(np.float32)
    o = [k * nmax for k in range(9)]          # residual, dense, routed, wd, wr, wf, scratch (2n), out

    def run(n, res, dense, routed, wd, wr, wf):
        for off, arr in zip(o[:6], (res, dense, routed, wd, wr, wf)):
            f[off:off + n] = arr
        cell = bm.exact_cell(bm.EXACT_PARALLEL_COMBINE, [buf] * 8, [o[0], o[1], o[2], o[3], o[4], o[5], o[6], o[8]],
                             n, eps=eps, scalar=scalar)
        assert g.exact_cells([cell]) == 0
        combine, scratch = f[o[8]:o[8] + n].copy(), f[o[6]:o[6] + 2 * n].copy()
        cell = bm.exact_cell(bm.EXACT_RESIDUAL_POSTNORM, [buf] * 4, [o[0], o[1], o[3], o[8]], n, eps=eps)
        assert g.exact_cells([cell]) == 0
        return combine, scratch, f[o[8]:o[8] + n].copy()

    for n in (int(v) for v in fx["sizes"]):
        a = [fx[f"n{n}_{k}"] for k in ("res", "dense", "routed", "wd", "wr", "wf")]
        combine, scratch, residual = run(n, *a)
        assert_bits_equal(combine, fx[f"n{n}_combine"], f"combine cell n={n}")
        assert_bits_equal(scratch, fx[f"n{n}_scratch"], f"combine scratch n={n}")
        assert_bits_equal(residual, fx[f"n{n}_residual"], f"residual cell n={n}")
    rng = np.random.default_rng(11)
    for n in (1000, 4096, 4097, 5120):       # beyond the fixtures: block-parallel and serial sum paths
        a = [rng.standard_normal(n).astype(np.float32) for _ in range(3)] + \
            [(1.0 + 0.1 * rng.standard_normal(n)).astype(np.float32) for _ in range(3)]
        combine, scratch, residual = run(n, *a)
        rc, want, want_scratch = orc.parallel_ffn_combine(*a, scalar, eps)
        assert rc == 0
        assert_bits_equal(combine, want, f"combine cell vs oracle n={n}")
        assert_bits_equal(scratch, want_scratch, f"combine scratch vs oracle n={n}")
        assert_bits_equal(residual, orc.residual_postnorm(a[0], a[1], a[3], eps)[1], f"residual cell vs oracle n={n}")
    logits = fx["softcap_in"]
    f[0:logits.size] = logits
    cell = bm.exact_cell(bm.EXACT_SOFTCAP, [buf], [0], logits.size, scalar=float(fx["softcap_cap"]))
    assert g.exact_cells([cell]) == 0
    assert_bits_equal(f[0:logits.size].copy(), fx["softcap_out"], "softcap cell")
    # rejections: non-finite input, non-positive cap
    f[5] = np.nan
    assert g.exact_cells([cell]) == -1
    cell = bm.exact_cell(bm.EXACT_SOFTCAP, [buf], [0], 16, scalar=0.0)
    assert g.exact_cells([cell]) == -1
    assert g.shared_buffer_free(buf) == 0


def test_route_group_device_golden_and_reference_kat(orc):
    import torch
    g = gpu()
    cases = [(np.array([2, 0, 2, 1, 0, 2], np.int32), 3, 2, 4)]
    fx = golden("grouping.npz")
    cases.append((fx["selected"].ravel().astype(np.int32), fx["selected"].shape[0], fx["selected"].shape[1],
                  int(fx["n_experts"])))
    rng = np.random.default_rng(4)
    for rows, topk, ne in ((512, 8, 128), (2048, 8, 128), (37, 4, 64)):
        sel = np.stack([np.sort(rng.permutation(ne)[:topk]) for _ in range(rows)]).astype(np.int32)
        cases.append((sel.ravel(), rows, topk, ne))
    for sel, rows, topk, ne in cases:
        d_sel = torch.from_numpy(sel).cuda()
        d_off = torch.zeros(ne + 1, dtype=torch.int32, device="cuda")
        d_g2c = torch.zeros(rows * topk, dtype=torch.int32, device="cuda")
        d_c2g = torch.zeros(rows * topk, dtype=torch.int32, device="cuda")
        rc = g.lib.salt_b200_route_group_device(C.c_void_p(d_sel.data_ptr()), rows, topk, ne,
                                                C.c_void_p(d_off.data_ptr()), C.c_void_p(d_g2c.data_ptr()),
                                                C.c_void_p(d_c2g.data_ptr()), None)
        assert rc == 0
        rc, offs, g2c, c2g, _ = orc.route_group(sel, rows, topk, ne)
        assert rc == 0
        assert_bits_equal(d_g2c.cpu().numpy(), g2c, "grouped_to_canonical")
        assert_bits_equal(d_c2g.cpu().numpy(), c2g, "canonical_to_grouped")
        starts = np.concatenate([[0], offs]).astype(np.int32)  # the oracle leaves END offsets
        assert_bits_equal(d_off.cpu().numpy(), starts, "group offsets")
    assert cases[0][0] is not None and d_g2c is not None
    # reference tests/test_text_verify.c:1238-1239
    sel, rows, topk, ne = cases[0]
    rc, offs, g2c, c2g, _ = orc.route_group(sel, rows, topk, ne)
    assert g2c.tolist() == [1, 4, 3, 0, 2, 5] and c2g.tolist() == [3, 0, 4, 2, 1, 5]


def _expert_struct(bm, layer, e, group, key_base):
    def addr(a):
        return a.ctypes.data
    gv, gs, gb = layer.tensor(e, 0)
    uv, us, ub = layer.tensor(e, 1)
    dv, ds, db = layer.tensor(e, 2)
    return bm.MoeExpert(addr(gv), addr(gs), addr(gb), key_base + 3 * e, addr(uv), addr(us), addr(ub),
                        key_base + 3 * e + 1, addr(dv), addr(ds), addr(db), key_base + 3 * e + 2, group, -1, 0)


@pytest.mark.parametrize("groups", [[1], [1, 1, 1], [3, 1, 9, 2], [40]])
def test_q4_moe_chain_vs_oracle(orc, synth, groups):
    # reference call: salt_gpu_q4_moe_chain from g4_group_run_many (gemma4_text.c:9050)
    g, bm = gpu(), backend_mod()
    H, M = 256, 128
    layer = synth.make_q4_moe_layer(21, hidden=H, inter=M, n_experts=8, topk=2)
    assert g.expert_resource_bind(33, layer.pool) == 0
    key_base = 0x77000
    experts = []
    for i, grp in enumerate(groups):
        e = (i * 3 + 1) % 8
        for which in range(3):
            R, Cc = (M, H) if which < 2 else (H, M)
            v, s, b = layer.tensor(e, which)
            assert g.expert_resource_slot(33, key_base + 3 * e + which, v, s, b, R, Cc) == 0
        experts.append(_expert_struct(bm, layer, e, grp, key_base))
    total = sum(groups)
    x = synth.make_tokens(5, total, H)
    y = np.zeros((total, H), np.float32)
    assert g.q4_moe_chain(experts, H, M, x, y) == 0
    row = 0
    for i, grp in enumerate(groups):
        e = (i * 3 + 1) % 8
        for t in range(grp):
            gate = orc.q4_matvec(*layer.tensor(e, 0), M, H, x[row])
            up = orc.q4_matvec(*layer.tensor(e, 1), M, H, x[row])
            chain = orc.map_f32("gelu_tanh", gate) * up
            want = orc.q4_matvec(*layer.tensor(e, 2), H, M, chain)
            assert_bits_equal(y[row], want, f"expert {e} row {row}")
            row += 1
    assert g.expert_resource_unbind(33) == 0


def test_stack_small_geometry_golden(synth):
    fx = golden("moe_layer_small.npz")
    lseed, xseed, B, H, M, E, K = (int(v) for v in fx["meta"])
    layer = synth.make_q4_moe_layer(lseed, hidden=H, inter=M, n_experts=E, topk=K)
    x = synth.make_tokens(xseed, B, H)
    st = stack_mod().MoeStack(16, H, M, E, K)
    st.add_layer(layer)
    y = st.forward_host(x)
    ws = st.workspace()
    assert_bits_equal(d2h(ws.selected, B * K, np.int32).reshape(B, K), fx["sel"], "selected")
    assert_bits_equal(d2h(ws.weights, B * K, np.float32).reshape(B, K), fx["w"], "weights")
    assert_bits_equal(y, fx["y"], "layer output")
    st.close()


@pytest.mark.parametrize("B", [1, 2, 4, 8, 9, 16, 33, 64])
def test_stack_cfg2_layer_decode_sweep_vs_oracle(orc, synth, B):
    layer = synth.make_q4_moe_layer(2, )          # H=2816, E=128, top-8, M=704
    x = synth.make_tokens(100 + B, B, layer.hidden)
    st = stack_mod().MoeStack(64, layer.hidden, layer.inter, layer.n_experts, layer.topk)
    st.add_layer(layer)
    y = st.forward_host(x)
    want, sel, w = orc.moe_layer_q4(layer, x, threads=8)
    ws = st.workspace()
    assert_bits_equal(d2h(ws.selected, B * 8, np.int32).reshape(B, 8), sel, "selected")
    assert_bits_equal(d2h(ws.weights, B * 8, np.float32).reshape(B, 8), w, "weights")
    assert_bits_equal(y, want, f"cfg2 layer B={B}")
    y2 = st.forward_host(x)
    assert_bits_equal(y2, y, "run-to-run")
    st.close()


def test_stack_three_layers_with_rmsnorm_vs_oracle(orc, synth):
    H, M, E, K = 512, 128, 32, 4
    layers = [synth.make_q4_moe_layer(40 + i, hidden=H, inter=M, n_experts=E, topk=K) for i in range(3)]
    x = synth.make_tokens(9, 5, H)
    st = stack_mod().MoeStack(8, H, M, E, K)
    for layer in layers:
        st.add_layer(layer)
    y = st.forward_host(x)
    want, _ = oracle_stack(orc, layers, x, threads=4)
    assert_bits_equal(y, want, "3-layer stack")
    st.close()


@pytest.mark.parametrize("B", [1, 3, 12])
def test_stack_graph_replay_equals_stream_launches_and_oracle(orc, synth, B):
    """The captured CUDA graph (programmatic dependent launches become graph edges) must give
    the same bits as the stream launches and as the oracle, on every replay and after the
    input buffer changes."""
    import torch
    H, M, E, K = 2816, 704, 128, 8
    layers = [synth.make_q4_moe_layer_bulk(60 + i) for i in range(3)]
    st = stack_mod().MoeStack(16, H, M, E, K)
    for layer in layers:
        st.add_layer(layer)
    stream = torch.cuda.Stream()
    sp = stream.cuda_stream
    x0, x1 = synth.make_tokens(70 + B, B, H), synth.make_tokens(170 + B, B, H)
    d_x = torch.from_numpy(x0).cuda()
    d_y = torch.zeros_like(d_x)
    with torch.cuda.stream(stream):
        assert st.forward_device(d_x.data_ptr(), B, d_y.data_ptr(), stream=sp) == 0
        stream.synchronize()
        y_stream = d_y.cpu().numpy()
        assert st.graph_capture(d_x.data_ptr(), B, d_y.data_ptr(), sp) == 0
        for rep in range(3):
            d_y.zero_()
            assert st.graph_launch(sp) == 0
            stream.synchronize()
            assert_bits_equal(d_y.cpu().numpy(), y_stream, f"graph replay {rep}")
        d_x.copy_(torch.from_numpy(x1))
        for rep in range(2):
            assert st.graph_launch(sp) == 0
        stream.synchronize()
        y1 = d_y.cpu().numpy()
    assert st.status(sp) == 0
    want0, _ = oracle_stack(orc, layers, x0, threads=16)
    want1, _ = oracle_stack(orc, layers, x1, threads=16)
    assert_bits_equal(y_stream, want0, "stream launches vs oracle")
    assert_bits_equal(y1, want1, "graph replay on new input vs oracle")
    st.close()


def test_stack_expert_sharding_union_equals_single_device(orc, synth):
    """Two half-stacks (experts 0-15 and 16-31) on the same GPU: each fills only its
    rows of the grouped buffer; their union reproduces the unsharded result."""
    import torch
    H, M, E, K, B = 256, 128, 32, 4, 7
    layer = synth.make_q4_moe_layer(61, hidden=H, inter=M, n_experts=E, topk=K)
    x = synth.make_tokens(62, B, H)
    want, _, _ = orc.moe_layer_q4(layer, x, threads=4)
    sm = stack_mod()
    d_x = torch.from_numpy(x).cuda()
    shared = torch.zeros(8 * K * H, dtype=torch.float32, device="cuda")   # max_tokens rows
    halves = []
    for lo, hi in ((0, 16), (16, 32)):
        st = sm.MoeStack(8, H, M, E, K, expert_begin=lo, expert_end=hi)
        st.add_layer(layer)
        assert st.set_grouped_out(shared.data_ptr(), shared.numel() * 4) == 0
        assert st.layer_experts(0, d_x.data_ptr(), B) == 0
        halves.append(st)
    d_y = torch.zeros(B, H, dtype=torch.float32, device="cuda")
    assert halves[0].layer_combine(0, B, d_y.data_ptr(), apply_norm=False) == 0
    assert halves[0].status() == 0 and halves[1].status() == 0
    assert_bits_equal(d_y.cpu().numpy(), want, "sharded union")
    for st in halves:
        st.close()


def test_stack_eight_way_sharding_bench_geometry(orc, synth):
    """The bench layer (128 experts, top-8) cut into eight expert ranges, 8 tokens: what every rank of
    an 8-GPU run computes, here one range after the other over one shared grouped buffer."""
    import torch
    H, M, E, K, B = 2816, 704, 128, 8, 8
    layer = synth.make_q4_moe_layer_bulk(64)
    x = synth.make_tokens(65, B, H)
    want, _, _ = orc.moe_layer_q4(layer, x, threads=16)
    sm = stack_mod()
    d_x = torch.from_numpy(x).cuda()
    shared = torch.zeros(B * K * H, dtype=torch.float32, device="cuda")
    parts = []
    for r in range(8):
        st = sm.MoeStack(B, H, M, E, K, expert_begin=r * 16, expert_end=(r + 1) * 16)
        st.add_layer(layer)
        assert st.set_grouped_out(shared.data_ptr(), shared.numel() * 4) == 0
        assert st.layer_experts(0, d_x.data_ptr(), B) == 0
        parts.append(st)
    d_y = torch.zeros(B, H, dtype=torch.float32, device="cuda")
    assert parts[3].layer_combine(0, B, d_y.data_ptr(), apply_norm=False) == 0
    assert all(st.status() == 0 for st in parts)
    assert_bits_equal(d_y.cpu().numpy(), want, "eight-way sharded union")
    for st in parts:
        st.close()


def _oracle_ffn_block(orc, layer, block, residual):
    """CPU statement of the whole feed-forward block (reference gemma4_text.c:8293-8385, gemma4.c:215-276)
    from the oracle's functions: dense GeGLU MLP on RMSNorm(residual), router on the residual, experts on
    the second RMSNorm, parallel combine."""
    B, H = residual.shape
    out = np.empty_like(residual)
    gate, up, down = (block.tensor(k, H) for k in ("dense_gate", "dense_up", "dense_down"))
    vb = layer.hidden * layer.inter // 2
    gb = layer.hidden * layer.inter // 64 * 2
    tb = vb + 2 * gb

    def expert_tensor(e, which):
        base = e * layer.expert_stride + which * tb
        buf = layer.pool[base:base + tb]
        return buf[:vb].view(np.uint32), buf[vb:vb + gb].view(np.uint16), buf[vb + gb:].view(np.uint16)

    gelu = np.vectorize(orc.gelu_tanh, otypes=[np.float32])
    for t in range(B):
        res = residual[t]
        rc, norm_a = orc.rmsnorm(res, block.pre_ffn_norm, layer.eps, True)
        assert rc == 0
        g = orc.q4_matvec(*gate[:3], gate[3], gate[4], norm_a, threads=8)
        u = orc.q4_matvec(*up[:3], up[3], up[4], norm_a, threads=8)
        dense = orc.q4_matvec(*down[:3], down[3], down[4], (gelu(g) * u).astype(np.float32), threads=8)
        rc, rin = orc.router_input(res, layer.router_scale, layer.eps)
        assert rc == 0
        logits = orc.router_scores(layer.router_w, None, rin)
        rc, sel, w = orc.router_topk(logits, layer.per_expert_scale, layer.topk, True)
        assert rc == 0
        rc, norm_b = orc.rmsnorm(res, block.pre_ffn_norm_2, layer.eps, True)
        assert rc == 0
        routed = np.zeros(H, np.float32)
        for rank in range(layer.topk):
            e = int(sel[rank])
            eg = orc.q4_matvec(*expert_tensor(e, 0), layer.inter, H, norm_b, threads=8)
            eu = orc.q4_matvec(*expert_tensor(e, 1), layer.inter, H, norm_b, threads=8)
            ed = orc.q4_matvec(*expert_tensor(e, 2), H, layer.inter, (gelu(eg) * eu).astype(np.float32), threads=8)
            routed = (routed + (np.float32(w[rank]) * ed).astype(np.float32)).astype(np.float32)
        rc, y, _ = orc.parallel_ffn_combine(res, dense, routed, block.post_ffn_norm_1, block.post_ffn_norm_2,
                                            block.post_ffn_norm, block.layer_scalar, layer.eps)
        assert rc == 0
        out[t] = y
    return out


@pytest.mark.parametrize("geom", [(256, 128, 192, 16, 4, 5), (2816, 704, 2112, 128, 8, 2)])
def test_whole_ffn_block_vs_oracle(orc, synth, geom):
    import torch
    H, M, D, E, K, B = geom
    make = synth.make_q4_moe_layer_bulk if H == 2816 else synth.make_q4_moe_layer
    layer = make(81, hidden=H, inter=M, n_experts=E, topk=K)
    block = synth.make_ffn_block(82, hidden=H, dense_inter=D)
    st = stack_mod().MoeStack(8, H, M, E, K)
    st.add_layer(layer)
    assert st.attach_ffn_block(0, block) == 0
    residual = synth.make_tokens(83, B, H)
    d_res = torch.from_numpy(residual).cuda()
    d_out = torch.zeros_like(d_res)
    for rep in range(2):
        assert st.ffn_block_forward(0, d_res.data_ptr(), B, d_out.data_ptr()) == 0
    assert st.status() == 0
    want = _oracle_ffn_block(orc, layer, block, residual)
    assert_bits_equal(d_out.cpu().numpy(), want, f"whole FFN block H={H}")
    st.close()



@pytest.mark.parametrize("geom", [(320, 64, 24, 2, 300), (320, 64, 24, 2, 1030), (2816, 704, 128, 8, 1030)])
def test_router_logits_prefill_sized_batches_vs_oracle(orc, synth, geom):
    """Batches of several hundred rows take the large-tile logits kernels (32 experts x 16 or 32 rows
    per block); ragged tiles in both directions, a last column slab shorter than the others."""
    import torch
    H, M, E, K, B = geom
    make = synth.make_q4_moe_layer_bulk if H == 2816 else synth.make_q4_moe_layer
    layer = make(91, hidden=H, inter=M, n_experts=E, topk=K)
    st = stack_mod().MoeStack(B, H, M, E, K)
    st.add_layer(layer)
    x = synth.make_tokens(92, B, H)
    d_x = torch.from_numpy(x).cuda()
    assert st.layer_experts(0, d_x.data_ptr(), B) == 0
    assert st.status() == 0
    got = d2h(st.workspace().logits, B * E, np.float32).reshape(B, E)
    want = np.empty_like(got)
    for t in range(B):
        rc, rin = orc.router_input(x[t], layer.router_scale, layer.eps)
        assert rc == 0
        want[t] = orc.router_scores(layer.router_w, None, rin)
    assert_bits_equal(got, want, f"router logits B={B} H={H}")
    st.close()


def test_stack_two_layers_prefill_sized_batch_vs_oracle(orc, synth):
    """300 rows at the bench geometry: the reduce + RMSNorm + router-input glue runs one warp per row
    (dependent-add chains handed from lane to lane), the logits take the large tiles; the second layer's
    output depends on both."""
    B = 300
    layers = [synth.make_q4_moe_layer_bulk(95 + i) for i in range(2)]
    x = synth.make_tokens(97, B, 2816)
    st = stack_mod().MoeStack(B, 2816, 704, 128, 8)
    for layer in layers:
        st.add_layer(layer)
    y = st.forward_host(x)
    want, _ = oracle_stack(orc, layers, x, threads=16)
    assert_bits_equal(y, want, "2-layer stack, 300 rows")
    st.close()


def test_stack_two_layers_prefill_sized_batch_hidden_5120_vs_oracle(orc, synth):
    """The same at hidden = 5120 (160 columns per lane in the warp-per-row glue, the hidden size of the NVFP4
    configuration) with small experts so that the CPU side stays cheap: 260 rows, top-2 of 8."""
    B, H, M, E, K = 260, 5120, 64, 8, 2
    layers = [synth.make_q4_moe_layer(195 + i, hidden=H, inter=M, n_experts=E, topk=K) for i in range(2)]
    x = synth.make_tokens(197, B, H)
    st = stack_mod().MoeStack(B, H, M, E, K)
    for layer in layers:
        st.add_layer(layer)
    y = st.forward_host(x)
    want, _ = oracle_stack(orc, layers, x, threads=16)
    assert_bits_equal(y, want, "2-layer stack, 260 rows, hidden 5120")
    st.close()


def test_stack_wide_hidden_takes_any_shape_kernels_vs_oracle(orc, synth):
    """hidden = 5696 is beyond what the tiled projection kernels hold in shared memory: the stack runs the
    any-shape kernels, one grid row per token of a group.  Groups of more than four tokens must all be
    computed (6 tokens over 4 experts, top-2: every group holds several tokens)."""
    H, M, E, K, B = 5696, 128, 4, 2, 6
    layers = [synth.make_q4_moe_layer(97 + i, hidden=H, inter=M, n_experts=E, topk=K) for i in range(2)]
    x = synth.make_tokens(99, B, H)
    st = stack_mod().MoeStack(8, H, M, E, K)
    for layer in layers:
        st.add_layer(layer)
    y = st.forward_host(x)
    want, _ = oracle_stack(orc, layers, x, threads=8)
    assert_bits_equal(y, want, "wide hidden, any-shape kernels")
    st.close()
