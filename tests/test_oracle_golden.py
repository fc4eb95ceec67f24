"""The CPU oracle (oracle/salt_oracle.c) against fixtures produced by the
reference project's own code (tests/golden/make_golden.py) -- bit exact."""
import numpy as np

from conftest import assert_bits_equal, golden


def test_bitmath_tables(orc):
    g = golden("bitmath.npz")
    for name in ("expf", "tanhf", "gelu_tanh"):
        assert_bits_equal(orc.map_f32(name, g["xs"]), g[name], name)
    for name in ("rsqrtf", "sqrtf"):
        assert_bits_equal(orc.map_f32(name, g["pos"]), g[name], name)


def test_q4_matvec_small_cases(orc):
    g = golden("q4_matvec.npz")
    for i in range(int(g["n_cases"])):
        R, C, B = (int(v) for v in g[f"c{i}_shape"])
        y = orc.q4_matvec_batch(g[f"c{i}_vals"], g[f"c{i}_scales"], g[f"c{i}_biases"], R, C,
                                g[f"c{i}_x"], threads=3)
        assert_bits_equal(y, g[f"c{i}_y"], f"case {i} {R}x{C} B={B}")
        y1 = orc.q4_matvec(g[f"c{i}_vals"], g[f"c{i}_scales"], g[f"c{i}_biases"], R, C, g[f"c{i}_x"][0])
        assert_bits_equal(y1, g[f"c{i}_y"][0], f"case {i} single")


def test_q4_matvec_benchmark_shapes(orc, synth):
    g = golden("q4_matvec_seeded.npz")
    for name in ("cfg1_4096x4096", "gate_704x2816", "down_2816x704", "odd_705x2816"):
        R, C, seed = (int(v) for v in g[name + "_meta"])
        rng = np.random.default_rng(seed)
        vals, s, b = synth.make_q4(rng, R, C)
        x = rng.standard_normal(C).astype(np.float32)
        assert_bits_equal(orc.q4_matvec(vals, s, b, R, C, x, threads=8), g[name + "_y"], name)


def test_router_chain(orc):
    g = golden("router.npz")
    K, eps = int(g["topk"]), float(g["eps"])
    for t in range(g["x"].shape[0]):
        rc, rin = orc.router_input(g["x"][t], g["scale"], eps)
        assert rc == 0
        assert_bits_equal(rin, g["rin"][t], "router input")
        logits = orc.router_scores(g["W"], None, rin)
        assert_bits_equal(logits, g["logits"][t], "logits")
        rc, sel, w = orc.router_topk(logits, g["pes"], K, True)
        assert rc == 0
        assert_bits_equal(sel, g["sel"][t], "selected")
        assert_bits_equal(w, g["wts"][t], "weights")
        rc, sel, w = orc.router_topk(logits, g["pes"], K, False)
        assert_bits_equal(sel, g["sel_rank"][t], "selected (rank order)")
        assert_bits_equal(w, g["wts_rank"][t], "weights (rank order)")
        rc, nm = orc.rmsnorm(g["x"][t], g["nw"], eps, True)
        assert rc == 0
        assert_bits_equal(nm, g["norm"][t], "rmsnorm")
    # the duplicated router row is an exact tie: the lower expert index ranks first
    assert (g["logits"][:, 3] == g["logits"][:, 7]).all()


def test_q8_matvec(orc):
    g = golden("q8_matvec.npz")
    for i, (R, Cc) in enumerate(g["shapes"]):
        y = orc.q8_matvec(g[f"c{i}_vals"], g[f"c{i}_scales"], g[f"c{i}_biases"], int(R), int(Cc), g[f"c{i}_x"])
        assert_bits_equal(y, g[f"c{i}_y"], f"q8 matvec {R}x{Cc}")


def test_moe_layer_nvfp4_small(orc, synth):
    import oracle
    g = golden("moe_layer_nvfp4_small.npz")
    lseed, xseed, B, H, M, E, K = (int(v) for v in g["meta"])
    layer = synth.make_nvfp4_moe_layer(lseed, hidden=H, inter=M, n_experts=E, topk=K)
    y, sel, w = oracle.moe_layer_nvfp4(orc, layer, synth.make_tokens(xseed, B, H))
    assert_bits_equal(sel, g["sel"], "nvfp4 layer selected")
    assert_bits_equal(w, g["w"], "nvfp4 layer weights")
    assert_bits_equal(y, g["y"], "nvfp4 layer output")


def test_bf16_matvec(orc):
    g = golden("bf16_matvec.npz")
    for i, (R, Cc, B) in enumerate(g["shapes"]):
        W, xs = g[f"c{i}_W"], g[f"c{i}_xs"]
        for t in range(int(B)):
            assert_bits_equal(orc.bf16_matvec(W, int(R), int(Cc), xs[t]), g[f"c{i}_y"][t], f"bf16 matvec {R}x{Cc}")
        assert_bits_equal(orc.bf16_matvec(W, int(R), int(Cc), xs[0], g[f"c{i}_bias"]), g[f"c{i}_y_bias"], "bf16 matvec + bias")
        assert_bits_equal(orc.bf16_matvec_serial(W, int(R), int(Cc), xs), g[f"c{i}_y_serial"], f"bf16 serial {R}x{Cc}")


def test_residual_combine_softcap_cells(orc):
    g = golden("cells.npz")
    eps, scalar = float(g["eps"]), float(g["scalar"])
    for n in (int(v) for v in g["sizes"]):
        a = {k: g[f"n{n}_{k}"] for k in ("res", "dense", "routed", "wd", "wr", "wf")}
        rc, y, scratch = orc.parallel_ffn_combine(a["res"], a["dense"], a["routed"], a["wd"], a["wr"], a["wf"],
                                                  scalar, eps)
        assert rc == 0
        assert_bits_equal(y, g[f"n{n}_combine"], f"parallel combine n={n}")
        assert_bits_equal(scratch, g[f"n{n}_scratch"], f"parallel combine scratch n={n}")
        rc, r = orc.residual_postnorm(a["res"], a["dense"], a["wd"], eps)
        assert rc == 0
        assert_bits_equal(r, g[f"n{n}_residual"], f"residual post-norm n={n}")
    rc, capped = orc.softcap(g["softcap_in"], float(g["softcap_cap"]))
    assert rc == 0
    assert_bits_equal(capped, g["softcap_out"], "softcap")
    # rejections, as the reference functions return -1
    bad = g["n64_res"].copy()
    bad[3] = np.inf
    assert orc.residual_postnorm(bad, g["n64_dense"], g["n64_wd"], eps)[0] == -1
    assert orc.softcap(bad, 30.0)[0] == -1
    assert orc.softcap(g["n64_res"], 0.0)[0] == -1


def test_grouping_and_reduce(orc):
    g = golden("grouping.npz")
    rows, topk = g["selected"].shape
    rc, offs, g2c, c2g, routed = orc.route_group(g["selected"].ravel(), rows, topk,
                                                 int(g["n_experts"]), g["row_inputs"])
    assert rc == 0
    assert_bits_equal(offs, g["offs"], "offsets")
    assert_bits_equal(g2c, g["g2c"], "grouped_to_canonical")
    assert_bits_equal(c2g, g["c2g"], "canonical_to_grouped")
    assert_bits_equal(routed, g["routed"], "routed inputs")
    rc, red = orc.weighted_reduce(g["weights"], c2g, g["grouped_outputs"], rows, topk)
    assert rc == 0
    assert_bits_equal(red, g["reduced"], "weighted reduce")


def test_nvfp4(orc):
    g = golden("nvfp4.npz")
    enc = np.array([orc.e4m3fn_encode(float(v))[1] for v in g["enc_in"]], np.uint8)
    assert_bits_equal(enc, g["enc"], "e4m3 encode")
    dec = np.array([orc.e4m3fn(c) for c in range(256)], np.float32)
    assert_bits_equal(dec, g["dec"], "e4m3 decode")
    R, C = g["wpacked"].shape[0], g["wpacked"].shape[1] * 2
    rc, wdq = orc.nvfp4_dequant_weights(g["wpacked"], g["wscale"], float(g["divisor"]), R, C)
    assert rc == 0
    assert_bits_equal(wdq, g["wdq"], "weight dequant")
    for t in range(g["x"].shape[0]):
        rc, p, s, d = orc.nvfp4_qdq(g["x"][t], float(g["input_global"]))
        assert rc == 0
        assert_bits_equal(p, g["qdq_packed"][t], "qdq codes")
        assert_bits_equal(s, g["qdq_scales"][t], "qdq scales")
        assert_bits_equal(d, g["qdq_dequant"][t], "qdq dequant")
        rc, y = orc.nvfp4_matvec(g["wpacked"], g["wscale"], float(g["divisor"]),
                                 float(g["input_global"]), R, C, g["x"][t], threads=2)
        assert rc == 0
        assert_bits_equal(y, g["y"][t], "nvfp4 matvec")


def test_moe_layer_small(orc, synth):
    g = golden("moe_layer_small.npz")
    lseed, xseed, B, H, M, E, K = (int(v) for v in g["meta"])
    layer = synth.make_q4_moe_layer(lseed, hidden=H, inter=M, n_experts=E, topk=K)
    x = synth.make_tokens(xseed, B, H)
    y, sel, w = orc.moe_layer_q4(layer, x, threads=4)
    assert_bits_equal(sel, g["sel"], "selected")
    assert_bits_equal(w, g["w"], "weights")
    assert_bits_equal(y, g["y"], "layer output")
    # thread count changes row ownership only
    y1, _, _ = orc.moe_layer_q4(layer, x, threads=1)
    assert_bits_equal(y1, y, "1 vs 4 threads")
