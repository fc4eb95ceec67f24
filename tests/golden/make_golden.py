"""Regenerate tests/golden/*.npz from the reference project's own code.

Run in a container where the reference checkout is mounted and
``make -C oracle ref`` has produced ``oracle/_ref/libsalt_ref.so`` (the
reference sources compiled unmodified).  Every array written here is an output
of that library; small cases also store their inputs so the fixtures do not
depend on a PRNG implementation.

    python tests/golden/make_golden.py            # everything
    python tests/golden/make_golden.py cells      # only the residual / combine / softcap cells
"""
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle  # noqa: E402

synth = importlib.import_module("salt-core_b200.synth")
OUT = os.path.dirname(os.path.abspath(__file__))


def gen_cells(ref):
    """Consumers of the routed-expert output (reference gemma4.c:188-286): residual + post-norm,
    parallel FFN combine, logit soft-cap.  Inputs are stored next to the outputs."""
    rng = np.random.default_rng(20261126)
    out = {}
    sizes = (1, 5, 64, 257, 2816)
    out["sizes"] = np.array(sizes)
    for n in sizes:
        res, dense, routed = (rng.standard_normal(n).astype(np.float32) * np.float32(sc) for sc in (1.0, 3.0, 0.4))
        wd, wr, wf = ((1.0 + 0.2 * rng.standard_normal(n)).astype(np.float32) for _ in range(3))
        rc, y, scratch = ref.parallel_ffn_combine(res, dense, routed, wd, wr, wf, 0.8125, 1e-6)
        assert rc == 0
        rc2, r2 = ref.residual_postnorm(res, dense, wd, 1e-6)
        assert rc2 == 0
        out.update({f"n{n}_res": res, f"n{n}_dense": dense, f"n{n}_routed": routed, f"n{n}_wd": wd,
                    f"n{n}_wr": wr, f"n{n}_wf": wf, f"n{n}_combine": y, f"n{n}_scratch": scratch,
                    f"n{n}_residual": r2})
    logits = np.concatenate([rng.standard_normal(3000) * 25.0, np.linspace(-400, 400, 801),
                             [0.0, -0.0, 1e-30, -1e-30, 29.999, 30.0, 300.0, -300.0]]).astype(np.float32)
    rc, capped = ref.softcap(logits, 30.0)
    assert rc == 0
    out.update(softcap_in=logits, softcap_out=capped, softcap_cap=np.float32(30.0),
               scalar=np.float32(0.8125), eps=np.float32(1e-6))
    np.savez_compressed(os.path.join(OUT, "cells.npz"), **out)

    # affine 8-bit matvec (reference src/kernels.c:343-369): router-sized, ragged, tiny
    q8 = {"shapes": np.array([[16, 2816], [5, 200], [3, 64], [7, 72]])}
    for i, (R, Cc) in enumerate(q8["shapes"]):
        n = int(R) * int(Cc)
        vals = rng.integers(0, 256, (n + 3) // 4 * 4, dtype=np.uint8)
        groups = (n + 63) // 64
        sc = (rng.uniform(0.001, 0.02, groups).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
        bi = ((-128.0 * rng.uniform(0.001, 0.02, groups)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
        x = rng.standard_normal(int(Cc)).astype(np.float32)
        q8.update({f"c{i}_vals": vals, f"c{i}_scales": sc, f"c{i}_biases": bi, f"c{i}_x": x,
                   f"c{i}_y": ref.q8_matvec(vals, sc, bi, int(R), int(Cc), x)})
    np.savez_compressed(os.path.join(OUT, "q8_matvec.npz"), **q8)


def gen_bf16(ref):
    """BF16 matrices (reference src/kernels.c:139-174 salt_bf16_matvec; the serial batch form of
    models/gemma4-26b-a4b/src/gemma4_vision.c:700-717 is pinned through salt_f32_matvec, the same
    chain on the widened weights): router-sized, head-like, ragged and tiny shapes."""
    rng = np.random.default_rng(20261126)
    out = {"shapes": np.array([[128, 2816, 3], [16, 704, 2], [5, 200, 1], [3, 8, 2], [7, 75, 1]])}
    for i, (R, Cc, B) in enumerate(out["shapes"]):
        W = (rng.normal(0.0, 0.02, (int(R), int(Cc))).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
        W32 = (W.astype(np.uint32) << 16).view(np.float32)
        bias = rng.standard_normal(int(R)).astype(np.float32)
        xs = rng.standard_normal((int(B), int(Cc))).astype(np.float32)
        out.update({f"c{i}_W": W, f"c{i}_bias": bias, f"c{i}_xs": xs,
                    f"c{i}_y": np.stack([ref.bf16_matvec(W, int(R), int(Cc), xs[t]) for t in range(int(B))]),
                    f"c{i}_y_bias": ref.bf16_matvec(W, int(R), int(Cc), xs[0], bias),
                    f"c{i}_y_serial": np.stack([ref.f32_matvec(W32, int(R), int(Cc), xs[t]) for t in range(int(B))])})
    np.savez_compressed(os.path.join(OUT, "bf16_matvec.npz"), **out)


def gen_nvfp4_layer(ref):
    """A small MoE layer with NVFP4 experts through the reference's own functions."""
    lseed, xseed, B, H, M, E, K = 4401, 4402, 3, 512, 256, 8, 2
    layer = synth.make_nvfp4_moe_layer(lseed, hidden=H, inter=M, n_experts=E, topk=K)
    x = synth.make_tokens(xseed, B, H)
    y, sel, w = oracle.moe_layer_nvfp4(ref, layer, x)
    np.savez_compressed(os.path.join(OUT, "moe_layer_nvfp4_small.npz"), meta=np.array([lseed, xseed, B, H, M, E, K]),
                        y=y, sel=sel, w=w)


def main():
    ref = oracle.Reference()
    if len(sys.argv) > 1 and sys.argv[1] == "nvfp4_layer":
        gen_nvfp4_layer(ref)
        print("moe_layer_nvfp4_small.npz written to", OUT)
        return
    if len(sys.argv) > 1 and sys.argv[1] == "cells":
        gen_cells(ref)
        print("cells.npz written to", OUT)
        return
    if len(sys.argv) > 1 and sys.argv[1] == "bf16":
        gen_bf16(ref)
        print("bf16_matvec.npz written to", OUT)
        return
    rng = np.random.default_rng(20261125)

    # --- scalar math tables -------------------------------------------
    xs = np.concatenate([np.linspace(-100, 100, 1501), np.linspace(-3, 3, 1500),
                         [0.0, -0.0, 1.0, 88.7, -87.3, 1e-30, 3e38]]).astype(np.float32)
    pos = np.concatenate([np.abs(xs) + np.float32(1e-6), [1.0, 1e-40, 2816.0, 704.0]]).astype(np.float32)
    np.savez_compressed(
        os.path.join(OUT, "bitmath.npz"), xs=xs, pos=pos,
        expf=ref.map_f32("expf", xs), tanhf=ref.map_f32("tanhf", xs),
        gelu_tanh=ref.map_f32("gelu_tanh", xs),
        rsqrtf=ref.map_f32("rsqrtf", pos), sqrtf=ref.map_f32("sqrtf", pos))

    # --- Q4 matvec: small cases with inputs stored ---------------------
    q4 = {}
    for i, (R, C, B) in enumerate([(64, 64, 1), (8, 200, 1), (3, 32, 2), (16, 2816, 3),
                                   (40, 704, 5), (2, 8192, 1), (33, 128, 4)]):
        n = R * C
        vals = rng.integers(0, 2**32, (n + 7) // 8, dtype=np.uint32)
        ng = (n + 63) // 64
        s = synth.bf16_round(rng.uniform(0.005, 0.02, ng).astype(np.float32))
        b = synth.bf16_round(np.float32(-8.0) * synth.bf16_to_f32(s))
        x = rng.standard_normal((B, C)).astype(np.float32)
        y = np.stack([ref.q4_matvec(vals, s, b, R, C, x[t]) for t in range(B)])
        if C % 64 == 0 and R >= 16:
            # the batch form must agree with the single-vector form bit for bit
            # (tools/test/gemma4-bit-identity-test.c).  It is only consulted for
            # R >= its worker count: below that the reference's x86 batch path
            # leaves trailing rows unwritten.
            assert (ref.q4_matvec_batch(vals, s, b, R, C, x).view(np.uint32) == y.view(np.uint32)).all()
        q4.update({f"c{i}_shape": np.array([R, C, B]), f"c{i}_vals": vals, f"c{i}_scales": s,
                   f"c{i}_biases": b, f"c{i}_x": x, f"c{i}_y": y})
    q4["n_cases"] = np.array(7)
    np.savez_compressed(os.path.join(OUT, "q4_matvec.npz"), **q4)

    # --- Q4 matvec at benchmark shapes: seed + output only -------------
    big = {}
    for name, (R, C, seed) in {"cfg1_4096x4096": (4096, 4096, 101), "gate_704x2816": (704, 2816, 102),
                               "down_2816x704": (2816, 704, 103), "odd_705x2816": (705, 2816, 104)}.items():
        g = np.random.default_rng(seed)
        vals, s, b = synth.make_q4(g, R, C)
        x = g.standard_normal(C).astype(np.float32)
        big[name + "_y"] = ref.q4_matvec(vals, s, b, R, C, x)
        big[name + "_meta"] = np.array([R, C, seed])
    np.savez_compressed(os.path.join(OUT, "q4_matvec_seeded.npz"), **big)

    # --- router ----------------------------------------------------------
    H, E, K = 96, 24, 5
    x = rng.standard_normal((4, H)).astype(np.float32)
    x[3] *= 37.0
    scale = (1.0 + 0.25 * rng.standard_normal(H)).astype(np.float32)
    W = (rng.standard_normal((E, H)) * 0.02).astype(np.float32)
    W[7] = W[3]                                   # an exact tie: lower index must win
    pes = (1.0 + 0.1 * rng.standard_normal(E)).astype(np.float32)
    nw = (1.0 + 0.1 * rng.standard_normal(H)).astype(np.float32)
    rin, logits, sel, wts, sel_rank, wts_rank, norm = [], [], [], [], [], [], []
    for t in range(4):
        rc, ri = ref.router_input(x[t], scale, 1e-6); assert rc == 0
        lg = ref.router_scores(W, None, ri)
        rc, s_, w_ = ref.router_topk(lg, pes, K, sort_by_expert=True); assert rc == 0
        rc, s2, w2 = ref.router_topk(lg, pes, K, sort_by_expert=False); assert rc == 0
        rc, nm = ref.rmsnorm(x[t], nw, 1e-6, True); assert rc == 0
        rin.append(ri); logits.append(lg); sel.append(s_); wts.append(w_)
        sel_rank.append(s2); wts_rank.append(w2); norm.append(nm)
    np.savez_compressed(os.path.join(OUT, "router.npz"), x=x, scale=scale, W=W, pes=pes, nw=nw,
                        rin=np.stack(rin), logits=np.stack(logits), sel=np.stack(sel),
                        wts=np.stack(wts), sel_rank=np.stack(sel_rank), wts_rank=np.stack(wts_rank),
                        norm=np.stack(norm), topk=np.array(K), eps=np.float32(1e-6))

    # --- grouping / reduction -----------------------------------------
    rows, topk, ne, hid = 7, 3, 9, 5
    selected = np.stack([rng.permutation(ne)[:topk] for _ in range(rows)]).astype(np.int32)
    selected.sort(axis=1)
    rin_ = rng.standard_normal((rows, hid)).astype(np.float32)
    rc, offs, g2c, c2g, routed = ref.route_group(selected.ravel(), rows, topk, ne, rin_); assert rc == 0
    gout = rng.standard_normal((rows * topk, hid)).astype(np.float32)
    gw = rng.uniform(0.05, 0.5, rows * topk).astype(np.float32)
    rc, red = ref.weighted_reduce(gw, c2g, gout, rows, topk); assert rc == 0
    np.savez_compressed(os.path.join(OUT, "grouping.npz"), selected=selected, row_inputs=rin_, offs=offs,
                        g2c=g2c, c2g=c2g, routed=routed, grouped_outputs=gout, weights=gw, reduced=red,
                        n_experts=np.array(ne))

    # --- NVFP4 -------------------------------------------------------------
    R, C = 12, 96
    wf = (rng.standard_normal((R, C)) * 0.02).astype(np.float32)
    enc = np.array([ref.e4m3fn_encode(float(v))[1] for v in np.linspace(-500, 500, 4001).astype(np.float32)], np.uint8)
    dec = np.array([ref.e4m3fn(c) for c in range(256)], np.float32)
    xin = np.stack([rng.standard_normal(C), rng.standard_normal(C) * 40, np.zeros(C),
                    rng.standard_normal(C) * 1e-3]).astype(np.float32)
    # weights quantised with the reference's own encoders (divisor chosen so the
    # largest block scale sits near the top of the e4m3 range)
    amax = np.abs(wf).reshape(R, C // 16, 16).max(axis=2)
    divisor = np.float32(448.0 * 6.0 / np.abs(wf).max())
    wscale = np.array([[ref.e4m3fn_encode(float(np.float32(a / 6.0) * divisor))[1] for a in row] for row in amax], np.uint8)
    codes = np.zeros((R, C), np.uint8)
    e2 = np.array([ref.e2m1(c) for c in range(16)], np.float32)
    for r in range(R):
        for c in range(C):
            sc = np.float32(ref.e4m3fn(int(wscale[r, c // 16]))) / divisor
            t = 0.0 if sc == 0 else float(wf[r, c]) / float(sc)
            codes[r, c] = int(np.argmin(np.abs(e2 - np.float32(np.clip(t, -6, 6)))))
    wpacked = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    qp, qs, qd, ys = [], [], [], []
    for t in range(4):
        rc, p, s, d = ref.nvfp4_qdq(xin[t], 64.0); assert rc == 0
        rc, y = ref.nvfp4_matvec(wpacked, wscale, float(divisor), 64.0, R, C, xin[t]); assert rc == 0
        qp.append(p); qs.append(s); qd.append(d); ys.append(y)
    rc, wdq = ref.nvfp4_dequant_weights(wpacked, wscale, float(divisor), R, C); assert rc == 0
    np.savez_compressed(os.path.join(OUT, "nvfp4.npz"), enc_in=np.linspace(-500, 500, 4001).astype(np.float32),
                        enc=enc, dec=dec, x=xin, qdq_packed=np.stack(qp), qdq_scales=np.stack(qs),
                        qdq_dequant=np.stack(qd), wpacked=wpacked, wscale=wscale, divisor=divisor,
                        input_global=np.float32(64.0), y=np.stack(ys), wdq=wdq)

    # --- whole MoE layer, small geometry: seed + outputs -------------------
    layer = synth.make_q4_moe_layer(7, hidden=256, inter=128, n_experts=16, topk=4)
    xt = synth.make_tokens(8, 6, 256)
    y, sel_, w_ = ref.moe_layer_q4(layer, xt, threads=4)
    np.savez_compressed(os.path.join(OUT, "moe_layer_small.npz"), y=y, sel=sel_, w=w_,
                        meta=np.array([7, 8, 6, 256, 128, 16, 4]))
    gen_cells(ref)
    print("golden fixtures written to", OUT)


if __name__ == "__main__":
    main()
