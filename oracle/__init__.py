"""CPU checkers for the quantized MoE feed-forward path.  TEST INFRASTRUCTURE ONLY.

Two ctypes front-ends with the same method names:

* ``Oracle``    -- ``liboracle.so``, our own C99 restatement (``salt_oracle.c``).
* ``Reference`` -- ``_ref/libsalt_ref.so``, the reference project's own sources
  compiled unmodified by ``oracle/Makefile`` (present only where that build ran).

Only ``tests/``, the smoke check and the CPU legs of ``bench.py`` may import this
package; the shipped library never does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libsalt_ref.so")


def build(quiet: bool = True) -> None:
    """Compile liboracle.so (always) and _ref/libsalt_ref.so (when the reference
    checkout is mounted).  Building the checker is not using it."""
    subprocess.run(["make", "-C", HERE, "all"], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def _p(a, ctype=C.c_void_p):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(ctype)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


class MoeLayerDesc(C.Structure):
    _fields_ = [("hidden", C.c_int), ("inter", C.c_int), ("n_experts", C.c_int),
                ("topk", C.c_int), ("eps", C.c_float),
                ("router_w", C.c_void_p), ("router_scale", C.c_void_p),
                ("per_expert_scale", C.c_void_p), ("pool", C.c_void_p),
                ("expert_stride", C.c_size_t)]


class Oracle:
    """liboracle.so: every method returns fresh numpy arrays."""

    kind = "port"

    def __init__(self, path: str = ORACLE_SO):
        if not os.path.exists(path):
            build()
        self.lib = C.CDLL(path)
        L = self.lib
        for name in ("orc_expf", "orc_rsqrtf", "orc_sqrtf", "orc_tanhf", "orc_gelu_tanh"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [C.c_float]
        L.orc_e2m1.restype = C.c_float
        L.orc_e2m1.argtypes = [C.c_uint8]
        L.orc_e4m3fn.restype = C.c_float
        L.orc_e4m3fn.argtypes = [C.c_uint8]

    # -- scalar math -------------------------------------------------
    def expf(self, x): return self.lib.orc_expf(float(np.float32(x)))
    def rsqrtf(self, x): return self.lib.orc_rsqrtf(float(np.float32(x)))
    def sqrtf(self, x): return self.lib.orc_sqrtf(float(np.float32(x)))
    def tanhf(self, x): return self.lib.orc_tanhf(float(np.float32(x)))
    def gelu_tanh(self, x): return self.lib.orc_gelu_tanh(float(np.float32(x)))

    def map_f32(self, name, xs):
        fn = getattr(self.lib, "orc_" + name)
        xs = _f32(xs)
        return np.array([fn(float(v)) for v in xs.ravel()], dtype=np.float32).reshape(xs.shape)

    # -- Q4 ----------------------------------------------------------
    def q4_decode(self, vals, scales, biases, n):
        out = np.empty(n, np.float32)
        self.lib.orc_q4_decode(_p(vals), _p(scales), _p(biases), C.c_size_t(n), _p(out))
        return out

    def q4_matvec(self, vals, scales, biases, R, Ccols, x, threads=1):
        x = _f32(x)
        y = np.empty(R, np.float32)
        rc = self.lib.orc_q4_matvec(_p(vals), _p(scales), _p(biases), R, Ccols,
                                    _p(x), _p(y), threads)
        if rc:
            raise ValueError("orc_q4_matvec rejected its arguments")
        return y

    def q4_matvec_batch(self, vals, scales, biases, R, Ccols, xs, threads=1):
        xs = _f32(xs)
        B = xs.shape[0]
        ys = np.empty((B, R), np.float32)
        rc = self.lib.orc_q4_matvec_batch(_p(vals), _p(scales), _p(biases), R, Ccols, B,
                                          _p(xs), _p(ys), threads)
        if rc:
            raise ValueError("orc_q4_matvec_batch rejected its arguments")
        return ys

    # -- router ------------------------------------------------------
    def rmsnorm(self, x, weight, eps, with_scale=True):
        x = _f32(x)
        out = np.empty_like(x)
        w = _f32(weight) if weight is not None else None
        rc = self.lib.orc_rmsnorm(_p(out), _p(x), _p(w), x.size, C.c_float(eps),
                                  1 if with_scale else 0)
        return rc, out

    def bf16_matvec(self, W, R, Ccols, x, bias=None):
        y = np.empty(R, np.float32)
        self.lib.orc_bf16_matvec(_p(W), R, Ccols, _p(_f32(x)), _p(_f32(bias)) if bias is not None else None, _p(y))
        return y

    def bf16_matvec_serial(self, W, R, Ccols, xs):
        xs = _f32(xs).reshape(-1, Ccols)
        ys = np.empty((xs.shape[0], R), np.float32)
        self.lib.orc_bf16_matvec_serial(_p(W), R, Ccols, xs.shape[0], _p(xs), _p(ys))
        return ys

    def q8_matvec(self, vals, scales, biases, R, Ccols, x):
        y = np.empty(R, np.float32)
        self.lib.orc_q8_matvec(_p(vals), _p(scales), _p(biases) if biases is not None else None, R, Ccols,
                               _p(_f32(x)), _p(y))
        return y

    def residual_postnorm(self, residual, branch, weight, eps):
        residual = _f32(residual)
        out = np.empty_like(residual)
        rc = self.lib.orc_residual_postnorm(_p(out), _p(residual), _p(_f32(branch)), _p(_f32(weight)),
                                            residual.size, C.c_float(eps))
        return rc, out

    def parallel_ffn_combine(self, residual, dense, routed, dense_w, routed_w, final_w, scalar, eps):
        residual = _f32(residual)
        out = np.empty_like(residual)
        scratch = np.empty(2 * residual.size, np.float32)
        rc = self.lib.orc_parallel_ffn_combine(_p(out), _p(residual), _p(_f32(dense)), _p(_f32(routed)),
                                               _p(_f32(dense_w)), _p(_f32(routed_w)), _p(_f32(final_w)),
                                               C.c_float(scalar), residual.size, C.c_float(eps), _p(scratch))
        return rc, out, scratch

    def softcap(self, logits, cap):
        out = _f32(logits).copy()
        rc = self.lib.orc_softcap(_p(out), out.size, C.c_float(cap))
        return rc, out

    def router_input(self, x, scale, eps):
        x = _f32(x)
        out = np.empty_like(x)
        rc = self.lib.orc_router_input(_p(out), _p(x), _p(_f32(scale)), x.size, C.c_float(eps))
        return rc, out

    def router_scores(self, W, bias, x):
        W = _f32(W)
        E, H = W.shape
        out = np.empty(E, np.float32)
        b = _f32(bias) if bias is not None else None
        self.lib.orc_router_scores(_p(W), _p(b), E, H, _p(_f32(x)), _p(out))
        return out

    def router_topk(self, logits, per_expert_scale, topk, sort_by_expert=True):
        logits = _f32(logits)
        sel = np.empty(topk, np.int32)
        w = np.empty(topk, np.float32)
        pes = _f32(per_expert_scale) if per_expert_scale is not None else None
        rc = self.lib.orc_router_topk(_p(logits), _p(pes), logits.size, topk, _p(sel), _p(w),
                                      1 if sort_by_expert else 0)
        return rc, sel, w

    # -- grouping ----------------------------------------------------
    def route_group(self, selected, rows, topk, n_experts, row_inputs=None):
        selected = np.ascontiguousarray(selected, np.int32)
        jobs = rows * topk
        offs = np.zeros(n_experts, np.uint32)
        g2c = np.empty(jobs, np.int32)
        c2g = np.empty(jobs, np.int32)
        hidden = 0
        routed = None
        if row_inputs is not None:
            row_inputs = _f32(row_inputs)
            hidden = row_inputs.shape[1]
            routed = np.empty((jobs, hidden), np.float32)
        rc = self.lib.orc_route_group(_p(selected), rows, topk, n_experts, _p(row_inputs), hidden,
                                      _p(offs), _p(g2c), _p(c2g), _p(routed))
        return rc, offs, g2c, c2g, routed

    def weighted_reduce(self, weights, c2g, grouped_outputs, rows, topk):
        grouped_outputs = _f32(grouped_outputs)
        width = grouped_outputs.shape[1]
        out = np.empty((rows, width), np.float32)
        rc = self.lib.orc_weighted_reduce(_p(_f32(weights)), _p(np.ascontiguousarray(c2g, np.int32)),
                                          _p(grouped_outputs), rows, topk, width, _p(out))
        return rc, out

    # -- MoE layer ---------------------------------------------------
    def moe_layer_q4(self, layer, x, threads=1):
        """layer: object with hidden, inter, n_experts, topk, eps, router_w,
        router_scale, per_expert_scale, pool (uint8 array), expert_stride."""
        x = _f32(x).reshape(-1, layer.hidden)
        B = x.shape[0]
        d = MoeLayerDesc(layer.hidden, layer.inter, layer.n_experts, layer.topk, layer.eps,
                         layer.router_w.ctypes.data, layer.router_scale.ctypes.data,
                         layer.per_expert_scale.ctypes.data, layer.pool.ctypes.data,
                         layer.expert_stride)
        y = np.empty((B, layer.hidden), np.float32)
        sel = np.empty((B, layer.topk), np.int32)
        w = np.empty((B, layer.topk), np.float32)
        rc = self.lib.orc_moe_layer_q4(C.byref(d), _p(x), B, _p(y), _p(sel), _p(w), threads)
        if rc:
            raise ValueError("orc_moe_layer_q4 failed")
        return y, sel, w

    # -- NVFP4 -------------------------------------------------------
    def e2m1(self, code): return self.lib.orc_e2m1(code)
    def e4m3fn(self, code): return self.lib.orc_e4m3fn(code)

    def e4m3fn_encode(self, value):
        code = C.c_uint8(0)
        rc = self.lib.orc_e4m3fn_encode(C.c_float(value), C.byref(code))
        return rc, code.value

    def nvfp4_qdq(self, x, input_global_scale):
        x = _f32(x)
        n = x.size
        packed = np.empty(n // 2, np.uint8)
        scales = np.empty(n // 16, np.uint8)
        dq = np.empty(n, np.float32)
        rc = self.lib.orc_nvfp4_qdq(_p(x), n, C.c_float(input_global_scale),
                                    _p(packed), _p(scales), _p(dq))
        return rc, packed, scales, dq

    def nvfp4_dequant_weights(self, packed, scales, divisor, R, Ccols):
        out = np.empty((R, Ccols), np.float32)
        rc = self.lib.orc_nvfp4_dequant_weights(_p(packed), _p(scales), C.c_float(divisor),
                                                R, Ccols, _p(out))
        return rc, out

    def nvfp4_matvec(self, packed, scales, divisor, input_global_scale, R, Ccols, x, threads=1):
        x = _f32(x)
        y = np.empty(R, np.float32)
        xp = np.empty(Ccols // 2, np.uint8)
        xs = np.empty(Ccols // 16, np.uint8)
        xdq = np.empty(Ccols, np.float32)
        rc = self.lib.orc_nvfp4_matvec(_p(packed), _p(scales), C.c_float(divisor),
                                       C.c_float(input_global_scale), R, Ccols, _p(x), _p(y),
                                       _p(xp), _p(xs), _p(xdq), threads)
        return rc, y


def moe_layer_nvfp4(impl, layer, x, threads=1):
    """One MoE layer with NVFP4 experts composed from `impl`'s functions (an Oracle or a Reference):
    router input -> logits -> softmax top-k sorted by expert (models/gemma4-26b-a4b/src/gemma4.c:103-186,
    gemma4_text.c:8541-8550); per selection the W4A4 gate and up projections, GeGLU, the W4A4 down
    projection (src/nvfp4.c:228-256; caller gemma4_text.c:8912-8945); ordered weighted reduce in rank order
    from +0 (src/moe_group.c:211-224).  Returns (y, selected, weights)."""
    x = _f32(x).reshape(-1, layer.hidden)
    B, H, M, K = x.shape[0], layer.hidden, layer.inter, layer.topk
    y = np.zeros((B, H), np.float32)
    sel_all = np.empty((B, K), np.int32)
    w_all = np.empty((B, K), np.float32)
    for t in range(B):
        rc, rin = impl.router_input(x[t], layer.router_scale, layer.eps)
        assert rc == 0
        rc, sel, w = impl.router_topk(impl.router_scores(layer.router_w, None, rin), layer.per_expert_scale, K, True)
        assert rc == 0
        sel_all[t], w_all[t] = sel, w
        acc = np.zeros(H, np.float32)
        for rank in range(K):
            e = int(sel[rank])
            outs = []
            for which in (0, 1):
                codes, sc, dv, ig, R, Cc = layer.tensor(e, which)
                rc, o = impl.nvfp4_matvec(codes, sc, dv, ig, R, Cc, x[t], threads=threads)
                assert rc == 0
                outs.append(o)
            chain = (impl.map_f32("gelu_tanh", outs[0]) * outs[1]).astype(np.float32)
            codes, sc, dv, ig, R, Cc = layer.tensor(e, 2)
            rc, o = impl.nvfp4_matvec(codes, sc, dv, ig, R, Cc, chain, threads=threads)
            assert rc == 0
            acc = (acc + (np.float32(w[rank]) * o).astype(np.float32)).astype(np.float32)
        y[t] = acc
    return y, sel_all, w_all


class Reference:
    """_ref/libsalt_ref.so: the reference project's own functions."""

    kind = "reference"

    def __init__(self, path: str = REF_SO):
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = C.CDLL(path)
        L = self.lib
        for name in ("salt_expf", "salt_rsqrtf", "salt_sqrtf", "salt_tanhf",
                     "salt_gemma4_gelu_tanh"):
            getattr(L, name).restype = C.c_float
            getattr(L, name).argtypes = [C.c_float]
        L.salt_nvfp4_e2m1.restype = C.c_float
        L.salt_nvfp4_e2m1.argtypes = [C.c_uint8]
        L.salt_nvfp4_e4m3fn.restype = C.c_float
        L.salt_nvfp4_e4m3fn.argtypes = [C.c_uint8]
        L.salt_q4_matvec.restype = None

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_SO)

    def map_f32(self, name, xs):
        fn = getattr(self.lib, {"expf": "salt_expf", "rsqrtf": "salt_rsqrtf",
                                "sqrtf": "salt_sqrtf", "tanhf": "salt_tanhf",
                                "gelu_tanh": "salt_gemma4_gelu_tanh"}[name])
        xs = _f32(xs)
        return np.array([fn(float(v)) for v in xs.ravel()], dtype=np.float32).reshape(xs.shape)

    def set_simd(self, on: bool):
        self.lib.salt_kernels_set_simd(1 if on else 0)

    def set_expert_scope(self, on: bool):
        """Inside an 'expert scope' the reference never spawns its own row
        threads (src/kernels.c:294-297); used when the caller partitions rows."""
        self.lib.salt_kernels_set_cpu_expert_scope(1 if on else 0)

    def q4_matvec(self, vals, scales, biases, R, Ccols, x, threads=None):
        x = _f32(x)
        y = np.empty(R, np.float32)
        rc = self.lib.salt_q4_matvec_status(_p(vals), _p(scales), _p(biases), R, Ccols, _p(x), _p(y))
        if rc:
            raise ValueError("salt_q4_matvec_status failed")
        return y

    def q4_matvec_rows(self, vals, scales, biases, R, Ccols, x, y, r0, r1):
        """salt_simd_q4_matvec on rows [r0, r1) writing into y (include/salt/simd.h:60-62)."""
        self.lib.salt_simd_q4_matvec(_p(vals), _p(scales), _p(biases), R, Ccols, _p(x), _p(y), r0, r1)

    def q4_matvec_batch(self, vals, scales, biases, R, Ccols, xs, threads=None):
        xs = _f32(xs)
        B = xs.shape[0]
        ys = np.empty((B, R), np.float32)
        rc = self.lib.salt_q4_matvec_batch(_p(vals), _p(scales), _p(biases), R, Ccols, B, _p(xs), _p(ys))
        if rc:
            raise ValueError("salt_q4_matvec_batch failed")
        return ys

    def q4_decode(self, vals, scales, biases, n):
        out = np.empty(n, np.float32)
        self.lib.salt_q4_decode(_p(vals), _p(scales), _p(biases), n, _p(out))
        return out

    def rmsnorm(self, x, weight, eps, with_scale=True):
        x = _f32(x)
        out = np.empty_like(x)
        w = _f32(weight) if weight is not None else None
        rc = self.lib.salt_gemma4_rmsnorm(_p(out), _p(x), _p(w), x.size, C.c_float(eps),
                                          1 if with_scale else 0)
        return rc, out

    def bf16_matvec(self, W, R, Ccols, x, bias=None):
        y = np.empty(R, np.float32)
        self.lib.salt_bf16_matvec(_p(W), R, Ccols, _p(_f32(x)), _p(_f32(bias)) if bias is not None else None, _p(y))
        return y

    def f32_matvec(self, W, R, Ccols, x):
        """salt_f32_matvec (src/kernels.c:98-116): the serial column chain."""
        y = np.empty(R, np.float32)
        self.lib.salt_f32_matvec(_p(_f32(W)), R, Ccols, _p(_f32(x)), _p(y))
        return y

    def q8_matvec(self, vals, scales, biases, R, Ccols, x):
        y = np.empty(R, np.float32)
        self.lib.salt_q8_matvec(_p(vals), _p(scales), _p(biases) if biases is not None else None, R, Ccols,
                               _p(_f32(x)), _p(y))
        return y

    def residual_postnorm(self, residual, branch, weight, eps):
        residual = _f32(residual)
        out = np.empty_like(residual)
        rc = self.lib.salt_gemma4_residual_postnorm(_p(out), _p(residual), _p(_f32(branch)), _p(_f32(weight)),
                                            residual.size, C.c_float(eps))
        return rc, out

    def parallel_ffn_combine(self, residual, dense, routed, dense_w, routed_w, final_w, scalar, eps):
        residual = _f32(residual)
        out = np.empty_like(residual)
        scratch = np.empty(2 * residual.size, np.float32)
        rc = self.lib.salt_gemma4_parallel_ffn_combine(_p(out), _p(residual), _p(_f32(dense)), _p(_f32(routed)),
                                               _p(_f32(dense_w)), _p(_f32(routed_w)), _p(_f32(final_w)),
                                               C.c_float(scalar), residual.size, C.c_float(eps), _p(scratch))
        return rc, out, scratch

    def softcap(self, logits, cap):
        out = _f32(logits).copy()
        rc = self.lib.salt_gemma4_softcap(_p(out), out.size, C.c_float(cap))
        return rc, out

    def router_input(self, x, scale, eps):
        x = _f32(x)
        out = np.empty_like(x)
        rc = self.lib.salt_gemma4_router_input(_p(out), _p(x), _p(_f32(scale)), x.size, C.c_float(eps))
        return rc, out

    def router_scores(self, W, bias, x):
        W = _f32(W)
        E, H = W.shape
        out = np.empty(E, np.float32)
        b = _f32(bias) if bias is not None else None
        self.lib.salt_router_scores(_p(W), _p(b), E, H, _p(_f32(x)), _p(out))
        return out

    def router_topk(self, logits, per_expert_scale, topk, sort_by_expert=True):
        logits = _f32(logits)
        sel = np.empty(topk, np.int32)
        w = np.empty(topk, np.float32)
        rc = self.lib.salt_gemma4_router_topk(_p(logits), _p(_f32(per_expert_scale)),
                                              logits.size, topk, _p(sel), _p(w))
        if rc == 0 and sort_by_expert:
            # the adapter's own exchange sort (gemma4_text.c:8541-8550)
            for a in range(topk):
                for b in range(a + 1, topk):
                    if sel[b] < sel[a]:
                        sel[a], sel[b] = sel[b], sel[a]
                        w[a], w[b] = w[b], w[a]
        return rc, sel, w

    def route_group(self, selected, rows, topk, n_experts, row_inputs):
        selected = np.ascontiguousarray(selected, np.int32)
        row_inputs = _f32(row_inputs)
        hidden = row_inputs.shape[1]
        jobs = rows * topk
        offs = np.zeros(n_experts, np.uint32)
        g2c = np.empty(jobs, np.int32)
        c2g = np.empty(jobs, np.int32)
        routed = np.empty((jobs, hidden), np.float32)
        rc = self.lib.salt_tensor_selected_route_group(
            _p(selected), rows, topk, n_experts, _p(row_inputs), hidden,
            _p(offs), n_experts, _p(g2c), _p(c2g), _p(routed))
        return rc, offs, g2c, c2g, routed

    def weighted_reduce(self, weights, c2g, grouped_outputs, rows, topk):
        grouped_outputs = _f32(grouped_outputs)
        width = grouped_outputs.shape[1]
        out = np.empty((rows, width), np.float32)
        rc = self.lib.salt_tensor_selected_weighted_reduce(
            _p(_f32(weights)), _p(np.ascontiguousarray(c2g, np.int32)), _p(grouped_outputs),
            rows, topk, width, _p(out))
        return rc, out

    def e2m1(self, code): return self.lib.salt_nvfp4_e2m1(code)
    def e4m3fn(self, code): return self.lib.salt_nvfp4_e4m3fn(code)

    def e4m3fn_encode(self, value):
        code = C.c_uint8(0)
        rc = self.lib.salt_nvfp4_e4m3fn_encode(C.c_float(value), C.byref(code))
        return rc, code.value

    def nvfp4_qdq(self, x, input_global_scale):
        x = _f32(x)
        n = x.size
        packed = np.empty(n // 2, np.uint8)
        scales = np.empty(n // 16, np.uint8)
        dq = np.empty(n, np.float32)
        rc = self.lib.salt_nvfp4_quantize_input_reference(
            _p(x), n, C.c_float(input_global_scale), _p(packed), _p(scales), _p(dq))
        return rc, packed, scales, dq

    def nvfp4_dequant_weights(self, packed, scales, divisor, R, Ccols):
        out = np.empty((R, Ccols), np.float32)
        rc = self.lib.salt_nvfp4_dequantize_weights_reference(
            _p(packed), _p(scales), C.c_float(divisor), R, Ccols, _p(out))
        return rc, out

    def nvfp4_matvec(self, packed, scales, divisor, input_global_scale, R, Ccols, x, threads=None):
        x = _f32(x)
        y = np.empty(R, np.float32)
        xp = np.empty(Ccols // 2, np.uint8)
        xs = np.empty(Ccols // 16, np.uint8)
        xdq = np.empty(Ccols, np.float32)
        rc = self.lib.salt_nvfp4_matvec_reference(
            _p(packed), _p(scales), C.c_float(divisor), C.c_float(input_global_scale),
            R, Ccols, _p(x), _p(y), _p(xp), _p(xs), _p(xdq))
        return rc, y

    def moe_layer_q4(self, layer, x, threads=1):
        """The reference's decode chain (gemma4_text.c:8344-8363, 7908-8064)
        composed from its own functions; rows are partitioned over a Python
        thread pool (ctypes releases the GIL), which changes ownership only."""
        from concurrent.futures import ThreadPoolExecutor
        x = _f32(x).reshape(-1, layer.hidden)
        B, H, M, K = x.shape[0], layer.hidden, layer.inter, layer.topk
        y = np.zeros((B, H), np.float32)
        sel = np.empty((B, K), np.int32)
        w = np.empty((B, K), np.float32)
        for t in range(B):
            rc, rin = self.router_input(x[t], layer.router_scale, layer.eps)
            assert rc == 0
            logits = self.router_scores(layer.router_w, None, rin)
            rc, sel[t], w[t] = self.router_topk(logits, layer.per_expert_scale, K)
            assert rc == 0
        self.set_expert_scope(True)
        threads = max(1, threads)
        with ThreadPoolExecutor(threads) as pool:
            def rows(tensor, R, Ccols, xin, out):
                v, s, b = tensor
                step = -(-R // threads)
                futs = [pool.submit(self.q4_matvec_rows, v, s, b, R, Ccols, xin, out, r0, min(R, r0 + step))
                        for r0 in range(0, R, step)]
                for f in futs:
                    f.result()
            gate = np.empty(M, np.float32)
            up = np.empty(M, np.float32)
            down = np.empty(H, np.float32)
            for t in range(B):
                for j in range(K):
                    e = int(sel[t, j])
                    rows(layer.tensor(e, 0), M, H, x[t], gate)
                    rows(layer.tensor(e, 1), M, H, x[t], up)
                    chain = self.map_f32("gelu_tanh", gate) * up
                    rows(layer.tensor(e, 2), H, M, chain, down)
                    y[t] = y[t] + down * w[t, j]
        self.set_expert_scope(False)
        return y, sel, w


REF_DRIVER_SO = os.path.join(HERE, "_ref", "libref_driver.so")


class RefDriver:
    """_ref/libref_driver.so: the reference's own decode-path functions driven by
    a persistent pthread pool (oracle/ref_driver.c).  Used as the timed CPU
    baseline; only available where oracle/_ref was built."""

    kind = "reference"

    def __init__(self, threads: int):
        if not os.path.exists(REF_DRIVER_SO):
            raise FileNotFoundError(REF_DRIVER_SO)
        self.lib = C.CDLL(REF_DRIVER_SO)
        self.threads = int(self.lib.refdrv_pool_start(int(threads)))

    @staticmethod
    def available() -> bool:
        return os.path.exists(REF_DRIVER_SO)

    def moe_layer_q4(self, layer, x, threads=None):
        x = _f32(x).reshape(-1, layer.hidden)
        B = x.shape[0]
        d = MoeLayerDesc(layer.hidden, layer.inter, layer.n_experts, layer.topk, layer.eps,
                         layer.router_w.ctypes.data, layer.router_scale.ctypes.data,
                         layer.per_expert_scale.ctypes.data, layer.pool.ctypes.data, layer.expert_stride)
        y = np.empty((B, layer.hidden), np.float32)
        sel = np.empty((B, layer.topk), np.int32)
        w = np.empty((B, layer.topk), np.float32)
        rc = self.lib.refdrv_moe_layer_q4(C.byref(d), _p(x), B, _p(y), _p(sel), _p(w))
        if rc:
            raise ValueError("refdrv_moe_layer_q4 failed")
        return y, sel, w

    def rmsnorm_rows(self, x, weight, eps):
        x = _f32(x)
        out = np.empty_like(x)
        rc = self.lib.refdrv_rmsnorm_rows(_p(out), _p(x), _p(_f32(weight)), x.shape[0], x.shape[1], C.c_float(eps))
        if rc:
            raise ValueError("refdrv_rmsnorm_rows failed")
        return out

    def close(self):
        self.lib.refdrv_pool_stop()
