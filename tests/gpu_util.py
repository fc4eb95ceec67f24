"""Helpers shared by the -m gpu tests: everything goes through the C ABI of
libsalt_gpu_b200.so; torch is used only to hold device memory."""
import ctypes as C
import importlib

import numpy as np


def backend_mod():
    return importlib.import_module("salt-core_b200.backend")


def stack_mod():
    return importlib.import_module("salt-core_b200.stack")


_gpu = None


def gpu():
    """One initialised backend per process; init failure is a hard error."""
    global _gpu
    if _gpu is None:
        g = backend_mod().SaltGpu()
        if g.init() != 0:
            raise RuntimeError("salt_gpu_init failed on a GPU box")
        _gpu = g
    return _gpu


def d2h(ptr, count, dtype):
    out = np.empty(count, dtype)
    rc = gpu().lib.salt_b200_read_device(C.c_void_p(out.ctypes.data), C.c_void_p(ptr), C.c_size_t(out.nbytes))
    assert rc == 0
    return out


def oracle_stack(orc, layers, x, threads=8):
    """CPU statement of the stacked path: y_l = MoE_l(x_l); x_{l+1} = RMSNorm_l(y_l)."""
    cur = np.ascontiguousarray(x, np.float32)
    taps = []
    for i, layer in enumerate(layers):
        y, sel, w = orc.moe_layer_q4(layer, cur, threads=threads)
        taps.append((sel, w))
        if i + 1 < len(layers):
            nxt = np.empty_like(y)
            for t in range(y.shape[0]):
                rc, nxt[t] = orc.rmsnorm(y[t], layer.norm_weight, layer.eps, True)
                assert rc == 0
            cur = nxt
        else:
            cur = y
    return cur, taps
