"""ctypes mirror of the reference GPU operator surface (reference
include/salt/gpu.h) as exported by libsalt_gpu_b200.so.  Method names drop the
``salt_gpu_`` prefix; arguments keep the reference's meaning and every method
returns the C return code (0 success, -1 unavailable/failed) so tests read like
the reference's own conformance tests."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import load_library

RESOURCE_ARENA, RESOURCE_TRUNK, RESOURCE_EXPERT_LAYER = 0, 1, 2
EXACT_RMSNORM, EXACT_TOPK, EXACT_ROUTER_INPUT = 1, 2, 6
EXACT_RESIDUAL_POSTNORM, EXACT_PARALLEL_COMBINE, EXACT_SOFTCAP = 3, 4, 5
ADDRESS_REGISTERED_PERSISTENT = 2


class BatchStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("arena_batches", "trunk_batches", "expert_layer_batches",
                                          "mapped_only_misses", "direct_output_batches",
                                          "direct_output_jobs")]


class WeightResourceUsage(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("described_bytes", "registered_bytes", "pageable_bytes",
                                          "active_window_bytes", "peak_window_bytes",
                                          "device_copied_weight_bytes")] + \
               [(n, C.c_uint32) for n in ("described_resources", "active_resources", "active_windows",
                                          "reserved")]


class SharedBuffer(C.Structure):
    _fields_ = [("contents", C.c_void_p), ("nbytes", C.c_size_t), ("backend", C.c_void_p)]

    def array(self, dtype=np.float32):
        n = self.nbytes // np.dtype(dtype).itemsize
        return np.ctypeslib.as_array(C.cast(self.contents, C.POINTER(C.c_uint8)), (self.nbytes,)).view(dtype)[:n]


class ExactCell(C.Structure):
    _fields_ = [("kind", C.c_int), ("views", C.POINTER(SharedBuffer) * 8), ("offsets", C.c_size_t * 8),
                ("n", C.c_uint32), ("aux", C.c_uint32), ("eps", C.c_float), ("scalar", C.c_float)]


class MoeExpert(C.Structure):
    _fields_ = [("gate_vals", C.c_void_p), ("gate_scales", C.c_void_p), ("gate_biases", C.c_void_p),
                ("gate_id", C.c_void_p), ("up_vals", C.c_void_p), ("up_scales", C.c_void_p),
                ("up_biases", C.c_void_p), ("up_id", C.c_void_p), ("down_vals", C.c_void_p),
                ("down_scales", C.c_void_p), ("down_biases", C.c_void_p), ("down_id", C.c_void_p),
                ("group", C.c_int), ("resource_slot", C.c_int), ("logical_resource_id", C.c_uint64)]


class ResidencyPlan(C.Structure):
    """``SaltGpuResidencyPlan`` (reference include/salt/gpu_residency.h:26-36)."""
    _fields_ = [("device_budget_bytes", C.c_uint64), ("permanent_bytes", C.c_uint64),
                ("slot_base_offset", C.c_uint64), ("slot_bytes", C.c_uint64), ("staging_bytes", C.c_uint64),
                ("slot_count", C.c_uint32), ("staging_count", C.c_uint32), ("device_alignment", C.c_uint32),
                ("flags", C.c_uint32)]


class ResidencyBackendOps(C.Structure):
    """``SaltGpuResidencyBackendOps`` (reference include/salt/gpu_residency.h:63-89)."""
    _fields_ = [("abi_version", C.c_uint32), ("ops_size", C.c_size_t),
                ("create", C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(ResidencyPlan))),
                ("staging", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint32, C.POINTER(C.c_void_p),
                                        C.POINTER(C.c_size_t))),
                ("populate", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint32, C.c_uint64, C.c_uint32, C.c_size_t,
                                         C.c_uint64)),
                ("poll", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint32, C.c_uint64, C.POINTER(C.c_int))),
                ("resolve", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint64, C.c_size_t, C.POINTER(C.c_size_t))),
                ("retire", C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint32, C.c_uint64)),
                ("destroy", C.CFUNCTYPE(C.c_int, C.c_void_p)),
                ("permanent_layout", C.c_void_p), ("permanent_span", C.c_void_p),
                ("permanent_copy", C.c_void_p), ("permanent_publish", C.c_void_p)]


class SelectedProjectionJob(C.Structure):
    _fields_ = [("vals", C.c_void_p), ("scales", C.c_void_p), ("biases", C.c_void_p), ("id", C.c_void_p),
                ("inputs", C.c_void_p), ("outputs", C.c_void_p), ("rows", C.c_int), ("cols", C.c_int),
                ("batch", C.c_int), ("resource_slot", C.c_int), ("logical_resource_id", C.c_uint64)]


def ptr(a):
    """Host address of a numpy array (or None)."""
    return None if a is None else C.c_void_p(a.ctypes.data)


def _ptr_array(arrs):
    return (C.c_void_p * len(arrs))(*[a.ctypes.data if hasattr(a, "ctypes") else a for a in arrs])


class SaltGpu:
    def __init__(self):
        self.lib = load_library()
        self.lib.salt_b200_launch_count.restype = C.c_uint64

    # lifecycle
    def init(self): return self.lib.salt_gpu_init()
    def free(self): return self.lib.salt_gpu_free()
    def sync(self): return self.lib.salt_gpu_sync()
    def set_defer(self, on): return self.lib.salt_gpu_set_defer(int(on))
    def set_mapped_only(self, on): self.lib.salt_gpu_set_mapped_only(int(on))
    def mapped_only(self): return self.lib.salt_gpu_mapped_only()
    def launch_count(self): return int(self.lib.salt_b200_launch_count())

    def batch_stats(self):
        s = BatchStats()
        self.lib.salt_gpu_batch_stats_get(C.byref(s))
        return s

    def weight_resource_usage(self):
        u = WeightResourceUsage()
        rc = self.lib.salt_gpu_weight_resource_usage(C.byref(u), C.sizeof(u))
        return rc, u

    # resources: `base` is a numpy array whose bytes are the resource
    def weight_resource_bind(self, kind, rid, base):
        return self.lib.salt_gpu_weight_resource_bind(kind, rid, ptr(base), C.c_size_t(base.nbytes))

    def weight_resource_unbind(self, kind, rid):
        return self.lib.salt_gpu_weight_resource_unbind(kind, rid)

    def expert_resource_bind(self, rid, base):
        return self.lib.salt_gpu_expert_resource_bind(rid, ptr(base), C.c_size_t(base.nbytes))

    def expert_resource_slot(self, rid, key, vals, scales, biases, R, Ccols):
        return self.lib.salt_gpu_expert_resource_slot(rid, C.c_void_p(key), ptr(vals), ptr(scales), ptr(biases),
                                                      R, Ccols)

    def expert_resource_unbind(self, rid):
        return self.lib.salt_gpu_expert_resource_unbind(rid)

    def weight_resource_slot(self, kind, rid, key, vals, scales, biases, bits, R, Ccols):
        return self.lib.salt_gpu_weight_resource_slot(kind, rid, C.c_void_p(key), ptr(vals), ptr(scales),
                                                      ptr(biases), bits, R, Ccols)

    def nvfp4_resource_slot(self, kind, rid, key, packed, scales, weight_global, input_global, R, Ccols):
        return self.lib.salt_gpu_nvfp4_resource_slot(kind, rid, C.c_void_p(key), ptr(packed), ptr(scales),
                                                     ptr(weight_global), ptr(input_global), R, Ccols)

    def resident_trunk_map(self, base):
        return self.lib.salt_gpu_resident_trunk_map(ptr(base), C.c_size_t(base.nbytes))

    def resident_trunk_unmap(self): return self.lib.salt_gpu_resident_trunk_unmap()

    def selected_resources_prepare(self, capacity, logical_capacity):
        return self.lib.salt_gpu_selected_resources_prepare(capacity, logical_capacity)

    def selected_resource_bind(self, slot, logical_id, base, payload_offset=0):
        return self.lib.salt_gpu_selected_resource_bind(slot, C.c_uint64(logical_id), ptr(base),
                                                        C.c_size_t(base.nbytes),
                                                        C.c_void_p(base.ctypes.data + payload_offset))

    def selected_resource_bind_resident(self, slot, logical_id, payload, device_address, generation):
        """Publish a payload the residency engine already populated into seat ``slot`` (no copy)."""
        return self.lib.salt_gpu_selected_resource_bind_resident(
            slot, C.c_uint64(logical_id), ptr(payload), C.c_size_t(payload.nbytes),
            C.c_size_t(device_address), C.c_uint64(generation))

    def residency_backend_ops(self):
        """The physical residency operations (``ResidencyBackendOps``) for the reference's state machine."""
        self.lib.salt_gpu_residency_backend_ops.restype = C.POINTER(ResidencyBackendOps)
        return self.lib.salt_gpu_residency_backend_ops()

    def selected_resource_unbind(self, slot, logical_id):
        return self.lib.salt_gpu_selected_resource_unbind(slot, C.c_uint64(logical_id))

    def selected_resources_fence(self): return self.lib.salt_gpu_selected_resources_fence()

    # Q4 compute (host pointers)
    def q4_matvec(self, vals, scales, biases, R, Ccols, x, y):
        return self.lib.salt_gpu_q4_matvec(ptr(vals), ptr(scales), ptr(biases), R, Ccols, ptr(x), ptr(y))

    def q4_batch(self, vals, scales, biases, xs, ys, ids, Rj, Ccols):
        n = len(vals)
        rj = (C.c_int * n)(*Rj)
        return self.lib.salt_gpu_q4_batch(_ptr_array(vals), _ptr_array(scales), _ptr_array(biases),
                                          _ptr_array(xs), _ptr_array(ys), (C.c_void_p * n)(*ids), rj, Ccols, n)

    def bf16_resource_slot(self, kind, rid, key, weights, R, Ccols):
        return self.lib.salt_gpu_bf16_resource_slot(kind, rid, C.c_void_p(key), ptr(weights), R, Ccols)

    def bf16_matvec(self, key, R, Ccols, x, y):
        return self.lib.salt_gpu_bf16_matvec(C.c_void_p(key), R, Ccols, ptr(x), ptr(y))

    def bf16_matvec_batch(self, key, R, Ccols, B, xs, ys):
        return self.lib.salt_gpu_bf16_matvec_batch(C.c_void_p(key), R, Ccols, B, ptr(xs), ptr(ys))

    def q8_matvec(self, vals, scales, biases, R, Ccols, x, y):
        return self.lib.salt_gpu_q8_matvec(ptr(vals), ptr(scales), ptr(biases), R, Ccols, ptr(x), ptr(y))

    def q8_batch(self, vals, scales, biases, xs, ys, ids, Rj, Ccols):
        n = len(vals)
        rj = (C.c_int * n)(*Rj)
        return self.lib.salt_gpu_q8_batch(_ptr_array(vals), _ptr_array(scales), _ptr_array(biases),
                                          _ptr_array(xs), _ptr_array(ys), (C.c_void_p * n)(*ids), rj, Ccols, n)

    def proj_batch(self, vals, scales, biases, R, Ccols, xs, ys, key):
        """xs [B][C], ys [B][R] numpy arrays (row pointers are passed, as the reference does)."""
        B = xs.shape[0]
        xp = (C.c_void_p * B)(*[xs[b].ctypes.data for b in range(B)])
        yp = (C.c_void_p * B)(*[ys[b].ctypes.data for b in range(B)])
        return self.lib.salt_gpu_proj_batch(ptr(vals), ptr(scales), ptr(biases), R, Ccols, B, xp, yp,
                                            C.c_void_p(key))

    def proj_batch_indexed(self, vals, scales, biases, R, Ccols, B, first_job, job_count, xs, output,
                           y_float_offset, key):
        return self.lib.salt_gpu_proj_batch_indexed(ptr(vals), ptr(scales), ptr(biases), R, Ccols, B, first_job,
                                                    job_count, ptr(xs), C.byref(output),
                                                    C.c_size_t(y_float_offset), C.c_void_p(key))

    def q4_moe_chain(self, experts, hidden, routed, inputs, outputs, selected=False):
        arr = (MoeExpert * len(experts))(*experts)
        scratch = np.zeros(4, np.float32)
        fn = self.lib.salt_gpu_q4_moe_chain_selected if selected else self.lib.salt_gpu_q4_moe_chain
        return fn(arr, len(experts), hidden, routed, ptr(inputs), ptr(outputs), ptr(scratch), ptr(scratch),
                  C.c_size_t(scratch.size))

    def q4_selected_shared(self, jobs, arena):
        arr = (SelectedProjectionJob * len(jobs))(*jobs)
        return self.lib.salt_gpu_q4_selected_shared(arr, len(jobs), C.byref(arena))

    # NVFP4
    def nvfp4_qdq(self, x, input_global_scale, packed, scales, dequant):
        return self.lib.salt_gpu_nvfp4_qdq(ptr(x), x.size, C.c_float(input_global_scale), ptr(packed),
                                           ptr(scales), ptr(dequant))

    def nvfp4_matvec(self, key, R, Ccols, x, y):
        return self.lib.salt_gpu_nvfp4_matvec(C.c_void_p(key), R, Ccols, ptr(x), ptr(y))

    def nvfp4_matvec_batch(self, key, R, Ccols, xs, ys):
        return self.lib.salt_gpu_nvfp4_matvec_batch(C.c_void_p(key), R, Ccols, xs.shape[0], ptr(xs), ptr(ys))

    # shared buffers / exact cells
    def shared_buffer_alloc(self, nbytes):
        b = SharedBuffer()
        rc = self.lib.salt_gpu_shared_buffer_alloc(C.byref(b), C.c_size_t(nbytes))
        return rc, b

    def shared_buffer_free(self, b): return self.lib.salt_gpu_shared_buffer_free(C.byref(b))

    def exact_cells(self, cells):
        arr = (ExactCell * len(cells))(*cells)
        return self.lib.salt_gpu_exact_cells(arr, len(cells))


def exact_cell(kind, views, offsets, n, aux=0, eps=0.0, scalar=0.0):
    c = ExactCell()
    c.kind = kind
    for i, (v, o) in enumerate(zip(views, offsets)):
        c.views[i] = C.pointer(v)
        c.offsets[i] = o
    c.n, c.aux, c.eps, c.scalar = n, aux, eps, scalar
    return c
