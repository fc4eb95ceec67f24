"""The C-ABI library loads without a GPU and exports every symbol the header
declares, including every symbol of the reference's stub backend (no compute
call is made here)."""
import ctypes as C
import os
import re

from conftest import ROOT, load_package

# every function the reference's stub backend defines (reference src/gpu_stub.c:9-431)
REFERENCE_SURFACE = """
salt_gpu_residency_backend_ops salt_gpu_startup_requirements salt_gpu_init salt_gpu_free salt_gpu_q4_matvec
salt_gpu_q8_matvec salt_gpu_nvfp4_qdq salt_gpu_nvfp4_matvec salt_gpu_nvfp4_matvec_batch salt_gpu_nvfp4_batch
salt_gpu_nvfp4_mixed_batch salt_gpu_bf16_resource_slot salt_gpu_bf16_matvec salt_gpu_bf16_matvec_batch
salt_gpu_q4_batch salt_gpu_q8_batch salt_gpu_set_mapped_only salt_gpu_mapped_only salt_gpu_batch_stats_get
salt_gpu_batch_stats_get_v2 salt_gpu_proj_batch salt_gpu_shared_buffer_alloc salt_gpu_exact_cells
salt_gpu_shared_buffer_free salt_gpu_attention_batch salt_gpu_attention_prepare salt_gpu_attention_bind_kv
salt_gpu_attention_materialize salt_gpu_attention_import salt_gpu_attention_rewind salt_gpu_attention_transform
salt_gpu_q4_selected_shared salt_gpu_q4_moe_chain salt_gpu_q4_moe_chain_selected
salt_gpu_selected_resources_prepare salt_gpu_selected_resource_bind salt_gpu_selected_resource_bind_resident
salt_gpu_selected_resources_fence salt_gpu_selected_resource_unbind salt_gpu_proj_batch_indexed
salt_gpu_proj_batch_indexed_exact_views salt_gpu_resident_slot salt_gpu_expert_resource_bind
salt_gpu_expert_resource_slot salt_gpu_expert_resource_unbind salt_gpu_weight_resource_describe
salt_gpu_weight_resource_activate salt_gpu_weight_resource_pool_bind salt_gpu_weight_resource_deactivate
salt_gpu_weight_resource_usage salt_gpu_weight_resource_bind salt_gpu_weight_window_bind
salt_gpu_weight_window_unbind salt_gpu_weight_resource_slot salt_gpu_nvfp4_resource_slot
salt_gpu_weight_resource_unbind salt_gpu_resident_trunk_map salt_gpu_resident_trunk_unmap
salt_gpu_resident_pool_map salt_gpu_set_defer salt_gpu_defer salt_gpu_sync salt_gpu_tensor_program_ops
salt_dispatch_get salt_gpu_cuda_present salt_gpu_rocm_present salt_gpu_pageable_mmap_active
""".split()


def _declared():
    text = open(os.path.join(ROOT, "include", "salt_gpu_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(salt_(?:gpu|b200|dispatch)_[a-z0-9_]+|salt_dispatch_get)\s*\(", text)))


def test_library_loads_and_exports_every_declared_symbol():
    lib = load_package().load_library()
    names = _declared()
    assert len(names) > 70
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_reference_stub_surface_is_complete():
    lib = load_package().load_library()
    declared = set(_declared())
    for name in REFERENCE_SURFACE:
        assert name in declared, f"{name} not declared in include/salt_gpu_b200.h"
        assert hasattr(lib, name), f"{name} not exported"


def test_fail_closed_without_initialisation():
    """Before salt_gpu_init (and on a box with no GPU at all) operations return -1."""
    lib = load_package().load_library()
    assert lib.salt_gpu_q8_matvec(None, None, None, 1, 64, None, None) == -1
    assert lib.salt_gpu_attention_rewind(0) == -1
    assert lib.salt_gpu_tensor_program_ops() in (0, None)


def test_residency_operations_table():
    """The seven required residency operations are present (reference src/gpu_residency.c:70-76 rejects a
    table without them or with another size); creating a residency before salt_gpu_init fails closed."""
    import importlib
    bm = importlib.import_module("salt-core_b200.backend")
    lib = load_package().load_library()
    lib.salt_gpu_residency_backend_ops.restype = C.POINTER(bm.ResidencyBackendOps)
    ops = lib.salt_gpu_residency_backend_ops().contents
    assert ops.abi_version == 1 and ops.ops_size == C.sizeof(bm.ResidencyBackendOps) == 104
    for name in ("create", "staging", "populate", "poll", "resolve", "retire", "destroy"):
        assert getattr(ops, name)
    for name in ("permanent_layout", "permanent_span", "permanent_copy", "permanent_publish"):
        assert getattr(ops, name) is None
    plan = bm.ResidencyPlan(4096, 0, 0, 1024, 1024, 2, 1, 256, 0)
    assert ops.create(None, C.byref(plan)) == -1
    assert ops.destroy(None) == -1
    assert lib.salt_gpu_selected_resource_bind_resident(0, C.c_uint64(0), None, C.c_size_t(0), C.c_size_t(0),
                                                        C.c_uint64(0)) == -1
    lib.salt_gpu_cuda_present.restype = C.c_int
    assert lib.salt_gpu_cuda_present() == 1 and lib.salt_gpu_rocm_present() == 0
