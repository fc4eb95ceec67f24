"""Device-local expert residency: the reference's own residency state machine (src/gpu_residency.c, built
as oracle/_ref/libsalt_residency.so) drives the backend operations of libsalt_gpu_b200.so, the populated
seats are published with salt_gpu_selected_resource_bind_resident, and the selected expert chain computed
from them is compared with the CPU oracle (bit exact).  Flow as in the reference's caller,
models/gemma4-26b-a4b/src/gemma4_text.c:1886-1960."""
import ctypes as C
import os

import numpy as np
import pytest

from conftest import ROOT, assert_bits_equal
from gpu_util import backend_mod, gpu

pytestmark = pytest.mark.gpu

ENGINE = os.path.join(ROOT, "oracle", "_ref", "libsalt_residency.so")


class ResourceRef(C.Structure):      # reference include/salt/gpu_resource.h:16-22
    _fields_ = [("kind", C.c_uint32), ("resource_id", C.c_uint32), ("value_offset", C.c_uint64),
                ("scale_offset", C.c_uint64), ("bias_offset", C.c_uint64)]


READ_FN = C.CFUNCTYPE(C.c_int, C.c_void_p, C.c_uint64, C.c_void_p, C.c_size_t)


class Source(C.Structure):           # gpu_residency.h:42-49
    _fields_ = [("resource", ResourceRef), ("logical_resource_id", C.c_uint64), ("source_offset", C.c_uint64),
                ("nbytes", C.c_uint64), ("read", READ_FN), ("read_context", C.c_void_p)]


class Binding(C.Structure):          # gpu_residency.h:104-111
    _fields_ = [("logical_resource_id", C.c_uint64), ("generation", C.c_uint64), ("device_offset", C.c_uint64),
                ("nbytes", C.c_uint64), ("physical_slot", C.c_uint32), ("reserved", C.c_uint32)]


class Stats(C.Structure):            # gpu_residency.h:113-133
    _fields_ = [(n, C.c_uint64) for n in (
        "planned_device_bytes", "permanent_device_bytes", "slot_capacity_bytes", "staging_capacity_bytes",
        "population_submissions", "population_completions", "population_aborts", "population_bytes_submitted",
        "population_bytes_completed", "source_read_failures", "backend_failures", "retirements",
        "permanent_spans", "permanent_chunks", "permanent_bytes_populated")] + [
        (n, C.c_uint32) for n in ("ready_slots", "peak_ready_slots", "active_leases", "peak_active_leases")]


def _engine():
    if not os.path.exists(ENGINE):
        pytest.skip("oracle/_ref/libsalt_residency.so not built (needs the reference checkout at build time)")
    lib = C.CDLL(ENGINE)
    lib.salt_gpu_residency_arena_requirement.restype = C.c_size_t
    return lib


class Engine:
    """The reference state machine over our backend operations."""

    def __init__(self, plan):
        self.lib, self.g = _engine(), gpu()
        self.state = C.create_string_buffer(1024)          # SaltGpuResidency, opaque here (about 250 bytes)
        need = self.lib.salt_gpu_residency_arena_requirement(C.byref(plan))
        assert need > 0
        self.arena = C.create_string_buffer(need)
        self.ops = self.g.residency_backend_ops()
        assert self.lib.salt_gpu_residency_init(self.state, C.byref(plan), self.ops, None, self.arena,
                                                C.c_size_t(need)) == 0
        self.generation = 0
        self.keep = []

    def populate(self, seat, logical, payload, staging):
        """begin -> poll until READY -> acquire -> resolve; returns (device address, generation, binding)."""
        def read(_ctx, offset, dst, nbytes):
            if offset != 0 or nbytes != payload.nbytes:
                return -1
            C.memmove(dst, payload.ctypes.data, nbytes)
            return 0
        cb = READ_FN(read)
        self.keep.append(cb)
        src = Source()
        src.resource.kind, src.resource.resource_id = 2, logical       # SALT_GPU_RESOURCE_EXPERT_LAYER
        src.logical_resource_id, src.nbytes, src.read = logical, payload.nbytes, cb
        self.generation += 1
        gen, ticket = self.generation, C.c_uint64(0)
        assert self.lib.salt_gpu_residency_population_begin(self.state, seat, C.c_uint64(gen), C.byref(src),
                                                            staging, C.byref(ticket)) == 0
        for _ in range(10_000_000):
            rc = self.lib.salt_gpu_residency_population_poll(self.state, seat, C.c_uint64(logical),
                                                             C.c_uint64(gen), ticket)
            if rc != 0:
                break
        assert rc == 1
        b, addr = Binding(), C.c_size_t(0)
        assert self.lib.salt_gpu_residency_acquire(self.state, seat, C.c_uint64(logical), C.c_uint64(gen),
                                                   C.byref(b)) == 1
        assert self.lib.salt_gpu_residency_resolve(self.state, C.byref(b), C.byref(addr)) == 0
        return addr.value, gen, b

    def release(self, b):
        assert self.lib.salt_gpu_residency_release(self.state, C.byref(b)) == 0

    def retire(self, seat, logical, gen):
        return self.lib.salt_gpu_residency_retire(self.state, seat, C.c_uint64(logical), C.c_uint64(gen))

    def stats(self):
        s = Stats()
        assert self.lib.salt_gpu_residency_stats(self.state, C.byref(s), C.c_size_t(C.sizeof(s))) == 0
        return s

    def destroy(self):
        return self.lib.salt_gpu_residency_destroy(self.state)


def _expert(bm, layer, e, group, seat):
    def addr(a):
        return a.ctypes.data
    t = [layer.tensor(e, w) for w in range(3)]
    return bm.MoeExpert(addr(t[0][0]), addr(t[0][1]), addr(t[0][2]), addr(t[0][0]),
                        addr(t[1][0]), addr(t[1][1]), addr(t[1][2]), addr(t[1][0]),
                        addr(t[2][0]), addr(t[2][1]), addr(t[2][2]), addr(t[2][0]), group, seat, e)


def _chain_want(orc, layer, e, x, H, M):
    gate = orc.q4_matvec(*layer.tensor(e, 0), M, H, x)
    up = orc.q4_matvec(*layer.tensor(e, 1), M, H, x)
    return orc.q4_matvec(*layer.tensor(e, 2), H, M, orc.map_f32("gelu_tanh", gate) * up)


def test_resident_seats_feed_the_selected_chain(orc, synth):
    g, bm = gpu(), backend_mod()
    H, M, E = 256, 128, 8
    layer = synth.make_q4_moe_layer(61, hidden=H, inter=M, n_experts=E, topk=2)
    stride = layer.expert_stride
    seat_bytes = (stride + 255) // 256 * 256
    plan = bm.ResidencyPlan(1024 + 3 * seat_bytes, 1000, 1024, seat_bytes, seat_bytes, 3, 2, 256, 0)
    eng = Engine(plan)
    assert g.selected_resources_prepare(3, E) == 0
    payload = lambda e: layer.pool[e * stride:(e + 1) * stride]

    seats = {}                                   # seat -> (expert, generation)
    for seat, e in enumerate([5, 0, 7]):
        addr, gen, b = eng.populate(seat, e, payload(e), staging=seat % 2)
        assert addr % 256 == 0
        # a wrong device address or a zero generation is refused; the right one binds, and binds again
        assert g.selected_resource_bind_resident(seat, e, payload(e), addr + 256, gen) == -1
        assert g.selected_resource_bind_resident(seat, e, payload(e), addr, 0) == -1
        assert g.selected_resource_bind_resident(seat, e, payload(e), addr, gen) == 0
        assert g.selected_resource_bind_resident(seat, e, payload(e), addr, gen) == 0
        assert g.selected_resource_bind_resident(seat, e, payload(e), addr, gen + 1) == -1
        eng.release(b)
        seats[seat] = (e, gen)

    def run_and_check(groups):
        experts, total = [], 0
        for seat, grp in groups:
            experts.append(_expert(bm, layer, seats[seat][0], grp, seat))
            total += grp
        x = synth.make_tokens(9, total, H)
        y = np.zeros((total, H), np.float32)
        assert g.q4_moe_chain(experts, H, M, x, y, selected=True) == 0
        row = 0
        for seat, grp in groups:
            for _ in range(grp):
                assert_bits_equal(y[row], _chain_want(orc, layer, seats[seat][0], x[row], H, M), "resident chain")
                row += 1

    run_and_check([(0, 1), (1, 3), (2, 2)])

    # replace the occupant of seat 1: fence, unbind, retire, populate another expert, bind, compute
    assert g.selected_resources_fence() == 0
    assert g.selected_resource_unbind(1, seats[1][0]) == 0
    assert eng.retire(1, *seats[1]) == 0
    addr, gen, b = eng.populate(1, 3, payload(3), staging=1)
    assert g.selected_resource_bind_resident(1, 3, payload(3), addr, gen) == 0
    eng.release(b)
    seats[1] = (3, gen)
    run_and_check([(1, 4), (0, 1)])

    st = eng.stats()
    assert (st.population_submissions, st.population_completions, st.retirements) == (4, 4, 1)
    assert st.population_bytes_completed == 4 * stride and st.backend_failures == 0 and st.ready_slots == 3

    assert g.selected_resources_fence() == 0
    for seat, (e, gen) in seats.items():
        assert g.selected_resource_unbind(seat, e) == 0
        assert eng.retire(seat, e, gen) == 0
    assert eng.destroy() == 0


def test_pool_file_streams_through_staging_into_seats(orc, synth, tmp_path):
    """disk mapping -> pinned staging -> HBM seat, two layers of experts in one pool file; tensor pointers
    handed to the chain are addresses inside the mapping (8 modulo 16), the seat copy is what is read."""
    import importlib
    pf = importlib.import_module("salt-core_b200.pool_file")
    g, bm = gpu(), backend_mod()
    H, M, E = 256, 128, 8
    layers = [synth.make_q4_moe_layer(71 + i, hidden=H, inter=M, n_experts=E, topk=2) for i in range(2)]
    path = str(tmp_path / "experts.pool")
    slot = pf.write_pool(path, layers)
    pool = pf.ExpertPool(path, H, M)
    assert (pool.slot_bytes, pool.layers, pool.experts) == (slot, 2, E)
    assert pool.payload(1, 2).ctypes.data % 16 == 8
    seat_bytes = (slot + 255) // 256 * 256
    eng = Engine(bm.ResidencyPlan(3 * seat_bytes, 0, 0, seat_bytes, seat_bytes, 3, 2, 256, 0))
    assert g.selected_resources_prepare(3, E) == 0      # the table of the test above (same capacity)
    picks = [(1, 6), (0, 2), (1, 1)]
    experts, gens = [], []
    for seat, (li, e) in enumerate(picks):
        pay = pool.payload(li, e)
        addr, gen, b = eng.populate(seat, e, pay, staging=seat % 2)
        assert g.selected_resource_bind_resident(seat, e, pay, addr, gen) == 0
        eng.release(b)
        gens.append(gen)
        t = [pool.tensor(li, e, w) for w in range(3)]
        a = lambda v: v.ctypes.data
        experts.append(bm.MoeExpert(a(t[0][0]), a(t[0][1]), a(t[0][2]), a(t[0][0]), a(t[1][0]), a(t[1][1]),
                                    a(t[1][2]), a(t[1][0]), a(t[2][0]), a(t[2][1]), a(t[2][2]), a(t[2][0]),
                                    2, seat, e))
    x = synth.make_tokens(13, 6, H)
    y = np.zeros((6, H), np.float32)
    assert g.q4_moe_chain(experts, H, M, x, y, selected=True) == 0
    for i, (li, e) in enumerate(picks):
        for r in (2 * i, 2 * i + 1):
            assert_bits_equal(y[r], _chain_want(orc, layers[li], e, x[r], H, M), "pool file chain")
    assert g.selected_resources_fence() == 0
    for seat, (li, e) in enumerate(picks):
        assert g.selected_resource_unbind(seat, e) == 0
        assert eng.retire(seat, e, gens[seat]) == 0
    assert eng.destroy() == 0
    pool.close()


def test_backend_operations_check_their_arguments():
    g, bm = gpu(), backend_mod()
    ops = g.residency_backend_ops().contents
    assert ops.abi_version == 1 and ops.ops_size == C.sizeof(bm.ResidencyBackendOps)
    bad = bm.ResidencyPlan(4096, 0, 100, 1024, 1024, 2, 1, 256, 0)          # seat base not aligned
    assert ops.create(None, C.byref(bad)) == -1
    bad = bm.ResidencyPlan(4096, 0, 0, 1024, 512, 2, 1, 256, 0)             # staging smaller than a seat
    assert ops.create(None, C.byref(bad)) == -1
    bad = bm.ResidencyPlan(1024, 0, 0, 1024, 1024, 2, 1, 256, 0)            # seats beyond the budget
    assert ops.create(None, C.byref(bad)) == -1
    plan = bm.ResidencyPlan(4096, 0, 0, 1024, 1024, 4, 2, 256, 0)
    assert ops.create(None, C.byref(plan)) == 0
    assert ops.create(None, C.byref(plan)) == -1                            # one residency per backend
    addr, cap = C.c_void_p(0), C.c_size_t(0)
    assert ops.staging(None, 2, C.byref(addr), C.byref(cap)) == -1
    assert ops.staging(None, 1, C.byref(addr), C.byref(cap)) == 0 and cap.value == 1024 and addr.value
    C.memset(addr, 0x5A, 1024)
    assert ops.populate(None, 1, 0, 1, 1024, 7) == -1                       # offset is not seat 1's
    assert ops.populate(None, 1, 1024, 1, 2048, 7) == -1                    # larger than a seat
    assert ops.populate(None, 1, 1024, 1, 1024, 0) == -1                    # ticket 0 is "none"
    assert ops.populate(None, 1, 1024, 1, 1024, 7) == 0
    assert ops.populate(None, 1, 1024, 0, 1024, 8) == -1                    # seat busy
    assert ops.populate(None, 2, 2048, 1, 1024, 8) == -1                    # staging buffer busy
    done = C.c_int(0)
    assert ops.poll(None, 1, 9, C.byref(done)) == -1                        # stale ticket
    for _ in range(10_000_000):
        assert ops.poll(None, 1, 7, C.byref(done)) == 0
        if done.value:
            break
    assert done.value == 1
    assert ops.poll(None, 1, 7, C.byref(done)) == -1                        # the ticket is spent
    dev = C.c_size_t(0)
    assert ops.resolve(None, 4096, 1, C.byref(dev)) == -1
    assert ops.resolve(None, 1024, 1024, C.byref(dev)) == 0
    back = np.zeros(1024, np.uint8)
    assert g.lib.salt_b200_read_device(C.c_void_p(back.ctypes.data), C.c_void_p(dev.value), C.c_size_t(1024)) == 0
    assert (back == 0x5A).all()
    # retire with a copy in flight waits for it and frees both tickets
    assert ops.populate(None, 3, 3072, 0, 512, 11) == 0
    assert ops.retire(None, 3, 1) == 0
    assert ops.populate(None, 3, 3072, 0, 512, 12) == 0
    assert ops.retire(None, 3, 2) == 0
    assert ops.retire(None, 4, 1) == -1
    assert ops.destroy(None) == 0
    assert ops.destroy(None) == -1
