// Device-local expert residency: the physical half of the reference's residency state machine
// (reference include/salt/gpu_residency.h:63-89; the state machine itself, src/gpu_residency.c, stays
// reference host code and drives these operations).
//
// The plan fixes everything at start-up: ONE arena in HBM of device_budget_bytes (a permanent part
// followed by slot_count seats of slot_bytes from slot_base_offset) and staging_count pinned host buffers
// of staging_bytes.  A population is: the engine reads a slot's payload from its source into a staging
// buffer (host side), `populate` enqueues one asynchronous copy staging -> seat on a dedicated
// non-blocking stream and records the seat's event, `poll` asks the event, `resolve` turns an arena offset
// into the device address that salt_gpu_selected_resource_bind_resident publishes, `retire` waits for a
// copy still in flight before the seat is reused.  Nothing is allocated after `create`.
// The permanent_* operations (bulk population of the permanent part) are not provided: the entries are
// NULL, which the reference's permanent-population call treats as "not available" (src/gpu_residency.c:317-322).
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include <vector>

#include "../../include/salt_gpu_b200.h"
#include "backend_state.h"

namespace sb {

struct ResidencyState {
    bool ready = false;
    SaltGpuResidencyPlan plan = {};
    uint8_t* arena = nullptr;            // HBM
    uint8_t* staging = nullptr;          // pinned host memory, staging_count buffers
    cudaStream_t stream = nullptr;
    std::vector<cudaEvent_t> events;     // one per seat
    std::vector<uint64_t> seat_ticket;   // ticket of the copy in flight into the seat (0: none)
    std::vector<uint64_t> staging_ticket;
    std::vector<uint32_t> seat_staging;  // staging buffer the seat's copy reads (UINT32_MAX: none)
};
static ResidencyState g_res;

static void residency_release() {
    if (g_res.stream) cudaStreamSynchronize(g_res.stream);
    for (cudaEvent_t e : g_res.events) cudaEventDestroy(e);
    if (g_res.stream) cudaStreamDestroy(g_res.stream);
    if (g_res.staging) cudaFreeHost(g_res.staging);
    if (g_res.arena) cudaFree(g_res.arena);
    g_res = ResidencyState();
}

// plan rules of the reference (src/gpu_residency.c, salt_gpu_residency_plan_validate): seats lie inside the
// budget behind the permanent part, a payload fits a staging buffer, alignment is a power of two
static bool plan_ok(const SaltGpuResidencyPlan* p) {
    if (!p || p->flags != 0 || p->device_budget_bytes < 1 || p->slot_count < 1 || p->staging_count < 1 || p->slot_bytes < 1 || p->staging_bytes < p->slot_bytes ||
        p->device_alignment < 1 || (p->device_alignment & (p->device_alignment - 1)) != 0)
        return false;
    if (p->slot_base_offset < p->permanent_bytes || (p->slot_base_offset % p->device_alignment) != 0 ||
        (p->slot_bytes % p->device_alignment) != 0)
        return false;
    const uint64_t seats = (uint64_t)p->slot_count * p->slot_bytes;
    if (seats / p->slot_count != p->slot_bytes || p->slot_base_offset > p->device_budget_bytes ||
        seats > p->device_budget_bytes - p->slot_base_offset)
        return false;
    return p->staging_bytes <= UINT64_MAX / p->staging_count;
}

static int res_create(void*, const SaltGpuResidencyPlan* plan) {
    if (!g_backend.ready || g_res.ready || !plan_ok(plan) || plan->device_alignment > 256) return -1;
    g_res.plan = *plan;
    const size_t staging_total = (size_t)(plan->staging_bytes * plan->staging_count);
    bool ok = cuda_ok(cudaMalloc((void**)&g_res.arena, (size_t)plan->device_budget_bytes), "residency arena") &&
              cuda_ok(cudaHostAlloc((void**)&g_res.staging, staging_total, cudaHostAllocDefault), "residency staging") &&
              cuda_ok(cudaStreamCreateWithFlags(&g_res.stream, cudaStreamNonBlocking), "residency stream");
    for (uint32_t i = 0; ok && i < plan->slot_count; i++) {
        cudaEvent_t e = nullptr;
        ok = cuda_ok(cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "residency event");
        if (ok) g_res.events.push_back(e);
    }
    if (!ok) {
        residency_release();
        return -1;
    }
    g_res.seat_ticket.assign(plan->slot_count, 0);
    g_res.staging_ticket.assign(plan->staging_count, 0);
    g_res.seat_staging.assign(plan->slot_count, UINT32_MAX);
    g_res.ready = true;
    return 0;
}

static int res_staging(void*, uint32_t staging_slot, void** address, size_t* capacity) {
    if (!g_res.ready || !address || !capacity || staging_slot >= g_res.plan.staging_count) return -1;
    *address = g_res.staging + (size_t)staging_slot * (size_t)g_res.plan.staging_bytes;
    *capacity = (size_t)g_res.plan.staging_bytes;
    return 0;
}

static int res_populate(void*, uint32_t seat, uint64_t device_offset, uint32_t staging_slot, size_t nbytes,
                        uint64_t ticket) {
    const SaltGpuResidencyPlan& p = g_res.plan;
    if (!g_res.ready || ticket == 0 || nbytes == 0 || seat >= p.slot_count || staging_slot >= p.staging_count ||
        nbytes > p.slot_bytes || g_res.seat_ticket[seat] != 0 || g_res.staging_ticket[staging_slot] != 0 ||
        device_offset != p.slot_base_offset + (uint64_t)seat * p.slot_bytes)
        return -1;
    if (!cuda_ok(cudaMemcpyAsync(g_res.arena + (size_t)device_offset,
                                 g_res.staging + (size_t)staging_slot * (size_t)p.staging_bytes, nbytes,
                                 cudaMemcpyHostToDevice, g_res.stream), "residency populate"))
        return -1;
    if (!cuda_ok(cudaEventRecord(g_res.events[seat], g_res.stream), "residency event record")) {
        cudaStreamSynchronize(g_res.stream);      // the copy is enqueued: let it finish before the buffers are reused
        return -1;
    }
    g_res.seat_ticket[seat] = ticket;
    g_res.staging_ticket[staging_slot] = ticket;
    g_res.seat_staging[seat] = staging_slot;
    return 0;
}

static int res_poll(void*, uint32_t seat, uint64_t ticket, int* complete) {
    if (!g_res.ready || !complete || ticket == 0 || seat >= g_res.plan.slot_count || g_res.seat_ticket[seat] != ticket)
        return -1;
    const cudaError_t e = cudaEventQuery(g_res.events[seat]);
    if (e == cudaErrorNotReady) {
        *complete = 0;
        return 0;
    }
    if (!cuda_ok(e, "residency poll")) return -1;
    const uint32_t st = g_res.seat_staging[seat];
    if (st >= g_res.plan.staging_count || g_res.staging_ticket[st] != ticket) return -1;
    g_res.seat_ticket[seat] = 0;
    g_res.staging_ticket[st] = 0;
    g_res.seat_staging[seat] = UINT32_MAX;
    *complete = 1;
    return 0;
}

static int res_resolve(void*, uint64_t device_offset, size_t nbytes, uintptr_t* address) {
    if (!g_res.ready || !address || nbytes == 0 || device_offset > g_res.plan.device_budget_bytes ||
        nbytes > g_res.plan.device_budget_bytes - device_offset)
        return -1;
    *address = (uintptr_t)(g_res.arena + (size_t)device_offset);
    return 0;
}

static int res_retire(void*, uint32_t seat, uint64_t) {
    if (!g_res.ready || seat >= g_res.plan.slot_count) return -1;
    const uint64_t ticket = g_res.seat_ticket[seat];
    const uint32_t st = g_res.seat_staging[seat];
    if (ticket != 0) {
        if (!cuda_ok(cudaEventSynchronize(g_res.events[seat]), "residency retire")) return -1;
        if (st >= g_res.plan.staging_count || g_res.staging_ticket[st] != ticket) return -1;
        g_res.staging_ticket[st] = 0;
    } else if (st != UINT32_MAX) {
        return -1;
    }
    g_res.seat_ticket[seat] = 0;
    g_res.seat_staging[seat] = UINT32_MAX;
    return 0;
}

static int res_destroy(void*) {
    if (!g_res.ready) return -1;
    residency_release();
    return 0;
}

// Device address of a seat, for the resident bind: 0 when there is no residency, no such seat, or the
// payload does not fit the seat.
uintptr_t residency_seat_address(int seat, size_t nbytes) {
    const SaltGpuResidencyPlan& p = g_res.plan;
    if (!g_res.ready || seat < 0 || (uint32_t)seat >= p.slot_count || nbytes == 0 || nbytes > p.slot_bytes) return 0;
    return (uintptr_t)(g_res.arena + (size_t)(p.slot_base_offset + (uint64_t)seat * p.slot_bytes));
}

void residency_shutdown() { residency_release(); }

static const SaltGpuResidencyBackendOps g_residency_ops = {
    SALT_GPU_RESIDENCY_ABI_VERSION, sizeof(SaltGpuResidencyBackendOps),
    res_create, res_staging, res_populate, res_poll, res_resolve, res_retire, res_destroy,
    nullptr, nullptr, nullptr, nullptr,
};

}  // namespace sb

extern "C" const SaltGpuResidencyBackendOps* salt_gpu_residency_backend_ops(void) { return &sb::g_residency_ops; }
