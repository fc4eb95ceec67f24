"""Expert parallelism by token dispatch.  On one GPU: the three per-layer entry points (route on the home
rank, experts on the owner of each row's expert, combine on the home rank) with the all-to-alls replaced by
index arithmetic over several stacks of one process, against the unsharded stack bit for bit.  On two or
more GPUs: ep.forward_dispatch over NCCL all-to-alls, one process per GPU (tests/ep_dispatch_worker.py)."""
import importlib
import os
import subprocess
import sys

import numpy as np
import pytest

from conftest import ROOT, assert_bits_equal
from gpu_util import stack_mod

pytestmark = pytest.mark.gpu


def _emulated_forward(ep, homes, owners, x_all, per_rank, tensor_core=False):
    """forward_dispatch for all ranks at once in one process: what every all_to_all_single would move is
    concatenated in source-rank order per destination, as the collective delivers it."""
    import torch
    world, L = len(homes), homes[0].n_layers
    K, H, E = homes[0].topk, homes[0].hidden, homes[0].n_experts
    ops = [ep.StackOps(h, tensor_core) for h in homes]
    own = [ep.StackOps(o, tensor_core) for o in owners]
    cur = [torch.from_numpy(np.ascontiguousarray(x_all[r * per_rank:(r + 1) * per_rank])).cuda() for r in range(world)]
    for layer in range(L):
        plans = []
        for r in range(world):
            sel, w = ops[r].route(layer, cur[r], layer > 0)
            order, counts, ids, pos = ep.dispatch_plan(sel, E, world)
            plans.append((sel, w, order, counts.tolist(), ids, cur[r].index_select(0, order // K), pos))
        back = [[None] * world for _ in range(world)]
        for d in range(world):
            rows, ids = [], []
            for r in range(world):
                c = plans[r][3]
                a, b = sum(c[:d]), sum(c[:d + 1])
                rows.append(plans[r][5][a:b])
                ids.append(plans[r][4][a:b])
            done = own[d].experts(layer, torch.cat(rows).contiguous(), torch.cat(ids).contiguous())
            off = 0
            for r in range(world):
                n = plans[r][3][d]
                back[r][d] = done[off:off + n]
                off += n
        nxt = []
        for r in range(world):
            w, pos = plans[r][1], plans[r][6]
            out = torch.empty_like(cur[r])
            ops[r].combine(layer, torch.cat(back[r]).contiguous(), pos, w, out, True, layer + 1 < L)
            nxt.append(out)
        cur = nxt
    torch.cuda.synchronize()
    return np.concatenate([c.cpu().numpy() for c in cur])


@pytest.mark.parametrize("world,per_rank", [(2, 5), (4, 3), (8, 1)])
def test_token_dispatch_matches_unsharded_stack(synth, world, per_rank):
    ep = importlib.import_module("salt-core_b200.ep")
    sm = stack_mod()
    H, M, E, K, L = 256, 128, 32, 4, 3
    layers = [synth.make_q4_moe_layer(900 + i, hidden=H, inter=M, n_experts=E, topk=K) for i in range(L)]
    B = world * per_rank
    x = synth.make_tokens(905, B, H)
    full = sm.MoeStack(B, H, M, E, K)
    homes = [sm.MoeStack(per_rank, H, M, E, K, expert_begin=0, expert_end=1) for _ in range(world)]   # router only
    owners = []
    for r in range(world):
        lo, hi = ep.expert_range(r, world, E)
        owners.append(sm.MoeStack(B, H, M, E, K, expert_begin=lo, expert_end=hi))
    for layer in layers:
        for st in [full] + homes + owners:
            st.add_layer(layer)
    # the unsharded statement: RMSNorm after every layer, as the emulation applies it
    import torch
    d_x = torch.from_numpy(x).cuda()
    act = [torch.empty_like(d_x), torch.empty_like(d_x)]
    cur = d_x.data_ptr()
    for l in range(L):
        out = act[l & 1]
        assert full.layer_experts(l, cur, B, router_input_ready=l > 0) == 0
        assert full.layer_combine(l, B, out.data_ptr(), apply_norm=True, prepare_next=l + 1 < L) == 0
        cur = out.data_ptr()
    torch.cuda.synchronize()
    want = act[(L - 1) & 1].cpu().numpy()
    got = _emulated_forward(ep, homes, owners, x, per_rank)
    assert_bits_equal(got, want, f"token dispatch over {world} ranks")
    for st in [full] + homes + owners:
        assert st.status() == 0
        st.close()


@pytest.mark.parametrize("n,E,world", [(9, 8, 2), (4096 * 8, 128, 8), (1000, 128, 3), (1, 128, 4), (2048 * 8, 128, 2)])
def test_dispatch_plan_kernel_equals_tensor_statement(n, E, world):
    import torch
    ep = importlib.import_module("salt-core_b200.ep")
    rng = np.random.default_rng(n + world)
    sel = torch.from_numpy(rng.integers(0, E, size=n).astype(np.int32))
    order_c, counts_c, ids_c, pos_c = ep.dispatch_plan(sel, E, world)               # tensor operations on the CPU
    order_g, counts_g, ids_g, pos_g = ep.dispatch_plan(sel.cuda(), E, world)        # the library's kernel
    torch.cuda.synchronize()
    assert counts_g.cpu().tolist() == counts_c.tolist() and int(counts_c.sum()) == n
    assert order_g.cpu().tolist() == order_c.tolist()
    assert ids_g.cpu().tolist() == ids_c.tolist()
    assert pos_g.cpu().tolist() == pos_c.tolist()


def test_token_dispatch_with_nvfp4_layers(synth):
    """The same three entry points over NVFP4 layers (exact kernels): 2 ranks, against the unsharded stack."""
    import torch
    ep = importlib.import_module("salt-core_b200.ep")
    sm = stack_mod()
    H, M, E, K, L, world, per_rank = 512, 256, 8, 2, 2, 2, 4
    layers = [synth.make_nvfp4_moe_layer(920 + i, hidden=H, inter=M, n_experts=E, topk=K) for i in range(L)]
    B = world * per_rank
    x = synth.make_tokens(925, B, H)
    full = sm.MoeStack(B, H, M, E, K)
    homes = [sm.MoeStack(per_rank, H, M, E, K, expert_begin=0, expert_end=1) for _ in range(world)]
    owners = [sm.MoeStack(B, H, M, E, K, expert_begin=r * E // world, expert_end=(r + 1) * E // world)
              for r in range(world)]
    for layer in layers:
        for st in [full] + homes + owners:
            st.add_nvfp4_layer(layer)
    d_x = torch.from_numpy(x).cuda()
    act = [torch.empty_like(d_x), torch.empty_like(d_x)]
    cur = d_x.data_ptr()
    for l in range(L):
        out = act[l & 1]
        assert full.layer_experts(l, cur, B, router_input_ready=l > 0) == 0
        assert full.layer_combine(l, B, out.data_ptr(), apply_norm=True, prepare_next=l + 1 < L) == 0
        cur = out.data_ptr()
    torch.cuda.synchronize()
    want = act[(L - 1) & 1].cpu().numpy()
    got = _emulated_forward(ep, homes, owners, x, per_rank)
    assert_bits_equal(got, want, "token dispatch, nvfp4 layers")
    for st in [full] + homes + owners:
        assert st.status() == 0
        st.close()


def test_routed_rows_reject_foreign_experts_and_check_arguments(synth):
    import torch
    sm = stack_mod()
    H, M, E, K = 256, 128, 8, 2
    layer = synth.make_q4_moe_layer(910, hidden=H, inter=M, n_experts=E, topk=K)
    st = sm.MoeStack(4, H, M, E, K, expert_begin=0, expert_end=4)
    st.add_layer(layer)
    rows = torch.from_numpy(synth.make_tokens(911, 3, H)).cuda()
    out = torch.zeros_like(rows)
    ids = torch.tensor([1, 3, 2], dtype=torch.int32, device="cuda")
    assert st.layer_experts_routed(0, rows.data_ptr(), ids.data_ptr(), 3, out.data_ptr()) == 0
    assert st.status() == 0
    assert st.layer_experts_routed(0, rows.data_ptr(), ids.data_ptr(), 4 * K + 1, out.data_ptr()) == -1   # over capacity
    assert st.layer_experts_routed(0, rows.data_ptr(), ids.data_ptr(), 0, out.data_ptr()) == 0            # nothing to do
    assert st.layer_experts_routed(3, rows.data_ptr(), ids.data_ptr(), 3, out.data_ptr()) == -1           # no such layer
    bad = torch.tensor([1, 99, 2], dtype=torch.int32, device="cuda")
    assert st.layer_experts_routed(0, rows.data_ptr(), bad.data_ptr(), 3, out.data_ptr()) == 0
    assert st.status() & 2                                                                                # SB_ERR_INDEX
    st.close()


@pytest.mark.parametrize("world", [2, 4])
def test_token_dispatch_over_nccl(world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29710 + world),
           os.path.join(ROOT, "tests", "ep_dispatch_worker.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.count("EP_DISPATCH_OK") == world, r.stdout[-2000:] + r.stderr[-2000:]
