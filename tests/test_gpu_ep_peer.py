"""Expert-parallel exchange over peer memory (salt_b200_stack_ep_*): the result must equal the
unsharded stack bit for bit, for any number of ranks.

On one GPU the ranks are stacks of one process and the two halves of the exchange are enqueued
separately (every rank's push before any rank's pull), so that no launch waits for a later one.
With two or more GPUs the ranks are child processes, one per GPU, and the kernel pushes, waits
and pulls in one launch."""
import os
import subprocess
import sys

import numpy as np
import pytest

from gpu_util import stack_mod

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def synth():
    import importlib
    return importlib.import_module("salt-core_b200").synth


@pytest.mark.parametrize("world,B", [(2, 3), (4, 5), (8, 8)])
def test_ranks_on_one_device_equal_unsharded_stack(synth, world, B):
    import torch
    H, M, E, K, L = 256, 128, 32, 4, 3
    layers = [synth.make_q4_moe_layer(700 + i, hidden=H, inter=M, n_experts=E, topk=K) for i in range(L)]
    sm = stack_mod()
    full = sm.MoeStack(8, H, M, E, K)
    for layer in layers:
        full.add_layer(layer)
    ranks = []
    for r in range(world):
        st = sm.MoeStack(8, H, M, E, K, expert_begin=r * E // world, expert_end=(r + 1) * E // world)
        for layer in layers:
            st.add_layer(layer)
        ranks.append(st)
    regions = [st.ep_region()[1] for st in ranks]
    for r, st in enumerate(ranks):
        assert st.ep_connect(r, world, regions=regions) == 0
    # three exchanges per pass: the landing buffers change parity from pass to pass
    for rep in range(3):
        x = synth.make_tokens(710 + rep, B, H)
        want = full.forward_host(x)
        cur = [torch.from_numpy(x).cuda() for _ in range(world)]
        for l in range(L):
            out = [torch.empty(B, H, dtype=torch.float32, device="cuda") for _ in range(world)]
            for r, st in enumerate(ranks):
                assert st.layer_experts(l, cur[r].data_ptr(), B) == 0
            for st in ranks:
                assert st.ep_exchange(B, phase=st.EP_PUSH) == 0
            for st in ranks:
                assert st.ep_exchange(B, phase=st.EP_PULL) == 0
            for r, st in enumerate(ranks):
                assert st.layer_combine(l, B, out[r].data_ptr(), apply_norm=l + 1 < L) == 0
            cur = out
        for r, st in enumerate(ranks):
            assert st.status() == 0
            got = cur[r].cpu().numpy()
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), f"rank {r} of {world}, pass {rep}"
    for st in ranks + [full]:
        st.close()


def test_exchange_refuses_unconnected_stack_and_bad_world(synth):
    sm = stack_mod()
    st = sm.MoeStack(4, 256, 128, 32, 4, expert_begin=0, expert_end=16)
    st.add_layer(synth.make_q4_moe_layer(720, hidden=256, inter=128, n_experts=32, topk=4))
    assert st.ep_exchange(1) == -1                       # not connected
    _, region = st.ep_region()
    assert st.ep_connect(0, 1, regions=[region]) == -1   # a world of one has nothing to exchange
    assert st.ep_connect(0, 9, regions=[region] * 9) == -1
    assert st.ep_connect(2, 2, regions=[region] * 2) == -1
    st.close()


@pytest.mark.parametrize("world", [2, 4])
def test_ranks_on_separate_gpus(world):
    import torch
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(29610 + world),
           os.path.join(ROOT, "tests", "ep_peer_worker.py")]
    r = subprocess.run(cmd, cwd=ROOT, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert r.stdout.count("EP_PEER_OK") == world, r.stdout[-2000:] + r.stderr[-2000:]


def test_exchange_wait_runs_out_then_reset_recovers(synth):
    """A rank pulls rows that nobody pushed: with a short poll limit the kernel gives up, reports the
    timeout in the error word and returns (nothing hangs, the device stays usable).  After every rank
    resets its landing region a normal push + pull is bit-exact again."""
    import torch
    H, M, E, K, B, world = 256, 128, 32, 4, 5, 2
    layer = synth.make_q4_moe_layer(730, hidden=H, inter=M, n_experts=E, topk=K)
    sm = stack_mod()
    full = sm.MoeStack(8, H, M, E, K)
    full.add_layer(layer)
    ranks = []
    for r in range(world):
        st = sm.MoeStack(8, H, M, E, K, expert_begin=r * E // world, expert_end=(r + 1) * E // world)
        st.add_layer(layer)
        ranks.append(st)
    regions = [st.ep_region()[1] for st in ranks]
    for r, st in enumerate(ranks):
        assert st.ep_connect(r, world, regions=regions) == 0
        assert st.ep_set_poll_limit(2000) == 0          # about a millisecond
    x = synth.make_tokens(731, B, H)
    want = full.forward_host(x)
    d_x = torch.from_numpy(x).cuda()
    for st in ranks:
        assert st.layer_experts(0, d_x.data_ptr(), B) == 0
    # rank 0 waits for rank 1's rows, which were never pushed
    assert ranks[0].ep_exchange(B, phase=ranks[0].EP_PULL) == 0
    assert ranks[0].status() == 8                       # SB_ERR_TIMEOUT, and the call returned
    for st in ranks:
        assert st.ep_reset() == 0
        assert st.ep_set_poll_limit(1 << 23) == 0
    outs = []
    for st in ranks:
        assert st.layer_experts(0, d_x.data_ptr(), B) == 0
    for st in ranks:
        assert st.ep_exchange(B, phase=st.EP_PUSH) == 0
    for st in ranks:
        assert st.ep_exchange(B, phase=st.EP_PULL) == 0
    for st in ranks:
        out = torch.empty(B, H, dtype=torch.float32, device="cuda")
        assert st.layer_combine(0, B, out.data_ptr(), apply_norm=False) == 0
        outs.append(out)
    for r, st in enumerate(ranks):
        assert st.status() == 0
        assert (outs[r].cpu().numpy().view(np.uint32) == want.view(np.uint32)).all(), f"rank {r} after reset"
    for st in ranks + [full]:
        st.close()
