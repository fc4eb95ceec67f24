"""Expert-parallel host logic on CPU: two gloo ranks each fill only their experts'
rows of the grouped buffer (computed here with the CPU oracle standing in for the
device kernels), exchange once, and every rank must end with exactly the
single-process result."""
import importlib
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _worker(rank, world, port, out_path):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    synth = importlib.import_module("salt-core_b200.synth")
    ep = importlib.import_module("salt-core_b200.ep")
    orc = oracle.Oracle()
    H, M, E, K, B = 128, 64, 8, 3, 5
    layer = synth.make_q4_moe_layer(11, hidden=H, inter=M, n_experts=E, topk=K)
    x = synth.make_tokens(12, B, H)
    want, sel, w = orc.moe_layer_q4(layer, x, threads=1)
    rc, offs, g2c, c2g, _ = orc.route_group(sel.ravel(), B, K, E)
    lo, hi = ep.expert_range(rank, world, E)
    grouped = np.zeros((B * K, H), np.float32)
    for g in range(B * K):
        canonical = int(g2c[g])
        e = int(sel.ravel()[canonical])
        if lo <= e < hi:                       # this rank owns the expert: compute its row
            t = canonical // K
            gate = orc.q4_matvec(*layer.tensor(e, 0), M, H, x[t])
            up = orc.q4_matvec(*layer.tensor(e, 1), M, H, x[t])
            chain = orc.map_f32("gelu_tanh", gate) * up
            grouped[g] = orc.q4_matvec(*layer.tensor(e, 2), H, M, chain)
    buf = torch.from_numpy(grouped)
    ep.exchange_grouped(buf)
    rc, got = orc.weighted_reduce(w.ravel(), c2g, buf.numpy(), B, K)
    ok = rc == 0 and (got.view(np.uint32) == want.view(np.uint32)).all()
    covered = sum(1 for e in range(E) if ep.owner_of(e, world, E) == rank)
    flags = torch.tensor([int(ok), covered])
    gathered = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(gathered, flags)
    if rank == 0:
        np.save(out_path, torch.stack(gathered).numpy())
    dist.destroy_process_group()


def test_two_rank_exchange_reproduces_single_process_result(tmp_path):
    out = str(tmp_path / "flags.npy")
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    flags = np.load(out)
    assert flags[:, 0].tolist() == [1, 1]          # both ranks bit-identical to the single-process oracle
    assert flags[:, 1].sum() == 8                  # every expert has exactly one owner


def test_expert_ranges_partition_the_experts():
    ep = importlib.import_module("salt-core_b200.ep")
    for world in (1, 2, 4, 8):
        covered = []
        for r in range(world):
            lo, hi = ep.expert_range(r, world, 128)
            covered += list(range(lo, hi))
        assert covered == list(range(128))


class _FakeStack:
    """Stands in for MoeStack in the handle exchange: records what connect_peer_memory does."""

    def __init__(self, rank, fail):
        self.rank, self.fail, self.connected, self.disconnected, self.seen = rank, fail, False, False, None

    def ep_region(self):
        return bytes([self.rank + 1]) * 64, 0x1000 * (self.rank + 1)

    def ep_connect(self, rank, world, ipc_handles=None, regions=None):
        self.seen = (rank, world, [h[0] for h in ipc_handles], [len(h) for h in ipc_handles])
        if self.fail:
            return -1
        self.connected = True
        return 0

    def ep_disconnect(self):
        self.disconnected = True
        self.connected = False
        return 0


def _connect_worker(rank, world, port, out_path, failing_rank):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ep = importlib.import_module("salt-core_b200.ep")
    st = _FakeStack(rank, fail=rank == failing_rank)
    good = ep.connect_peer_memory(st)
    ordered = st.seen == (rank, world, [r + 1 for r in range(world)], [64] * world)
    flags = torch.tensor([int(good), int(st.connected), int(st.disconnected), int(ordered)])
    gathered = [torch.zeros(4, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(gathered, flags)
    if rank == 0:
        np.save(out_path, torch.stack(gathered).numpy())
    dist.destroy_process_group()


def test_peer_memory_handles_are_gathered_in_rank_order(tmp_path):
    out = str(tmp_path / "connect.npy")
    mp.spawn(_connect_worker, args=(2, 31500 + os.getpid() % 2000, out, -1), nprocs=2, join=True)
    flags = np.load(out)
    assert flags.tolist() == [[1, 1, 0, 1], [1, 1, 0, 1]]      # connected everywhere, handles in rank order


def test_peer_memory_connect_failure_on_one_rank_disconnects_all(tmp_path):
    out = str(tmp_path / "connect_fail.npy")
    mp.spawn(_connect_worker, args=(2, 33500 + os.getpid() % 2000, out, 1), nprocs=2, join=True)
    flags = np.load(out)
    assert flags[:, 0].tolist() == [0, 0]                      # every rank reports failure ...
    assert flags[:, 1].tolist() == [0, 0] and flags[:, 2].tolist() == [1, 1]   # ... and none stays connected
