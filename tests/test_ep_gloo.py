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


class _OracleOps:
    """route / experts / combine of ep.forward_dispatch computed by the CPU oracle (stands in for StackOps)."""

    def __init__(self, orc, layers, rank, world):
        self.orc, self.layers = orc, layers
        L0 = layers[0]
        self.n_experts, self.topk, self.n_layers = L0.n_experts, L0.topk, len(layers)
        ep = importlib.import_module("salt-core_b200.ep")
        self.lo, self.hi = ep.expert_range(rank, world, L0.n_experts)
        self.rows_done = 0

    def route(self, layer, x, router_input_ready):
        L, xs = self.layers[layer], x.numpy()
        sel = np.empty((xs.shape[0], L.topk), np.int32)
        w = np.empty((xs.shape[0], L.topk), np.float32)
        for t in range(xs.shape[0]):
            rc, rin = self.orc.router_input(xs[t], L.router_scale, L.eps)
            assert rc == 0
            rc, sel[t], w[t] = self.orc.router_topk(self.orc.router_scores(L.router_w, None, rin), L.per_expert_scale,
                                                    L.topk, True)
            assert rc == 0
        return torch.from_numpy(sel), torch.from_numpy(w)

    def experts(self, layer, rows, ids):
        L, orc = self.layers[layer], self.orc
        out = np.empty(tuple(rows.shape), np.float32)
        for i in range(rows.shape[0]):
            e = int(ids[i])
            assert self.lo <= e < self.hi, "a row reached a rank that does not own its expert"
            x = rows[i].numpy()
            gate = orc.q4_matvec(*L.tensor(e, 0), L.inter, L.hidden, x)
            up = orc.q4_matvec(*L.tensor(e, 1), L.inter, L.hidden, x)
            out[i] = orc.q4_matvec(*L.tensor(e, 2), L.hidden, L.inter, orc.map_f32("gelu_tanh", gate) * up)
        self.rows_done += rows.shape[0]
        return torch.from_numpy(out)

    def combine(self, layer, rows, pos, w, out, apply_norm, prepare_next):
        L, B = self.layers[layer], w.shape[0]
        rc, y = self.orc.weighted_reduce(w.numpy().ravel(), pos.numpy().astype(np.int32), rows.numpy(), B, L.topk)
        assert rc == 0
        if apply_norm:
            y = np.stack([self.orc.rmsnorm(y[t], L.norm_weight, L.eps, True)[1] for t in range(B)])
        out.copy_(torch.from_numpy(np.ascontiguousarray(y)))
        return out


def _dispatch_worker(rank, world, port, out_path):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import oracle
    synth = importlib.import_module("salt-core_b200.synth")
    ep = importlib.import_module("salt-core_b200.ep")
    orc = oracle.Oracle()
    H, M, E, K, B = 128, 64, 8, 3, 3                       # B tokens per rank
    layers = [synth.make_q4_moe_layer(31 + i, hidden=H, inter=M, n_experts=E, topk=K) for i in range(2)]
    x_all = synth.make_tokens(33, B * world, H)
    # single-process statement of the two-layer stack (RMSNorm after each layer)
    cur = x_all
    for L in layers:
        y, _, _ = orc.moe_layer_q4(L, cur, threads=1)
        cur = np.stack([orc.rmsnorm(y[t], L.norm_weight, L.eps, True)[1] for t in range(y.shape[0])])
    want = cur[rank * B:(rank + 1) * B]
    ops = _OracleOps(orc, layers, rank, world)
    x = torch.from_numpy(np.ascontiguousarray(x_all[rank * B:(rank + 1) * B]))
    out, act, stats = torch.empty_like(x), [torch.empty_like(x), torch.empty_like(x)], {}
    ep.forward_dispatch(ops, x, out, act, stats=stats)
    ok = (out.numpy().view(np.uint32) == want.view(np.uint32)).all()
    flags = torch.tensor([int(ok), stats["rows_sent"], stats["rows_received"], ops.rows_done])
    gathered = [torch.zeros(4, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(gathered, flags)
    if rank == 0:
        np.save(out_path, torch.stack(gathered).numpy())
    dist.destroy_process_group()


def test_token_dispatch_and_combine_reproduce_single_process_result(tmp_path):
    """Tokens partitioned by home rank; rows go only to the owners of their experts and come back only to
    the home rank; every rank ends with exactly the unsharded result for its tokens."""
    world, out = 2, str(tmp_path / "dispatch.npy")
    port = 31500 + os.getpid() % 2000
    mp.spawn(_dispatch_worker, args=(world, port, out), nprocs=world, join=True)
    flags = np.load(out)
    assert flags[:, 0].tolist() == [1] * world
    assert flags[:, 1].tolist() == [2 * 3 * 3] * world         # each rank sends its B*K selections per layer
    assert flags[:, 2].sum() == flags[:, 1].sum()               # every row sent is received exactly once
    assert (flags[:, 2] == flags[:, 3]).all()


def test_dispatch_plan_orders_rows_by_owner():
    ep = importlib.import_module("salt-core_b200.ep")
    sel = torch.tensor([[0, 5, 7], [1, 2, 6], [3, 4, 5]], dtype=torch.int32)
    order, counts, ids, pos = ep.dispatch_plan(sel, 8, 2)
    assert counts.tolist() == [4, 5]
    assert order.tolist() == [0, 3, 4, 6, 1, 2, 5, 7, 8]         # canonical order inside each destination
    assert ids.tolist() == [0, 1, 2, 3, 5, 7, 6, 4, 5]
    assert pos[order].tolist() == list(range(9))                 # pos is the inverse permutation
    order, counts, ids, pos = ep.dispatch_plan(sel, 8, 4)
    assert counts.tolist() == [2, 2, 3, 2]
