"""One rank of the multi-GPU token-dispatch test (launched by test_gpu_ep_dispatch.py through
torch.distributed.run, one process per GPU): tokens partitioned by home rank, ep.forward_dispatch over NCCL
all-to-alls, checked against the unsharded stack (held by every rank) bit for bit."""
import importlib
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
    pkg = importlib.import_module("salt-core_b200")
    synth, ep = pkg.synth, importlib.import_module("salt-core_b200.ep")
    sm = importlib.import_module("salt-core_b200.stack")
    H, M, E, K, L, per_rank = 256, 128, 32, 4, 4, 6
    B = per_rank * world
    layers = [synth.make_q4_moe_layer(820 + i, hidden=H, inter=M, n_experts=E, topk=K) for i in range(L)]
    full = sm.MoeStack(B, H, M, E, K)
    lo, hi = ep.expert_range(rank, world, E)
    part = sm.MoeStack(B, H, M, E, K, expert_begin=lo, expert_end=hi)      # holds world * per_rank * K rows
    for layer in layers:
        full.add_layer(layer)
        part.add_layer(layer)
    x_all = synth.make_tokens(830, B, H)
    d_all = torch.from_numpy(x_all).cuda()
    act = [torch.empty_like(d_all), torch.empty_like(d_all)]
    cur = d_all.data_ptr()
    for l in range(L):
        out = act[l & 1]
        assert full.layer_experts(l, cur, B, router_input_ready=l > 0) == 0
        assert full.layer_combine(l, B, out.data_ptr(), apply_norm=True, prepare_next=l + 1 < L) == 0
        cur = out.data_ptr()
    torch.cuda.synchronize()
    want = act[(L - 1) & 1].cpu().numpy()[rank * per_rank:(rank + 1) * per_rank]
    x = d_all[rank * per_rank:(rank + 1) * per_rank].contiguous()
    out = torch.empty_like(x)
    mine = [torch.empty_like(x), torch.empty_like(x)]
    stats = {}
    for rep in range(2):
        ep.forward_dispatch(ep.StackOps(part), x, out, mine, stats=stats)
        torch.cuda.synchronize()
        assert part.status() == 0
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32)), f"pass {rep}"
    assert stats["rows_sent"] == 2 * L * per_rank * K
    dist.barrier()
    print("EP_DISPATCH_OK", flush=True)
    part.close()
    full.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
