"""One rank of the multi-GPU peer-memory exchange test (launched by test_gpu_ep_peer.py through
torch.distributed.run, one process per GPU).  Every rank also holds the unsharded stack and checks
its own expert-parallel output against it bit for bit: stream launches, then CUDA-graph replays."""
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
    H, M, E, K, L, B = 256, 128, 32, 4, 5, world
    layers = [synth.make_q4_moe_layer(800 + i, hidden=H, inter=M, n_experts=E, topk=K) for i in range(L)]
    full = sm.MoeStack(8, H, M, E, K)
    lo, hi = ep.expert_range(rank, world, E)
    part = sm.MoeStack(8, H, M, E, K, expert_begin=lo, expert_end=hi)
    for layer in layers:
        full.add_layer(layer)
        part.add_layer(layer)
    if not ep.connect_peer_memory(part):
        raise SystemExit("peer memory could not be mapped")
    stream = torch.cuda.Stream()
    sp = stream.cuda_stream
    x = synth.make_tokens(810, B, H)
    want = full.forward_host(x)
    d_x = torch.from_numpy(x).cuda()
    d_y = torch.zeros_like(d_x)
    with torch.cuda.stream(stream):
        dist.barrier()
        for rep in range(3):                      # odd layer count: landing-buffer parity flips per pass
            d_y.zero_()
            assert part.forward_device(d_x.data_ptr(), B, d_y.data_ptr(), stream=sp) == 0
            assert part.status(sp) == 0
            assert np.array_equal(d_y.cpu().numpy().view(np.uint32), want.view(np.uint32)), f"stream pass {rep}"
        dist.barrier()
        assert part.graph_capture(d_x.data_ptr(), B, d_y.data_ptr(), sp) == 0
        dist.barrier()
        for rep in range(5):
            d_y.zero_()
            assert part.graph_launch(sp) == 0
            assert part.status(sp) == 0
            assert np.array_equal(d_y.cpu().numpy().view(np.uint32), want.view(np.uint32)), f"graph pass {rep}"
    dist.barrier()
    torch.cuda.synchronize()
    print("EP_PEER_OK", flush=True)
    part.close()
    full.close()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
