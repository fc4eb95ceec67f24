"""Expert-parallel plumbing for the MoE stack (one process per GPU, torch.distributed).

Sharding rule: rank r of W owns the contiguous expert range
[r*E//W, (r+1)*E//W) of every layer.  Activations are replicated; each rank
fills only the rows of the grouped expert-output buffer that belong to its
experts (global grouped order), and one exchange per layer completes the buffer
on every rank.  Each row is written by exactly one rank and is +0 elsewhere, so a
sum over ranks reproduces it exactly, in any order: the result is independent
of the number of ranks.
"""
from __future__ import annotations


def expert_range(rank: int, world: int, n_experts: int) -> tuple[int, int]:
    if not 0 <= rank < world or world < 1 or n_experts < world:
        raise ValueError("invalid expert-parallel layout")
    return rank * n_experts // world, (rank + 1) * n_experts // world


def owner_of(expert: int, world: int, n_experts: int) -> int:
    for r in range(world):
        lo, hi = expert_range(r, world, n_experts)
        if lo <= expert < hi:
            return r
    raise ValueError("expert out of range")


def exchange_grouped(grouped, group=None):
    """Complete the zero-padded grouped buffer on every rank (in place)."""
    import torch.distributed as dist
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(grouped, op=dist.ReduceOp.SUM, group=group)
    return grouped


def connect_peer_memory(stack, group=None) -> bool:
    """Map every rank's landing region into this process (CUDA IPC) so that the stack exchanges
    the grouped outputs itself, inside salt_b200_stack_forward_device, instead of through
    exchange_grouped.  Returns False on every rank when any rank could not map its peers; the
    caller then stays on forward().  Ends with a barrier: no rank starts an exchange before all
    are connected."""
    import torch
    import torch.distributed as dist
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    # the handles travel through whatever the process group moves: device tensors for NCCL, host tensors otherwise
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    handle, _ = stack.ep_region()
    mine = torch.tensor(list(handle), dtype=torch.uint8, device=dev)
    gathered = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(gathered, mine, group=group)
    handles = [bytes(t.cpu().tolist()) for t in gathered]
    ok = torch.tensor([1 if stack.ep_connect(rank, world, ipc_handles=handles) == 0 else 0], dtype=torch.int32,
                      device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
    good = bool(ok.item())
    if not good:
        stack.ep_disconnect()
    dist.barrier(group)
    return good


def forward(stack, grouped, d_x, B, d_out, act, stream=0, first=0, count=None, group=None):
    """One pass of layers [first, first+count) with one exchange per layer.
    d_x / d_out / act[0..1] are torch tensors [B][hidden] on the device;
    `grouped` is the stack's grouped-output buffer (set_grouped_out)."""
    count = stack.n_layers - first if count is None else count
    cur = d_x.data_ptr()
    for i in range(count):
        layer = first + i
        last = i == count - 1
        out = d_out if last else act[i & 1]
        if stack.layer_experts(layer, cur, B, zero_remote=True, router_input_ready=i > 0, stream=stream) != 0:
            raise RuntimeError("salt_b200_layer_experts failed")
        exchange_grouped(grouped, group)
        if stack.layer_combine(layer, B, out.data_ptr(), apply_norm=not last, prepare_next=not last,
                               stream=stream) != 0:
            raise RuntimeError("salt_b200_layer_combine failed")
        cur = out.data_ptr()
    return d_out
