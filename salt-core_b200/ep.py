"""Expert-parallel plumbing for the MoE stack (one process per GPU, torch.distributed).

Sharding rule: rank r of W owns the contiguous expert range
[r*E//W, (r+1)*E//W) of every layer.  Two data planes:

* replicated activations (``forward``, and the stack's own peer-memory exchange): every rank routes
  all tokens, fills only the rows of the grouped expert-output buffer that belong to its
  experts (global grouped order), and one exchange per layer completes the buffer
  on every rank.  Each row is written by exactly one rank and is +0 elsewhere, so a
  sum over ranks reproduces it exactly, in any order.
* token dispatch (``forward_dispatch``): tokens are partitioned by home rank; a layer routes its
  own tokens, sends each selection's activation row to the owner of its expert (all-to-all),
  the owner applies the expert, the result returns to the home rank (all-to-all), which reduces
  its tokens' rows in rank order.

Both give results that are independent of the number of ranks: a selection's output depends only
on (expert weights, token row) and the reduce order is fixed at the token.
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


def dispatch_plan(selected, n_experts: int, world: int):
    """For a home rank's selections ``selected`` ([B][K] int32 expert ids, torch): the order in which its B*K
    selections are sent (grouped by destination rank, canonical order inside a group), the number sent to
    every rank (int64), the expert id of every sent row and the position of every selection in that order
    (both int32).  On the GPU this is one launch of the library's counting sort; elsewhere the same thing in
    tensor operations."""
    import torch
    flat = selected.reshape(-1)
    n = flat.numel()
    if flat.is_cuda and world <= 8:
        import ctypes as C
        from ._lib import load_library
        flat = flat.to(torch.int32).contiguous()
        order = torch.empty(n, dtype=torch.int32, device=flat.device)
        pos, ids = torch.empty_like(order), torch.empty_like(order)
        counts = torch.empty(world, dtype=torch.int32, device=flat.device)
        rc = load_library().salt_b200_dispatch_plan(
            C.c_void_p(flat.data_ptr()), n, n_experts, world, C.c_void_p(order.data_ptr()), C.c_void_p(pos.data_ptr()),
            C.c_void_p(ids.data_ptr()), C.c_void_p(counts.data_ptr()), C.c_void_p(torch.cuda.current_stream().cuda_stream))
        if rc != 0:
            raise RuntimeError("salt_b200_dispatch_plan failed")
        return order.to(torch.int64), counts.to(torch.int64), ids, pos
    flat = flat.to(torch.int64)
    dest = torch.zeros_like(flat)
    for r in range(1, world):                                   # owner of each selection's expert
        dest += (flat >= r * n_experts // world).to(torch.int64)
    order = torch.argsort(dest, stable=True)
    counts = torch.bincount(dest, minlength=world)
    pos = torch.empty_like(order)
    pos[order] = torch.arange(n, device=flat.device)
    return order, counts, flat[order].to(torch.int32), pos.to(torch.int32)


class StackOps:
    """The three per-layer steps of token dispatch on a MoeStack (device tensors, current CUDA stream)."""

    def __init__(self, stack, tensor_core=False):
        self.stack, self.tc = stack, tensor_core
        self.n_experts, self.topk, self.n_layers = stack.n_experts, stack.topk, stack.n_layers

    def _sp(self):
        import torch
        return torch.cuda.current_stream().cuda_stream

    def route(self, layer, x, router_input_ready):
        import torch
        B = x.shape[0]
        sel = torch.empty((B, self.topk), dtype=torch.int32, device=x.device)
        w = torch.empty((B, self.topk), dtype=torch.float32, device=x.device)
        if self.stack.layer_route(layer, x.data_ptr(), B, sel.data_ptr(), w.data_ptr(), router_input_ready,
                                  stream=self._sp()) != 0:
            raise RuntimeError("salt_b200_layer_route failed")
        return sel, w

    def experts(self, layer, rows, ids):
        import torch
        out = torch.empty_like(rows)
        if rows.shape[0] and self.stack.layer_experts_routed(layer, rows.data_ptr(), ids.data_ptr(), rows.shape[0],
                                                             out.data_ptr(), tensor_core=self.tc,
                                                             stream=self._sp()) != 0:
            raise RuntimeError("salt_b200_layer_experts_routed failed")
        return out

    def combine(self, layer, rows, pos, w, out, apply_norm, prepare_next):
        """rows in the order they were sent; pos[t*K+k] = row of selection (t, k)."""
        if self.stack.layer_combine_rows(layer, rows.data_ptr(), w.data_ptr(), w.shape[0], out.data_ptr(),
                                         apply_norm, prepare_next, stream=self._sp(), d_row_index=pos.data_ptr()) != 0:
            raise RuntimeError("salt_b200_layer_combine_rows failed")
        return out


def forward_dispatch(ops, x, out, act, first=0, count=None, group=None, norm_last=True, stats=None):
    """Layers [first, first+count) for THIS rank's tokens ``x`` ([B_local][hidden]) with token dispatch and
    combine over ``torch.distributed`` all-to-alls (NCCL on GPUs).  ``ops`` supplies route / experts / combine
    (``StackOps`` on a GPU).  The stack of an owner must hold world * B_local * topk rows (every selection of
    every rank may land on one owner).  ``stats``: a dict that receives the rows sent and received."""
    import torch
    import torch.distributed as dist
    world = dist.get_world_size(group)
    count = ops.n_layers - first if count is None else count
    K, H = ops.topk, x.shape[1]
    cur = x
    for i in range(count):
        layer, last = first + i, i == count - 1
        sel, w = ops.route(layer, cur, i > 0)
        order, send_counts, ids, pos = dispatch_plan(sel, ops.n_experts, world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=group)
        sc, rc = send_counts.tolist(), recv_counts.tolist()          # the one host synchronisation of the layer
        rows = cur.index_select(0, order // K)
        n_recv = int(sum(rc))
        recv_rows = torch.empty((n_recv, H), dtype=cur.dtype, device=cur.device)
        recv_ids = torch.empty((n_recv,), dtype=torch.int32, device=cur.device)
        dist.all_to_all_single(recv_rows, rows, rc, sc, group=group)
        dist.all_to_all_single(recv_ids, ids, rc, sc, group=group)
        done = ops.experts(layer, recv_rows, recv_ids)
        back = torch.empty_like(rows)
        dist.all_to_all_single(back, done, sc, rc, group=group)
        dst = out if last else act[i & 1]
        ops.combine(layer, back, pos, w, dst, norm_last or not last, not last)   # pos: canonical (token, rank) -> row
        if stats is not None:
            stats["rows_sent"] = stats.get("rows_sent", 0) + int(rows.shape[0])
            stats["rows_received"] = stats.get("rows_received", 0) + n_recv
        cur = dst
    return out
