"""ctypes mirror of the device-resident MoE stack (salt_b200_* in
include/salt_gpu_b200.h)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from ._lib import load_library


class Q4LayerSpec(C.Structure):
    _fields_ = [("hidden", C.c_int), ("inter", C.c_int), ("n_experts", C.c_int), ("topk", C.c_int),
                ("eps", C.c_float), ("router_w", C.c_void_p), ("router_scale", C.c_void_p),
                ("per_expert_scale", C.c_void_p), ("pool", C.c_void_p), ("expert_stride", C.c_size_t),
                ("norm_weight", C.c_void_p)]


class Nvfp4LayerSpec(C.Structure):
    _fields_ = [("hidden", C.c_int), ("inter", C.c_int), ("n_experts", C.c_int), ("topk", C.c_int),
                ("eps", C.c_float), ("router_w", C.c_void_p), ("router_scale", C.c_void_p),
                ("per_expert_scale", C.c_void_p), ("pool", C.c_void_p), ("expert_stride", C.c_size_t),
                ("weight_divisors", C.c_void_p), ("input_globals", C.c_void_p), ("norm_weight", C.c_void_p)]


class FfnBlockSpec(C.Structure):
    _fields_ = [("dense_inter", C.c_int), ("dense_gate", C.c_void_p), ("dense_up", C.c_void_p),
                ("dense_down", C.c_void_p), ("pre_ffn_norm", C.c_void_p), ("pre_ffn_norm_2", C.c_void_p),
                ("post_ffn_norm_1", C.c_void_p), ("post_ffn_norm_2", C.c_void_p), ("post_ffn_norm", C.c_void_p),
                ("layer_scalar", C.c_float)]


class Workspace(C.Structure):
    _fields_ = [("grouped_out", C.c_void_p), ("group_offsets", C.c_void_p), ("selected", C.c_void_p),
                ("weights", C.c_void_p), ("canonical_to_grouped", C.c_void_p),
                ("grouped_to_canonical", C.c_void_p), ("logits", C.c_void_p), ("status", C.c_void_p),
                ("grouped_out_bytes", C.c_size_t)]


class MoeStack:
    """A stack of affine-Q4 MoE feed-forward layers resident in HBM."""

    def __init__(self, max_tokens, hidden, inter, n_experts, topk, expert_begin=0, expert_end=None):
        self.lib = load_library()
        self.lib.salt_b200_launch_count.restype = C.c_uint64
        self.handle = C.c_void_p()
        self.max_tokens, self.hidden, self.inter = max_tokens, hidden, inter
        self.n_experts, self.topk = n_experts, topk
        self.expert_begin = expert_begin
        self.expert_end = n_experts if expert_end is None else expert_end
        rc = self.lib.salt_b200_stack_create(max_tokens, hidden, inter, n_experts, topk, self.expert_begin,
                                             self.expert_end, C.byref(self.handle))
        if rc != 0:
            raise RuntimeError("salt_b200_stack_create failed (no sm_100 device, or out of memory)")
        self.n_layers = 0

    def add_layer(self, layer, with_norm=True):
        """layer: synth.Q4MoeLayer (host arrays are copied to HBM)."""
        nw = layer.norm_weight if with_norm else None
        spec = Q4LayerSpec(layer.hidden, layer.inter, layer.n_experts, layer.topk, layer.eps,
                           layer.router_w.ctypes.data, layer.router_scale.ctypes.data,
                           layer.per_expert_scale.ctypes.data, layer.pool.ctypes.data, layer.expert_stride,
                           nw.ctypes.data if nw is not None else None)
        idx = self.lib.salt_b200_stack_add_q4_layer(self.handle, C.byref(spec))
        if idx < 0:
            raise RuntimeError("salt_b200_stack_add_q4_layer failed")
        self.n_layers = idx + 1
        return idx

    def add_nvfp4_layer(self, layer, with_norm=True):
        """layer: synth.Nvfp4MoeLayer (host arrays are copied to HBM)."""
        nw = layer.norm_weight if with_norm else None
        spec = Nvfp4LayerSpec(layer.hidden, layer.inter, layer.n_experts, layer.topk, layer.eps,
                              layer.router_w.ctypes.data, layer.router_scale.ctypes.data,
                              layer.per_expert_scale.ctypes.data, layer.pool.ctypes.data, layer.expert_stride,
                              layer.weight_divisors.ctypes.data, layer.input_globals.ctypes.data,
                              nw.ctypes.data if nw is not None else None)
        idx = self.lib.salt_b200_stack_add_nvfp4_layer(self.handle, C.byref(spec))
        if idx < 0:
            raise RuntimeError("salt_b200_stack_add_nvfp4_layer failed")
        self.n_layers = idx + 1
        return idx

    def attach_ffn_block(self, layer, block):
        """block: synth.FfnBlock; completes MoE layer `layer` to the whole feed-forward block."""
        spec = FfnBlockSpec(block.dense_inter, block.dense_gate.ctypes.data, block.dense_up.ctypes.data,
                            block.dense_down.ctypes.data, block.pre_ffn_norm.ctypes.data,
                            block.pre_ffn_norm_2.ctypes.data, block.post_ffn_norm_1.ctypes.data,
                            block.post_ffn_norm_2.ctypes.data, block.post_ffn_norm.ctypes.data,
                            block.layer_scalar)
        return self.lib.salt_b200_stack_attach_ffn_block(self.handle, layer, C.byref(spec))

    def ffn_block_forward(self, layer, d_residual, B, d_out, stream=0):
        return self.lib.salt_b200_ffn_block_forward(self.handle, layer, C.c_void_p(d_residual), B,
                                                    C.c_void_p(d_out), C.c_void_p(stream))

    def workspace(self):
        w = Workspace()
        if self.lib.salt_b200_stack_workspace(self.handle, C.byref(w)) != 0:
            raise RuntimeError("salt_b200_stack_workspace failed")
        return w

    def nvfp4_buffers(self):
        """Device addresses (gate, up, chain_codes, chain_scales) of the NVFP4 intermediates of the last
        ``layer_experts`` call."""
        b = (C.c_void_p * 4)()
        if self.lib.salt_b200_stack_nvfp4_buffers(self.handle, b) != 0:
            raise RuntimeError("salt_b200_stack_nvfp4_buffers failed")
        return tuple(int(v or 0) for v in b)

    def set_fused_decode(self, enable):
        """Batches of up to 4 tokens: one-launch expert kernel (default) or the two-launch form."""
        level = int(enable)                                   # 0 phase kernels, 1 one launch per layer, 2 one per pass
        return self.lib.salt_b200_stack_set_fused_decode(self.handle, level)

    def set_grouped_out(self, device_ptr, nbytes):
        return self.lib.salt_b200_stack_set_grouped_out(self.handle, C.c_void_p(device_ptr), C.c_size_t(nbytes))

    def forward_host(self, x, first=0, count=None):
        """x [B][hidden] float32 numpy -> y; raises if the library reports failure."""
        x = np.ascontiguousarray(x, np.float32).reshape(-1, self.hidden)
        y = np.empty_like(x)
        count = self.n_layers - first if count is None else count
        rc = self.lib.salt_b200_stack_forward_host(self.handle, first, count, C.c_void_p(x.ctypes.data),
                                                   x.shape[0], C.c_void_p(y.ctypes.data))
        if rc != 0:
            raise RuntimeError(f"salt_b200_stack_forward_host failed (rc={rc})")
        return y

    def forward_device(self, d_x, B, d_y, first=0, count=None, stream=0):
        count = self.n_layers - first if count is None else count
        return self.lib.salt_b200_stack_forward_device(self.handle, first, count, C.c_void_p(d_x), B,
                                                       C.c_void_p(d_y), C.c_void_p(stream))

    EXPERTS_ZERO_REMOTE, EXPERTS_ROUTER_INPUT_READY = 1, 2
    COMBINE_NORM, COMBINE_PREPARE_NEXT = 1, 2

    def layer_experts(self, layer, d_x, B, zero_remote=False, router_input_ready=False, tensor_core=False,
                      two_launches=False, stream=0):
        """tensor_core: False (exact kernels), True / "split" (hi+lo fp16 operands), "single"."""
        tc = 0 if not tensor_core else (8 if tensor_core == "single" else 4)
        flags = (1 if zero_remote else 0) | (2 if router_input_ready else 0) | tc | (16 if two_launches else 0)
        return self.lib.salt_b200_layer_experts(self.handle, layer, C.c_void_p(d_x), B, flags, C.c_void_p(stream))

    def layer_combine(self, layer, B, d_y, apply_norm=True, prepare_next=False, stream=0):
        flags = (1 if apply_norm else 0) | (2 if prepare_next else 0)
        return self.lib.salt_b200_layer_combine(self.handle, layer, B, C.c_void_p(d_y), flags, C.c_void_p(stream))

    # expert parallelism by token dispatch (see ep.forward_dispatch)
    def layer_route(self, layer, d_x, B, d_selected, d_weights, router_input_ready=False, stream=0):
        return self.lib.salt_b200_layer_route(self.handle, layer, C.c_void_p(d_x), B, C.c_void_p(d_selected),
                                              C.c_void_p(d_weights), 2 if router_input_ready else 0, C.c_void_p(stream))

    def layer_experts_routed(self, layer, d_rows, d_experts, n_rows, d_out, tensor_core=False, stream=0):
        tc = 0 if not tensor_core else (8 if tensor_core == "single" else 4)
        return self.lib.salt_b200_layer_experts_routed(self.handle, layer, C.c_void_p(d_rows), C.c_void_p(d_experts),
                                                       n_rows, C.c_void_p(d_out), tc, C.c_void_p(stream))

    def layer_combine_rows(self, layer, d_rows, d_weights, B, d_y, apply_norm=True, prepare_next=False, stream=0,
                           d_row_index=None):
        """d_row_index (int32 [B*topk], device): where selection (token, rank) sits in d_rows; None = canonical order."""
        flags = (1 if apply_norm else 0) | (2 if prepare_next else 0)
        return self.lib.salt_b200_layer_combine_rows(self.handle, layer, C.c_void_p(d_rows), C.c_void_p(d_row_index),
                                                     C.c_void_p(d_weights), B, C.c_void_p(d_y), flags, C.c_void_p(stream))

    EP_PUSH, EP_PULL = 1, 2

    def ep_region(self):
        """(64-byte CUDA IPC handle, device address) of this stack's landing region."""
        handle = (C.c_ubyte * 64)()
        region = C.c_void_p()
        if self.lib.salt_b200_stack_ep_region(self.handle, handle, C.byref(region)) != 0:
            raise RuntimeError("salt_b200_stack_ep_region failed")
        return bytes(handle), int(region.value)

    def ep_connect(self, rank, world, ipc_handles=None, regions=None):
        """ipc_handles: list of `world` 64-byte handles (ranks in other processes), or regions: list of
        `world` device addresses (ranks in this process)."""
        if ipc_handles is not None:
            blob = b"".join(ipc_handles)
            assert len(blob) == 64 * world
            return self.lib.salt_b200_stack_ep_connect(self.handle, rank, world, blob, None)
        arr = (C.c_void_p * world)(*[C.c_void_p(r) for r in regions])
        return self.lib.salt_b200_stack_ep_connect(self.handle, rank, world, None, arr)

    def ep_disconnect(self):
        return self.lib.salt_b200_stack_ep_disconnect(self.handle)

    def ep_set_poll_limit(self, polls):
        return self.lib.salt_b200_stack_ep_set_poll_limit(self.handle, int(polls))

    def ep_reset(self):
        return self.lib.salt_b200_stack_ep_reset(self.handle)

    def ep_exchange(self, B, phase=3, stream=0):
        return self.lib.salt_b200_stack_ep_exchange(self.handle, B, phase, C.c_void_p(stream))

    KERNEL_CLASSES = ("router_input", "router_logits", "router_topk", "plan_topk", "gate_up_geglu", "down",
                      "reduce_norm_router_input", "rmsnorm")

    def graph_capture(self, d_x, B, d_y, stream, first=0, count=None):
        count = self.n_layers - first if count is None else count
        return self.lib.salt_b200_stack_graph_capture(self.handle, first, count, C.c_void_p(d_x), B,
                                                      C.c_void_p(d_y), C.c_void_p(stream))

    def graph_launch(self, stream):
        return self.lib.salt_b200_stack_graph_launch(self.handle, C.c_void_p(stream))

    def profile(self, enable, max_launches=4096):
        return self.lib.salt_b200_stack_profile(self.handle, int(enable), max_launches)

    def profile_read(self):
        ms = (C.c_float * 8)()
        n = (C.c_int * 8)()
        if self.lib.salt_b200_stack_profile_read(self.handle, ms, n, 8) != 0:
            raise RuntimeError("salt_b200_stack_profile_read failed")
        return {k: (float(ms[i]), int(n[i])) for i, k in enumerate(self.KERNEL_CLASSES)}

    def status(self, stream=0):
        return self.lib.salt_b200_stack_status(self.handle, C.c_void_p(stream))

    def launch_count(self):
        return int(self.lib.salt_b200_launch_count())

    def close(self):
        if self.handle:
            self.lib.salt_b200_stack_destroy(self.handle)
            self.handle = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
