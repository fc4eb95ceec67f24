#!/usr/bin/env python
"""Benchmark of the quantized MoE feed-forward decode path on B200.

Workload (config 2 of the baseline: one MoE-FFN layer, hidden 2816, 128 experts,
top-8, expert GeGLU 2816->704->2816, all affine-Q4 group-64, fp32 router),
decode batch B, run as the 30-layer stack of config 5 (independent seeds per
layer, RMSNorm between layers) so that every step streams ~0.85 GB of distinct
expert weights -- far more than the 126 MB L2.  The metric is tokens/s through
one MoE-FFN layer: B * layers / time of one pass over the stack.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--layers L]
    python bench.py --impl reference ...      # the reference's own CPU path

One JSON line is printed by rank 0.  With N > 1 (under torchrun) the experts of
every layer are sharded expert-parallel over the ranks, every rank holds N*B
tokens' activations (replicated, deterministic routing), and the per-selection
expert outputs are exchanged once per layer.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, M, E, K = 2816, 704, 128, 8
TENSOR_BYTES = 1_115_136                      # one 704x2816 Q4 projection (values + scales + biases)
METRIC = "q4_moe_ffn_decode_tokens_per_s"
UNIT = "tokens/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=1, help="decode tokens per GPU")
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--format", default="q4", choices=["q4", "nvfp4"],
                    help="q4: the headline workload (cfg 2 layers); nvfp4: cfg 4 layers (64 NVFP4 experts, hidden 5120, "
                         "intermediate 1536, top-4), 8 layers unless --layers is given")
    ap.add_argument("--cpu-seconds", type=float, default=10.0, help="budget of the CPU baseline sample")
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the untimed extras of the default run (batch sweep, expert-phase roofline, parity check)")
    ap.add_argument("--ep-exchange", choices=["peer", "nccl", "dispatch"], default="peer",
                    help="N>1: exchange of the grouped expert outputs by the stack's own kernel over peer "
                         "memory (falls back to nccl when the regions cannot be mapped), by an NCCL all-reduce, or "
                         "dispatch: tokens partitioned by home rank, rows sent to the owners of their experts and "
                         "results returned to the home rank by NCCL all-to-alls")
    ap.add_argument("--prefill", default=None, choices=["exact", "single", "split", "blockscaled"],
                    help="run the layers one by one with the expert projections on the exact kernels, or on the "
                         "tensor cores: affine-Q4 with operands rounded to fp16 once (single) or carried as hi+lo "
                         "halves (split); NVFP4 as block-scaled mxf4nvf4 GEMMs (blockscaled)")
    args = ap.parse_args()
    if args.layers is None:
        args.layers = 30 if args.format == "q4" else 8
    if args.format == "nvfp4":
        # cfg 4 geometry; one NVFP4 tensor = codes + E4M3 block scales (+ two fp32 scalars)
        globals().update(H=5120, M=1536, E=64, K=4, TENSOR_BYTES=5120 * 1536 // 2 + 5120 * 1536 // 16 + 8,
                         METRIC="nvfp4_moe_ffn_decode_tokens_per_s")
    return args


def workload_config(args, world):
    kind = "decode" if not args.prefill else f"prefill ({args.prefill} expert projections)"
    if args.format == "nvfp4":
        return {"workload": f"cfg4 MoE-FFN layer {kind} (H5120 E64 top4 M1536, NVFP4 W4A4 experts: E2M1 codes, E4M3 "
                            f"block scales, fp32 router), run as a {args.layers}-layer stack with RMSNorm between layers",
                "batch_per_gpu": args.batch, "global_batch": args.batch * world, "layers": args.layers,
                "parallelism": f"ep{world}" if world > 1 else "single",
                "l2": f"inputs larger than L2 ({args.layers} x 849 MB of expert weights, 53 MB of them selected per "
                      "layer at B=1)"}
    return {"workload": f"cfg2 MoE-FFN layer {kind} (H2816 E128 top8 M704, affine-Q4 g64, fp32 router), "
                        "run as the cfg5 30-layer stack with RMSNorm between layers",
            "batch_per_gpu": args.batch, "global_batch": args.batch * world, "layers": args.layers,
            "parallelism": f"ep{world}" if world > 1 else "single",
            "l2": "inputs larger than L2 (about 0.85 GB of distinct expert weights streamed per step at B=1)"}


class ClockSampler:
    """nvidia-smi clocks during the timed region (read-only query)."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.rows = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def make_layer(synth, fmt, seed):
    return synth.make_q4_moe_layer_bulk(seed) if fmt == "q4" else synth.make_nvfp4_moe_layer(seed)


def cpu_layer(drv, orc, fmt, layer, x, threads):
    """One layer on the CPU checker: the compiled reference functions when they were built, else the port."""
    import oracle
    if fmt == "nvfp4":
        impl = oracle.Reference() if oracle.Reference.available() else orc
        return oracle.moe_layer_nvfp4(impl, layer, x, threads=threads)[0]
    if drv is not None:
        return drv.moe_layer_q4(layer, x)[0]
    return orc.moe_layer_q4(layer, x, threads=threads)[0]


def generate_layers(synth, n_layers, keep_host, consume, fmt="q4"):
    """Generate the stack's layers on a thread pool and hand each to `consume`
    (upload) in order; returns the first `keep_host` layers for the CPU baseline."""
    kept = []
    with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        futs = []
        window = 6                                # bounds host memory: 6 x 428 MB in flight
        nxt = 0
        for i in range(n_layers):
            while len(futs) < window and nxt < n_layers:
                futs.append(pool.submit(make_layer, synth, fmt, 5000 + nxt))
                nxt += 1
            layer = futs.pop(0).result()
            consume(i, layer)
            if i < keep_host:
                kept.append(layer)
    return kept


def cpu_baseline(layers, B, seconds, threads, fmt="q4"):
    """The reference's own CPU decode path (oracle/_ref, all host cores) on a bounded
    sample: the host-kept layers are cycled for about `seconds`."""
    import oracle
    synth = importlib.import_module("salt-core_b200.synth")
    x = synth.make_tokens(77, B, H)
    if fmt == "nvfp4":
        # the reference's NVFP4 CPU path takes about a second per token and layer: a bounded sample of tokens
        kind = "reference" if oracle.Reference.available() else "port"
        orc, used = oracle.Oracle(), threads
        x = x[:max(1, min(B, int(seconds / 4)))]
        B = x.shape[0]
        run = lambda layer: cpu_layer(None, orc, fmt, layer, x, threads)
    elif oracle.RefDriver.available():
        drv, kind = oracle.RefDriver(threads), "reference"
        run = lambda layer: drv.moe_layer_q4(layer, x)
        used = drv.threads
    else:
        orc, kind, used = oracle.Oracle(), "port", threads
        run = lambda layer: orc.moe_layer_q4(layer, x, threads=threads)
    run(layers[0])
    t0 = time.perf_counter()
    n = 0
    while True:
        run(layers[n % len(layers)])
        n += 1
        el = time.perf_counter() - t0
        if el >= seconds or n >= 100000:
            break
    return {"value": B * n / el, "unit": UNIT, "cores": used, "kind": kind,
            "sample": f"{n} single-layer passes at B={B} cycling {len(layers)} distinct layers "
                      f"({el:.1f} s); reference functions on " +
                      ("a persistent pthread pool" if fmt == "q4" else "the reference's own row threads, one projection at a time"),
            "ms_per_layer": 1e3 * el / n}


def cpu_parity(layers, x, y_gpu, threads, fmt="q4"):
    """Part of the CPU-baseline leg: the same layers on the CPU checker (the compiled reference where it
    was built, else the port), compared with the GPU result bit for bit.  Not timed."""
    import oracle
    cur = np.ascontiguousarray(x, np.float32)
    if fmt == "nvfp4":
        # tokens are independent: the first two of the batch bound the CPU time
        cur, y_gpu = cur[:2], y_gpu[:2]
        orc = oracle.Oracle()
        kind = "reference functions (oracle/_ref)" if oracle.Reference.available() else "CPU port (oracle/salt_oracle.c)"
        for i, layer in enumerate(layers):
            cur = cpu_layer(None, orc, fmt, layer, cur, threads)
            if i + 1 < len(layers):
                cur = np.stack([orc.rmsnorm(cur[t], layer.norm_weight, layer.eps, True)[1] for t in range(cur.shape[0])])
    elif oracle.RefDriver.available():
        drv, kind = oracle.RefDriver(threads), "reference functions (oracle/_ref)"
        for i, layer in enumerate(layers):
            cur, _, _ = drv.moe_layer_q4(layer, cur)
            if i + 1 < len(layers):
                cur = drv.rmsnorm_rows(cur, layer.norm_weight, layer.eps)
    else:
        orc, kind = oracle.Oracle(), "CPU port (oracle/salt_oracle.c)"
        for i, layer in enumerate(layers):
            cur, _, _ = orc.moe_layer_q4(layer, cur, threads=threads)
            if i + 1 < len(layers):
                cur = np.stack([orc.rmsnorm(cur[t], layer.norm_weight, layer.eps, True)[1] for t in range(cur.shape[0])])
    same = bool((np.ascontiguousarray(cur).view(np.uint32) == np.ascontiguousarray(y_gpu).view(np.uint32)).all())
    return {"vs": f"{kind}, first {len(layers)} layers of the stack, {cur.shape[0]} of the {x.shape[0]} tokens",
            "bit_identical": same}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    synth = importlib.import_module("salt-core_b200.synth")
    threads = os.cpu_count() or 1
    n_host = min(3, args.layers)
    layers = [make_layer(synth, args.format, 5000 + i) for i in range(n_host)]
    world = max(1, args.gpus)
    B = args.batch * world
    import oracle
    x = synth.make_tokens(77, B, H)
    if args.format == "nvfp4":
        orc = oracle.Oracle()
        kind, used = ("reference" if oracle.Reference.available() else "port"), threads
        x = x[:max(1, min(B, 2))]             # about a second per token and layer on the host
        B = x.shape[0]
        def step():
            cur = x
            for layer in layers:
                y = cpu_layer(None, orc, "nvfp4", layer, cur, threads)
                cur = np.stack([orc.rmsnorm(y[t], layer.norm_weight, layer.eps, True)[1] for t in range(B)])
    elif oracle.RefDriver.available():
        drv = oracle.RefDriver(threads)
        kind, used = "reference", drv.threads
        def step():
            cur = x
            for layer in layers:
                y, _, _ = drv.moe_layer_q4(layer, cur)
                cur = drv.rmsnorm_rows(y, layer.norm_weight, layer.eps)
    else:
        orc = oracle.Oracle()
        kind, used = "port", threads
        def step():
            cur = x
            for layer in layers:
                y, _, _ = orc.moe_layer_q4(layer, cur, threads=threads)
                cur = np.stack([orc.rmsnorm(y[t], layer.norm_weight, layer.eps, True)[1] for t in range(B)])
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    el = time.perf_counter() - t0
    ms = 1e3 * el / args.steps
    value = B * n_host / (ms * 1e-3)
    sample = (f"each step = {n_host} layers of the stack (of {args.layers}) at B={B}, RMSNorm between layers; "
              f"reference CPU functions, {used} threads")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args, world),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": used, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))


def nvfp4_extra(torch, stack_mod, synth, stream, peak):
    """Configuration 4 (64 NVFP4 experts, hidden 5120, intermediate 1536, top-4) on a two-layer stack of its
    own, device-timed, outside the headline: decode at B = 1 on the bit-exact kernels and B = 256 with the
    expert projections as block-scaled tcgen05 GEMMs."""
    import ctypes as C
    H4, M4, E4, K4, L4 = 5120, 1536, 64, 4, 2
    tensor_bytes = H4 * M4 // 2 + H4 * M4 // 16 + 8
    st = stack_mod.MoeStack(256, H4, M4, E4, K4)
    for i in range(L4):
        st.add_nvfp4_layer(synth.make_nvfp4_moe_layer(5400 + i))
    sp = stream.cuda_stream
    out = {}
    for bb, tc in ((1, False), (1, True), (16, False), (16, True), (256, True)):
        xs = torch.from_numpy(synth.make_tokens(77, bb, H4)).cuda()
        acts = [torch.empty_like(xs), torch.empty_like(xs)]
        ys = torch.empty_like(xs)

        def run():
            cur = xs.data_ptr()
            for l in range(L4):
                o = ys if l == L4 - 1 else acts[l & 1]
                assert st.layer_experts(l, cur, bb, router_input_ready=l > 0, tensor_core=tc, stream=sp) == 0
                assert st.layer_combine(l, bb, o.data_ptr(), apply_norm=True, prepare_next=l + 1 < L4, stream=sp) == 0
                cur = o.data_ptr()
        for _ in range(3):
            run()
        n_it = 10
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(n_it):
            run()
        e1.record(stream)
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / n_it
        assert st.status(sp) == 0
        offs = np.empty(E4 + 1, np.int32)
        st.lib.salt_b200_read_device(C.c_void_p(offs.ctypes.data), C.c_void_p(st.workspace().group_offsets),
                                     C.c_size_t(offs.nbytes))
        distinct = int((np.diff(offs) > 0).sum())     # of the last layer run
        by = distinct * 3 * tensor_bytes + E4 * H4 * 4 + bb * H4 * 4 * 3 + bb * K4 * (2 * M4 + 2 * H4) * 4
        out[f"B{bb}" + ("_blockscaled" if tc else "_exact")] = {"tokens_per_s": bb * L4 / (ms * 1e-3), "us_per_layer": 1e3 * ms / L4,
                         "expert_projections": ("tcgen05.mma.kind::mxf4nvf4 block-scaled (each projection within 1e-3 of "
                                                "the exact path)") if tc else "exact (bit-exact vs CPU)",
                         "algorithmic_bytes_per_layer": by, "hbm_frac": by / (1e3 * ms / L4 * 1e-6) / 1e9 / peak}
    st.close()
    return out


def run_b200(args):
    import torch
    import torch.distributed as dist
    pkg = importlib.import_module("salt-core_b200")
    pkg.load_library()                        # raises when the CUDA library is missing: no fallback
    synth = pkg.synth
    stack_mod = importlib.import_module("salt-core_b200.stack")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    if world > 1:
        # NCCL's version banner goes to stdout, where exactly one JSON line is expected
        if os.environ.get("NCCL_DEBUG", "VERSION").upper() == "VERSION":
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    B = args.batch * world
    L = args.layers
    lo, hi = importlib.import_module("salt-core_b200.ep").expert_range(rank, world, E)
    fmt = args.format
    if (fmt == "nvfp4") != (args.prefill in (None, "exact", "blockscaled")) and args.prefill not in (None, "exact"):
        raise SystemExit("--prefill single/split are the affine-Q4 tensor-core kernels, blockscaled the NVFP4 one")
    extras = world == 1 and not args.prefill and not args.no_extra and B == 1 and fmt == "q4"
    stack = stack_mod.MoeStack(max(B, 512 if extras else 1), H, M, E, K, expert_begin=lo, expert_end=hi)
    upload = stack.add_layer if fmt == "q4" else stack.add_nvfp4_layer
    host_layers = generate_layers(synth, L, (3 if fmt == "q4" else 2) if rank == 0 else 0, lambda i, layer: upload(layer), fmt)
    x_host = synth.make_tokens(77, B, H)
    stream = torch.cuda.Stream()
    sp = stream.cuda_stream
    d_x = torch.from_numpy(x_host).cuda()
    d_y = torch.empty_like(d_x)
    act = [torch.empty_like(d_x), torch.empty_like(d_x)]
    grouped = None
    if world > 1:                             # the NCCL exchange works on a buffer this process owns
        grouped = torch.zeros(B * K * H, dtype=torch.float32, device="cuda")
        assert stack.set_grouped_out(grouped.data_ptr(), grouped.numel() * 4) == 0

    ep = importlib.import_module("salt-core_b200.ep")

    dispatch = world > 1 and args.ep_exchange == "dispatch"
    b_loc = args.batch
    x_loc = d_x[rank * b_loc:(rank + 1) * b_loc]
    y_loc = d_y[rank * b_loc:(rank + 1) * b_loc]
    act_loc = [act[0][:b_loc], act[1][:b_loc]]
    dispatch_stats = {}

    def forward_ep(src, dst):
        """Expert-parallel pass: one exchange of the grouped expert outputs per layer, or token dispatch."""
        if dispatch:
            # the last layer's norm as the single-GPU path of the same mode has it (token 0's CRC then agrees)
            ep.forward_dispatch(ep.StackOps(stack, tc_mode), x_loc, y_loc, act_loc, norm_last=bool(args.prefill),
                                stats=dispatch_stats)
        else:
            ep.forward(stack, grouped, src, B, dst, act, stream=sp)

    tc_mode = {None: False, "exact": False, "single": "single", "split": "split", "blockscaled": True}[args.prefill]

    def forward_layers(src, dst):
        """Layer by layer through the two-phase entry points (the only way to pick the projection kernels)."""
        cur = src.data_ptr()
        for l in range(L):
            out = dst if l == L - 1 else act[l & 1]
            assert stack.layer_experts(l, cur, B, router_input_ready=l > 0, tensor_core=tc_mode, stream=sp) == 0
            assert stack.layer_combine(l, B, out.data_ptr(), apply_norm=True, prepare_next=l + 1 < L, stream=sp) == 0
            cur = out.data_ptr()

    peer = world > 1 and args.ep_exchange == "peer" and not args.prefill and ep.connect_peer_memory(stack)
    if world > 1 and args.prefill and not dispatch:
        raise SystemExit("expert-parallel prefill runs with --ep-exchange dispatch")
    use_graph = (world == 1 or peer) and not args.no_graph and not args.prefill
    with torch.cuda.stream(stream):
        n0 = stack.launch_count()
        if world > 1 and not peer:
            forward_ep(d_x, d_y)
        elif args.prefill:
            forward_layers(d_x, d_y)
        else:
            assert stack.forward_device(d_x.data_ptr(), B, d_y.data_ptr(), stream=sp) == 0
        launches_per_step = stack.launch_count() - n0
        dispatch_stats.clear()
        if peer:
            # a rank that never saw a peer's rows (bounded wait ran out) sends every rank back to NCCL
            failed = torch.tensor([stack.status(sp)], dtype=torch.int32, device="cuda")
            dist.all_reduce(failed, op=dist.ReduceOp.MAX)
            if int(failed.item()) != 0:
                dist.barrier()
                stack.ep_disconnect()
                peer, use_graph = False, False
                n0 = stack.launch_count()
                forward_ep(d_x, d_y)
                launches_per_step = stack.launch_count() - n0
        assert stack.status(sp) == 0
        if use_graph:
            assert stack.graph_capture(d_x.data_ptr(), B, d_y.data_ptr(), sp) == 0
        if peer:
            dist.barrier()                    # ranks start their exchanges together

        def step():
            if use_graph:
                assert stack.graph_launch(sp) == 0
            elif world > 1 and not peer:
                forward_ep(d_x, d_y)
            elif args.prefill:
                forward_layers(d_x, d_y)
            else:
                assert stack.forward_device(d_x.data_ptr(), B, d_y.data_ptr(), stream=sp) == 0

        def timed(fn, steps):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(steps):
                fn()
            e1.record(stream)
            torch.cuda.synchronize()
            ms = torch.tensor([e0.elapsed_time(e1)], device="cuda")
            if world > 1:
                dist.barrier()
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return float(ms.item()) / steps

        for _ in range(max(3, args.warmup)):
            step()
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
            time.sleep(0.3)
        ms_step = timed(step, args.steps)
        clocks = sampler.stop() if rank == 0 else None
        assert stack.status(sp) == 0

        # end to end through the public host API: pinned host input -> H2D -> stack -> D2H
        h_in = torch.from_numpy(x_host).pin_memory()
        h_out = torch.empty_like(h_in).pin_memory()

        def e2e_step():
            if world == 1 and not args.prefill:
                stack.forward_host(x_host)
            else:
                if dispatch:
                    x_loc.copy_(h_in[rank * b_loc:(rank + 1) * b_loc], non_blocking=True)
                else:
                    d_x.copy_(h_in, non_blocking=True)
                if use_graph:
                    assert stack.graph_launch(sp) == 0
                elif peer:
                    assert stack.forward_device(d_x.data_ptr(), B, d_y.data_ptr(), stream=sp) == 0
                elif world > 1:
                    forward_ep(d_x, d_y)
                else:
                    forward_layers(d_x, d_y)
                if dispatch:
                    h_out[rank * b_loc:(rank + 1) * b_loc].copy_(y_loc, non_blocking=True)
                else:
                    h_out.copy_(d_y, non_blocking=True)
                stream.synchronize()

        if peer:
            dist.barrier()
        for _ in range(3):
            e2e_step()
        if world == 1 and not args.prefill:
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(args.steps):
                e2e_step()
            ms_e2e = 1e3 * (time.perf_counter() - t0) / args.steps
        else:
            ms_e2e = timed(e2e_step, args.steps)

        # per-kernel-class device time (CUDA event pairs around every launch), separate pass
        kernels, roofline, roofline_layer, extra = {}, None, None, {}
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_tf = float(peaks.get("bf16_tflops", 1590.0))
        peak_source = "measured (MEASURED_PEAKS.json)" if peaks else "fallback 6650 GB/s / 1590 TFLOP/s"
        if world == 1:
            import ctypes as C

            def profiled(run, steps):
                stack.profile(True, max_launches=8 * L * steps + 16)
                for _ in range(steps):
                    run()
                prof = stack.profile_read()
                stack.profile(False, 0)
                return {name: {"launches": n, "total_ms": ms, "us_per_launch": 1e3 * ms / n}
                        for name, (ms, n) in prof.items() if n}

            def distinct_experts(batch, src, bufs):
                """Mean number of distinct experts a layer selects (decides its algorithmic bytes)."""
                out, offs, cur = [], np.empty(E + 1, np.int32), src.data_ptr()
                ws = stack.workspace()
                for l in range(L):
                    nxt = bufs[l & 1]
                    stack.layer_experts(l, cur, batch, router_input_ready=l > 0, stream=sp)
                    stack.layer_combine(l, batch, nxt.data_ptr(), apply_norm=True, prepare_next=True, stream=sp)
                    stack.lib.salt_b200_read_device(C.c_void_p(offs.ctypes.data), C.c_void_p(ws.group_offsets),
                                                    C.c_size_t(offs.nbytes))
                    out.append(int((np.diff(offs) > 0).sum()))
                    cur = nxt.data_ptr()
                return float(np.mean(out))

            def layer_bytes(distinct, batch):
                """Algorithmic bytes of one layer: the selected experts' three tensors, the router
                weights, and the activation rows read and written along the way."""
                act_bytes = batch * H * 4 * 3 + batch * K * (2 * M + 2 * H) * 4
                return distinct * 3 * TENSOR_BYTES + E * H * 4 + act_bytes

            # events are recorded around direct launches (a graph replay has no host-side launch to bracket)
            direct = (lambda: forward_layers(d_x, d_y)) if args.prefill else \
                     (lambda: stack.forward_device(d_x.data_ptr(), B, d_y.data_ptr(), stream=sp))
            kernels = profiled(direct, args.steps)
            mean_distinct = distinct_experts(B, d_x, act)
            gu = kernels["gate_up_geglu"]
            one_launch = fmt == "q4" and B == 1 and not args.prefill and "down" not in kernels
            if one_launch:
                # one launch per layer: the kernel holds the router phases too, so its bytes are the layer's
                alg = layer_bytes(mean_distinct, B)
                kname = "q4_layer_decode_kernel (reduce + norm + router + top-k + gate/up + GeGLU + down of one layer)"
            else:
                alg = mean_distinct * 2 * TENSOR_BYTES + B * H * 4 + B * K * M * 4
                kname = ("q4_gemm_tc_kernel<fused> (tcgen05 gate/up + GeGLU)" if tc_mode
                         else "q4_tile16_kernel<2,TT> / q4_fused_expert_kernel (gate/up + GeGLU)")
                if fmt == "nvfp4":
                    # the class brackets the whole NVFP4 expert phase of a layer (five launches)
                    alg = mean_distinct * 3 * TENSOR_BYTES + B * H * 4 + B * K * (2 * H + 4 * M) * 4
                    kname = ("NVFP4 expert phase of a layer: plan, activation quantise-dequantise, nvfp4_tile_kernel "
                             "gate + up, GeGLU + quantise-dequantise, nvfp4_tile_kernel down (five launches)")
                    if tc_mode:
                        kname = ("NVFP4 expert phase of a layer: plan, activation quantise, nvfp4_gemm_tc_kernel "
                                 "(tcgen05.mma.kind::mxf4nvf4 block-scaled) gate + up, GeGLU + quantise, "
                                 "nvfp4_gemm_tc_kernel down (five launches)")
            us_launch = gu["us_per_launch"]
            if one_launch and use_graph:
                # the timed region itself: L launches of this kernel and one small reduce per step (the event
                # pairs of the profiling pass above serialise the launches and lose their dependent-launch overlap)
                tail = kernels.get("reduce_norm_router_input", {}).get("us_per_launch", 0.0)
                us_launch = (1e3 * ms_step - tail) / L
            achieved = alg / (us_launch * 1e-6) / 1e9
            roofline = {"bound": "hbm", "kernel": kname, "achieved": achieved, "peak": peak, "unit": "GB/s",
                        "frac": achieved / peak, "peak_source": peak_source, "algorithmic_bytes_per_launch": alg,
                        "us_per_launch": us_launch, "us_per_launch_serialised": gu["us_per_launch"],
                        "mean_distinct_experts": mean_distinct,
                        "traffic": None,
                        "traffic_note": "not measured by this run (an ncu capture of this kernel gives the DRAM bytes per launch)"}
            if tc_mode and fmt == "q4" and B * K / E >= 96:
                # rows per expert beyond the ridge: the expert GEMMs are bound by the tensor pipe
                flops = 2.0 * B * K * 2 * H * M
                tf = flops / (gu["us_per_launch"] * 1e-6) / 1e12
                roofline.update({"bound": "tensor", "achieved": tf, "peak": peak_tf, "unit": "TFLOP/s",
                                 "frac": tf / peak_tf, "flops_per_launch": flops})
            lb = layer_bytes(mean_distinct, B)
            us_layer = 1e3 * ms_step / L
            roofline_layer = {"bound": "hbm", "what": "one whole layer (all its kernels), graph replay",
                              "algorithmic_bytes": lb, "us_per_layer": us_layer,
                              "achieved": lb / (us_layer * 1e-6) / 1e9, "peak": peak, "unit": "GB/s",
                              "frac": lb / (us_layer * 1e-6) / 1e9 / peak}
            if extras:
                # (a) the expert phases alone (gate/up + GeGLU + down of the selected experts in one launch)
                def two_phase():
                    cur = d_x.data_ptr()
                    for l in range(L):
                        nxt = act[l & 1]
                        stack.layer_experts(l, cur, B, router_input_ready=l > 0, stream=sp)
                        stack.layer_combine(l, B, nxt.data_ptr(), apply_norm=True, prepare_next=True, stream=sp)
                        cur = nxt.data_ptr()
                kx = profiled(two_phase, max(3, args.steps // 4))["gate_up_geglu"]
                xb = mean_distinct * 3 * TENSOR_BYTES + B * H * 4 + B * K * (2 * M + H) * 4
                extra["expert_phases_kernel"] = {
                    "kernel": "q4_fused_expert_kernel (gate/up + GeGLU + down, one launch)", "us_per_launch": kx["us_per_launch"],
                    "algorithmic_bytes_per_launch": xb, "achieved_gbs": xb / (kx["us_per_launch"] * 1e-6) / 1e9,
                    "frac": xb / (kx["us_per_launch"] * 1e-6) / 1e9 / peak}
                # (b) batch sweep of the same stack (device-resident, graph replay; outside the headline)
                sweep = {}
                for bb, mode in ((4, None), (16, None), (64, None), (512, "split"), (512, "single")):
                    xs = torch.from_numpy(synth.make_tokens(77, bb, H)).cuda()
                    ys = torch.empty_like(xs)
                    acts = [torch.empty_like(xs), torch.empty_like(xs)]
                    if mode is None:
                        assert stack.graph_capture(xs.data_ptr(), bb, ys.data_ptr(), sp) == 0
                        run = lambda: stack.graph_launch(sp)
                    else:
                        def run(xs=xs, ys=ys, acts=acts, bb=bb, mode=mode):
                            cur = xs.data_ptr()
                            for l in range(L):
                                o = ys if l == L - 1 else acts[l & 1]
                                stack.layer_experts(l, cur, bb, router_input_ready=l > 0, tensor_core=mode, stream=sp)
                                stack.layer_combine(l, bb, o.data_ptr(), apply_norm=True, prepare_next=l + 1 < L, stream=sp)
                                cur = o.data_ptr()
                    for _ in range(3):
                        run()
                    n_it = 5
                    torch.cuda.synchronize()
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record(stream)
                    for _ in range(n_it):
                        run()
                    e1.record(stream)
                    torch.cuda.synchronize()
                    ms = e0.elapsed_time(e1) / n_it
                    dist = distinct_experts(bb, xs, acts)
                    by = layer_bytes(dist, bb)
                    sweep[f"B{bb}" + ("_single" if mode == "single" else "")] = {
                                       "tokens_per_s": bb * L / (ms * 1e-3), "us_per_layer": 1e3 * ms / L,
                                       "expert_projections": "exact (bit-exact vs CPU)" if mode is None else
                                       "tcgen05, hi+lo fp16 operands (max rel. error <= 1e-3)" if mode == "split" else
                                       "tcgen05, fp16 operands rounded once (max error <= 1e-3 of the row maximum)",
                                       "mean_distinct_experts": dist, "algorithmic_bytes_per_layer": by,
                                       "hbm_frac": by / (1e3 * ms / L * 1e-6) / 1e9 / peak}
                    assert stack.status(sp) == 0
                extra["batch_sweep"] = sweep
                extra["nvfp4_cfg4"] = nvfp4_extra(torch, stack_mod, synth, stream, peak)
                if use_graph:                 # leave the headline graph in place
                    assert stack.graph_capture(d_x.data_ptr(), B, d_y.data_ptr(), sp) == 0

        # token 0's final output row: the same bits at every GPU count when the path is bit-identical
        # across expert-parallel shardings (token 0 of the seeded batch is the same row for every batch size)
        import zlib
        step()
        stream.synchronize()
        y_token0_crc32 = zlib.crc32(d_y[0].cpu().numpy().tobytes()) & 0xffffffff
        parity = None
        if rank == 0 and world == 1 and not args.prefill and not args.no_extra:
            n_chk = min(len(host_layers), L)
            y_chk = torch.empty_like(d_x)
            assert stack.forward_device(d_x.data_ptr(), B, y_chk.data_ptr(), first=0, count=n_chk, stream=sp) == 0
            stream.synchronize()
            parity = (host_layers[:n_chk], y_chk.cpu().numpy())

    value = B * L / (ms_step * 1e-3)
    out = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
           "warmup": max(3, args.warmup), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
           "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": workload_config(args, world),
           "clocks": clocks,
           "e2e": {"value": B * L / (ms_e2e * 1e-3), "unit": UNIT, "h2d_bytes_per_step": B * H * 4,
                   "d2h_bytes_per_step": B * H * 4, "ms_per_step": ms_e2e,
                   "api": ("salt_b200_stack_forward_host" if world == 1 and not args.prefill else
                           "salt_b200_layer_experts / salt_b200_layer_combine per layer" if world == 1 else
                           "salt_b200_stack_forward_device with the peer-memory exchange" if peer else
                           "layer_experts/all_reduce/layer_combine")},
           "gpu_launches": launches_per_step * args.steps,
           "launch_mode": "cuda graph replay" if use_graph else "stream launches",
           "us_per_layer": 1e3 * ms_step / L}
    if world > 1:
        out["ep_exchange"] = ("peer memory (own kernel over NVLink)" if peer else
                              "token dispatch and combine by NCCL all-to-alls (tokens partitioned by home rank)"
                              if dispatch else "nccl all_reduce")
        if dispatch:
            out["e2e"]["h2d_bytes_per_step"] = b_loc * H * 4
            out["e2e"]["d2h_bytes_per_step"] = b_loc * H * 4
            out["e2e"]["api"] = "ep.forward_dispatch: salt_b200_layer_route / _experts_routed / _combine_rows + all_to_all"
    if roofline:
        out["roofline"] = roofline
        out["roofline_layer"] = roofline_layer
        out["kernels"] = kernels
    if extra:
        out["extra"] = extra
    out["y_token0_crc32"] = y_token0_crc32
    if rank == 0 and world == 1:
        out["cpu_baseline"] = cpu_baseline(host_layers, B, args.cpu_seconds, os.cpu_count() or 1, args.format)
        if parity is not None:
            out["parity"] = cpu_parity(parity[0], x_host, parity[1], os.cpu_count() or 1, args.format)
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()                        # no rank unmaps a peer's region while it is still in use
    stack.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
