"""Seeded synthetic tensors with the shapes and value distributions of the
benchmark configurations (no real checkpoints are involved anywhere).

Affine-Q4 tensors follow the reference storage format
(include/salt/kernels.h:117-130): eight 4-bit codes per little-endian uint32,
low nibble first, packed along K; one bf16 scale and one bf16 bias per 64
consecutive elements (row-major, absolute group index); w = q*scale + bias.

An expert occupies one contiguous slot ``gate | up | down``, each tensor stored
as ``values | scales | biases`` -- the slot order of the reference's expert pool
(tools/gemma4-mlx4-source.py:180-199).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

GROUP = 64


def bf16_round(x: np.ndarray) -> np.ndarray:
    """fp32 -> bf16 bits (round to nearest even), returned as uint16."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def bf16_to_f32(h: np.ndarray) -> np.ndarray:
    return (h.astype(np.uint32) << 16).view(np.float32)


def q4_tensor_bytes(R: int, C: int) -> tuple[int, int]:
    """(value bytes, scale bytes == bias bytes) of one R x C affine-Q4 tensor."""
    elems = R * C
    return elems // 2, elems // GROUP * 2


def fill_q4(rng: np.random.Generator, out: np.ndarray, R: int, C: int) -> None:
    """Write one Q4 tensor (values|scales|biases) into the uint8 view ``out``:
    nibbles iid uniform 0..15, scale ~ U(0.005, 0.02) rounded to bf16,
    bias = bf16(-8*scale)."""
    vb, gb = q4_tensor_bytes(R, C)
    assert out.size == vb + 2 * gb
    out[:vb] = rng.integers(0, 256, vb, dtype=np.uint8)
    s = bf16_round(rng.uniform(0.005, 0.02, gb // 2).astype(np.float32))
    b = bf16_round(np.float32(-8.0) * bf16_to_f32(s))
    out[vb:vb + gb] = s.view(np.uint8)
    out[vb + gb:] = b.view(np.uint8)


def make_q4(rng, R, C):
    """Stand-alone Q4 tensor: (vals uint32[R*C/8], scales uint16, biases uint16)."""
    vb, gb = q4_tensor_bytes(R, C)
    buf = np.empty(vb + 2 * gb, np.uint8)
    fill_q4(rng, buf, R, C)
    return (buf[:vb].view(np.uint32), buf[vb:vb + gb].view(np.uint16),
            buf[vb + gb:].view(np.uint16))


@dataclass
class Q4MoeLayer:
    """One MoE feed-forward layer with affine-Q4 experts, host resident."""
    hidden: int
    inter: int
    n_experts: int
    topk: int
    eps: float
    router_w: np.ndarray          # [E][H] fp32
    router_scale: np.ndarray      # [H] fp32
    per_expert_scale: np.ndarray  # [E] fp32
    pool: np.ndarray              # uint8 [E * expert_stride]
    expert_stride: int
    norm_weight: np.ndarray | None = None  # [H] fp32, RMSNorm applied to this layer's output

    @property
    def tensor_bytes(self) -> int:
        vb, gb = q4_tensor_bytes(self.inter, self.hidden)
        return vb + 2 * gb

    def tensor(self, expert: int, which: int):
        """(vals, scales, biases) views of gate (0), up (1) or down (2)."""
        vb, gb = q4_tensor_bytes(self.inter, self.hidden)
        base = expert * self.expert_stride + which * (vb + 2 * gb)
        p = self.pool
        return (p[base:base + vb].view(np.uint32),
                p[base + vb:base + vb + gb].view(np.uint16),
                p[base + vb + gb:base + vb + 2 * gb].view(np.uint16))


def make_q4_moe_layer(seed: int, hidden=2816, inter=704, n_experts=128, topk=8,
                      eps=1e-6, router_std=0.02) -> Q4MoeLayer:
    """Router weight fp32 N(0, router_std); router_scale = per_expert_scale = 1;
    experts as ``fill_q4``; RMSNorm weight 1 + 0.1*N(0,1)."""
    rng = np.random.default_rng(seed)
    vb, gb = q4_tensor_bytes(inter, hidden)
    tb = vb + 2 * gb
    stride = 3 * tb
    pool = np.empty(n_experts * stride, np.uint8)
    for e in range(n_experts):
        for which in range(3):
            R, C = (inter, hidden) if which < 2 else (hidden, inter)
            fill_q4(rng, pool[e * stride + which * tb: e * stride + (which + 1) * tb], R, C)
    return Q4MoeLayer(
        hidden, inter, n_experts, topk, eps,
        router_w=(rng.standard_normal((n_experts, hidden)) * router_std).astype(np.float32),
        router_scale=np.ones(hidden, np.float32),
        per_expert_scale=np.ones(n_experts, np.float32),
        pool=pool, expert_stride=stride,
        norm_weight=(1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32))


@dataclass
class FfnBlock:
    """Dense branch and norms that complete a MoE layer to the whole feed-forward block."""
    dense_inter: int
    dense_gate: np.ndarray          # uint8 blobs: values | scales | biases
    dense_up: np.ndarray
    dense_down: np.ndarray
    pre_ffn_norm: np.ndarray
    pre_ffn_norm_2: np.ndarray
    post_ffn_norm_1: np.ndarray
    post_ffn_norm_2: np.ndarray
    post_ffn_norm: np.ndarray
    layer_scalar: float

    def tensor(self, which: str, hidden: int):
        """(vals uint32, scales uint16, biases uint16, R, C) of dense_gate / dense_up / dense_down."""
        R, C = (hidden, self.dense_inter) if which == "dense_down" else (self.dense_inter, hidden)
        vb, gb = q4_tensor_bytes(R, C)
        buf = getattr(self, which)
        return buf[:vb].view(np.uint32), buf[vb:vb + gb].view(np.uint16), buf[vb + gb:].view(np.uint16), R, C


def make_ffn_block(seed: int, hidden=2816, dense_inter=2112) -> FfnBlock:
    """Dense GeGLU MLP (affine-Q4 as ``fill_q4``) and five RMSNorm weights 1 + 0.1*N(0,1)."""
    rng = np.random.default_rng(seed)
    blobs = []
    for R, C in ((dense_inter, hidden), (dense_inter, hidden), (hidden, dense_inter)):
        vb, gb = q4_tensor_bytes(R, C)
        buf = np.empty(vb + 2 * gb, np.uint8)
        fill_q4(rng, buf, R, C)
        blobs.append(buf)
    norms = [(1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32) for _ in range(5)]
    return FfnBlock(dense_inter, *blobs, *norms, layer_scalar=0.8125)


def make_tokens(seed: int, B: int, hidden: int) -> np.ndarray:
    return np.random.default_rng(seed).standard_normal((B, hidden)).astype(np.float32)


def make_q4_moe_layer_bulk(seed: int, hidden=2816, inter=704, n_experts=128, topk=8, eps=1e-6,
                           router_std=0.02) -> Q4MoeLayer:
    """Same distributions as ``make_q4_moe_layer`` drawn in a few vectorised
    calls (a different value stream): used for the full-size benchmark stack,
    where a layer holds 428 MB of expert weights."""
    rng = np.random.default_rng(seed)
    vb, gb = q4_tensor_bytes(inter, hidden)
    tb = vb + 2 * gb
    stride = 3 * tb
    pool = rng.integers(0, 2**64, (n_experts * stride + 7) // 8, dtype=np.uint64).view(np.uint8)[:n_experts * stride]
    view = pool.reshape(n_experts * 3, tb)
    s = bf16_round(rng.uniform(0.005, 0.02, (n_experts * 3, gb // 2)).astype(np.float32))
    b = bf16_round(np.float32(-8.0) * bf16_to_f32(s))
    view[:, vb:vb + gb] = s.view(np.uint8).reshape(n_experts * 3, gb)
    view[:, vb + gb:] = b.view(np.uint8).reshape(n_experts * 3, gb)
    return Q4MoeLayer(
        hidden, inter, n_experts, topk, eps,
        router_w=(rng.standard_normal((n_experts, hidden)) * router_std).astype(np.float32),
        router_scale=np.ones(hidden, np.float32),
        per_expert_scale=np.ones(n_experts, np.float32),
        pool=pool, expert_stride=stride,
        norm_weight=(1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32))


# ---- NVFP4 (E2M1 codes, E4M3FN block scales, per-tensor fp32 scalars) -----------
E2M1_MAG = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], np.float32)


def e4m3fn_encode(v: np.ndarray) -> np.ndarray:
    """Non-negative fp32 -> E4M3FN code, round to nearest, ties to the even code,
    saturating at 448 (the arithmetic equivalent of reference src/nvfp4.c:41-63)."""
    v = np.minimum(np.asarray(v, np.float32), np.float32(448.0))
    sub = np.rint(v * np.float32(512.0)).astype(np.uint32)
    b = v.view(np.uint32).astype(np.uint64)
    b = (b + 0x7FFFF + ((b >> 20) & 1)) >> 20
    norm = ((((b >> 3) - 120) << 3) | (b & 7)).astype(np.uint32)
    return np.where(v < np.float32(2.0 ** -6), sub, norm).astype(np.uint8)


def e4m3fn_decode(code: np.ndarray) -> np.ndarray:
    code = np.asarray(code, np.uint8).astype(np.uint32)
    ex, man = (code >> 3) & 15, code & 7
    sub = man.astype(np.float32) * np.float32(2.0 ** -9)
    norm = (((ex + 120) << 23) | (man << 20)).astype(np.uint32).view(np.float32)
    return np.where(ex == 0, sub, norm).astype(np.float32)


def e2m1_encode(t: np.ndarray) -> np.ndarray:
    """fp32 in [-6, 6] -> E2M1 code, nearest with ties to the even code (nvfp4.c:65-80)."""
    m = np.abs(t)
    c = ((m > 0.25).astype(np.uint8) + (m >= 0.75) + (m > 1.25) + (m >= 1.75) + (m > 2.5) + (m >= 3.5) + (m > 5.0))
    return (c | (np.signbit(t).astype(np.uint8) << 3)).astype(np.uint8)


def make_nvfp4(rng: np.random.Generator, R: int, C: int, std=0.02):
    """Quantise an N(0, std) matrix to NVFP4.  Returns (packed uint8 [R][C/2],
    scales uint8 [R][C/16], weight_divisor float32): the dequantised weight is
    e2m1(code) * e4m3(scale) / divisor, as compressed-tensors stores it."""
    w = (rng.standard_normal((R, C)) * std).astype(np.float32)
    divisor = np.float32(448.0 * 6.0) / np.abs(w).max()
    blocks = w.reshape(R, C // 16, 16)
    amax = np.abs(blocks).max(axis=2)
    sc = e4m3fn_encode((amax / np.float32(6.0)) * divisor)
    scale_f = e4m3fn_decode(sc) / divisor
    safe = np.where(scale_f == 0, np.float32(1.0), scale_f)
    t = np.clip(blocks / safe[:, :, None], -6.0, 6.0).astype(np.float32)
    codes = e2m1_encode(t).reshape(R, C)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    return np.ascontiguousarray(packed), np.ascontiguousarray(sc), np.float32(divisor)


@dataclass
class Nvfp4MoeLayer:
    """A MoE layer whose experts are NVFP4 (reference src/nvfp4.c).  Expert slot in ``pool``: gate codes |
    gate scales | up codes | up scales | down codes | down scales."""
    hidden: int
    inter: int
    n_experts: int
    topk: int
    eps: float
    router_w: np.ndarray
    router_scale: np.ndarray
    per_expert_scale: np.ndarray
    pool: np.ndarray                # uint8
    expert_stride: int
    weight_divisors: np.ndarray     # float32 [n_experts][3] (gate, up, down)
    input_globals: np.ndarray       # float32 [n_experts][3]
    norm_weight: np.ndarray

    def tensor(self, e: int, which: int):
        """(codes uint8 [R][C/2], scales uint8 [R][C/16], divisor, input_global, R, C) of expert e's tensor."""
        R, C = (self.inter, self.hidden) if which < 2 else (self.hidden, self.inter)
        cb, sb = R * C // 2, R * C // 16
        base = e * self.expert_stride + which * (cb + sb)
        return (self.pool[base:base + cb].reshape(R, C // 2), self.pool[base + cb:base + cb + sb].reshape(R, C // 16),
                float(self.weight_divisors[e, which]), float(self.input_globals[e, which]), R, C)


def make_nvfp4_moe_layer(seed: int, hidden=5120, inter=1536, n_experts=64, topk=4, eps=1e-6, router_std=0.02,
                         input_global=64.0, distinct=None) -> Nvfp4MoeLayer:
    """NVFP4 experts whose dequantised weights are ~N(0, 0.02): ``distinct`` experts (default: all, at most 4
    for layers of more than 16 experts) are quantised from their own N(0, 0.02) matrices with the reference's
    encoders; the others repeat them with the rows rotated by the expert index, which keeps the distribution
    and makes every expert a different matrix at a fraction of the generation time."""
    rng = np.random.default_rng(seed)
    if distinct is None:
        distinct = n_experts if n_experts <= 16 else 4
    elems = hidden * inter
    tb = elems // 2 + elems // 16
    stride = 3 * tb
    pool = np.empty(n_experts * stride, np.uint8)
    div = np.empty((n_experts, 3), np.float32)
    ig = np.full((n_experts, 3), input_global, np.float32)
    base = []
    for e in range(n_experts):
        for which in range(3):
            R, C = (inter, hidden) if which < 2 else (hidden, inter)
            if e < distinct:
                packed, sc, d = make_nvfp4(rng, R, C)
                base.append((packed, sc, d))
            else:
                packed, sc, d = base[(e % distinct) * 3 + which]
                packed, sc = np.roll(packed, e, axis=0), np.roll(sc, e, axis=0)
            off = e * stride + which * tb
            pool[off:off + R * C // 2] = packed.reshape(-1)
            pool[off + R * C // 2:off + tb] = sc.reshape(-1)
            div[e, which] = d
    return Nvfp4MoeLayer(
        hidden, inter, n_experts, topk, eps,
        router_w=(rng.standard_normal((n_experts, hidden)) * router_std).astype(np.float32),
        router_scale=np.ones(hidden, np.float32), per_expert_scale=np.ones(n_experts, np.float32),
        pool=pool, expert_stride=stride, weight_divisors=div, input_globals=ig,
        norm_weight=(1.0 + 0.1 * rng.standard_normal(hidden)).astype(np.float32))
