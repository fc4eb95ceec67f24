"""The expert pool file format (header, slot order, alignment) without a GPU."""
import importlib
import struct

import numpy as np
import pytest


def test_pool_file_round_trip(synth, tmp_path):
    pf = importlib.import_module("salt-core_b200.pool_file")
    H, M, E = 128, 64, 4
    layers = [synth.make_q4_moe_layer(3 + i, hidden=H, inter=M, n_experts=E, topk=2) for i in range(3)]
    path = str(tmp_path / "p.pool")
    slot = pf.write_pool(path, layers)
    raw = open(path, "rb").read()
    assert struct.unpack_from("<QQQ", raw, 0) == (slot, 3, E)
    assert len(raw) == 24 + slot * 3 * E
    pool = pf.ExpertPool(path, H, M)
    for li in range(3):
        for e in range(E):
            assert pool.logical_id(li, e) == li * E + e
            assert (pool.payload(li, e) == layers[li].pool[e * slot:(e + 1) * slot]).all()
            for w in range(3):
                for got, want in zip(pool.tensor(li, e, w), layers[li].tensor(e, w)):
                    assert got.tobytes() == want.tobytes()
    assert pool.payload(0, 0).ctypes.data % 16 == 8          # 24-byte header, slots a multiple of 16
    pool.close()


def test_pool_file_header_is_checked(synth, tmp_path):
    pf = importlib.import_module("salt-core_b200.pool_file")
    layer = synth.make_q4_moe_layer(1, hidden=128, inter=64, n_experts=2, topk=1)
    path = str(tmp_path / "p.pool")
    pf.write_pool(path, [layer])
    with pytest.raises(ValueError):
        pf.ExpertPool(path, 128, 128)                          # another geometry: slot_bytes differs
    with open(path, "r+b") as f:
        f.truncate(24 + layer.expert_stride)                   # one slot missing
    with pytest.raises(ValueError):
        pf.ExpertPool(path, 128, 64)
    with open(path, "wb") as f:
        f.write(b"\0" * 8)
    with pytest.raises(ValueError):
        pf.ExpertPool(path, 128, 64)
