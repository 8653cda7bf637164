"""Tensor-parallel sharding logic on CPU: two gloo ranks shard a packed layer,
compute their partial products with the oracle (standing in for the kernel) and
all-reduce; the result must equal the unsharded oracle result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ixrun_b200 import parallel as P
from oracle import ixb_oracle as O


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _np_packed(p):
    q = dict(p)
    q["bitmaps"] = [t.numpy() for t in p["bitmaps"]]
    q["streams"] = [t.numpy() for t in p["streams"]]
    q["scale"] = int(p["scale"].view(torch.int16).item()) & 0xFFFF
    return q


def _worker(rank, world, port, out_f, in_f, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        codes = O.laplace_codes(out_f, in_f, seed=5)
        scale = torch.tensor(0.003, dtype=torch.bfloat16)
        sc_bits = int(scale.view(torch.int16).item()) & 0xFFFF
        xb = O.f32_to_bf16_bits(np.random.default_rng(9).standard_normal((2, in_f)).astype(np.float32))
        full = O.gemm_f32(codes, sc_bits, xb, out_f, in_f)
        # row-parallel: split in_f, all-reduce partial sums
        pr = P.shard_packed(codes, scale, out_f, in_f, world, rank, "row")
        lo, hi = P.shard_bounds(in_f, world, rank, 32)
        shard_codes = O.decode_codes(_np_packed(pr))
        assert np.array_equal(shard_codes.reshape(out_f, hi - lo), codes.reshape(out_f, in_f)[:, lo:hi])
        part = torch.from_numpy(O.gemm_f32(shard_codes, sc_bits, np.ascontiguousarray(xb[:, lo:hi]), out_f, hi - lo))
        dist.all_reduce(part)
        err = float(np.abs(part.numpy() - full).max() / np.abs(full).max())
        assert err < 2e-6, err
        # column-parallel with q|k|v sections: gather the sharded outputs back in section order
        secs = [out_f // 2, out_f // 4, out_f // 4]
        pc = P.shard_packed(codes, scale, out_f, in_f, world, rank, "column", sections=secs)
        yc = torch.from_numpy(O.gemm_f32(O.decode_codes(_np_packed(pc)), sc_bits, xb, pc["out_f"], in_f))
        outs = [torch.empty_like(yc) for _ in range(world)]
        dist.all_gather(outs, yc)
        cols, base_local = [], 0
        for n in secs:
            step = n // world
            cols += [o[:, base_local: base_local + step] for o in outs]
            base_local += step
        assert np.array_equal(torch.cat(cols, dim=1).numpy(), full)
        ret[rank] = 1
    finally:
        dist.destroy_process_group()


def test_row_and_column_parallel_match_unsharded_world2():
    world, port = 2, _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, 64, 1024, ret), nprocs=world, join=True)
        assert dict(ret) == {0: 1, 1: 1}


def test_shard_bounds_and_errors():
    assert P.shard_bounds(17408, 8, 3, 32) == (6528, 8704)
    with pytest.raises(ValueError):
        P.shard_bounds(5120 + 32, 8, 0, 32)
    codes = np.zeros((4, 64), dtype=np.int8)
    with pytest.raises(ValueError):
        P.shard_codes(codes, 4, 64, 2, 0, "diagonal")
    with pytest.raises(ValueError):
        P.shard_codes(codes, 4, 64, 2, 0, "column", sections=[1, 2])


def test_shard_geometry_of_the_full_model():
    from ixrun_b200.hybrid27b import HybridConfig, linear_shapes, shard_geometry

    cfg = HybridConfig()
    for world in (1, 2, 4, 8):
        g = shard_geometry(cfg, world)
        s = linear_shapes(cfg, world)
        assert g["hq"] % g["hkv"] == 0 and g["hv"] % g["hk"] == 0
        assert s["gdn"]["out_proj"][1] * world == cfg.gdn_v_heads * cfg.gdn_dim
        assert s["attn"]["o_proj"][1] * world == cfg.attn_heads * cfg.attn_dim
        assert s["mlp"]["down_proj"][1] * world == cfg.ffn
        for kind in s.values():
            for r, c in kind.values():
                assert c % 64 == 0
