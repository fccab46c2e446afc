"""Column sharding on two CPU ranks (gloo): each rank runs the FC oracle on its own shard of the
packed weights, the outputs are all-gathered, and the result equals the unsharded output exactly.
This covers the N > 1 host logic (which rows a rank owns, how fused matrices are split and
reassembled) without a GPU."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    import __graft_entry__ as g
    from oracle import oracle as orc
    shd = g.import_package().sharding
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    heads, hd, ffn, K = 4, 8, 24, 64
    d = heads * hd
    rng = np.random.default_rng(0)                         # every rank draws the same global model
    x = rng.standard_normal((1, K)).astype(np.float16).astype(np.float32)
    results = {}
    for kind, n_rows, rows in (("qkv", 3 * d, shd.qkv_shard_rows(heads, hd, rank, world)),
                               ("gate_up", 2 * ffn, shd.gate_up_shard_rows(ffn, rank, world)),
                               ("column", d, shd.column_shard_rows(d, rank, world))):
        w = (rng.standard_normal((n_rows, K)) * 0.02).astype(np.float32)
        # unsharded reference
        q, s = orc.quantize_int4_sym(w, 32)
        full = orc.fc_forward(orc.F32F16, 4, x, orc.rearrange_int8_as_uint4(q), N=n_rows, K=K, scale=s,
                              scale_mode=orc.SCALE_BLOCK, G=K // 32)[0]
        # this rank's shard, quantised and packed on its own
        qs, ss = orc.quantize_int4_sym(w[rows], 32)
        assert np.array_equal(qs, q[rows]) and np.array_equal(ss, s[rows])   # the split does not change the codes
        mine = orc.fc_forward(orc.F32F16, 4, x, orc.rearrange_int8_as_uint4(qs), N=len(rows), K=K, scale=ss,
                              scale_mode=orc.SCALE_BLOCK, G=K // 32)[0]
        gathered = [torch.empty(len(rows), dtype=torch.float32) for _ in range(world)]
        dist.all_gather(gathered, torch.from_numpy(mine.copy()))
        merged = shd.gathered_order(kind, [t.numpy() for t in gathered])
        results[kind] = bool(np.array_equal(merged, full))
    dist.barrier()
    dist.destroy_process_group()
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write(repr(results))


def test_two_rank_column_sharding_equals_unsharded(tmp_path):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        res = eval(open(tmp_path / f"rank{r}.txt").read())
        assert res == {"qkv": True, "gate_up": True, "column": True}


def test_shard_row_helpers():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as g
    shd = g.import_package().sharding
    assert shd.column_shard_rows(8, 1, 2).tolist() == [4, 5, 6, 7]
    assert shd.qkv_shard_rows(2, 2, 1, 2).tolist() == [2, 3, 6, 7, 10, 11]
    assert shd.gate_up_shard_rows(4, 0, 2).tolist() == [0, 4, 1, 5]
    allrows = np.sort(np.concatenate([shd.qkv_shard_rows(32, 128, r, 8) for r in range(8)]))
    assert np.array_equal(allrows, np.arange(3 * 4096))
    import pytest
    with pytest.raises(ValueError):
        shd.column_shard_rows(10, 0, 4)


def test_input_shard_cols_partition_the_inputs():
    """shard_layout 1: o / down take contiguous input-column slices that tile K exactly."""
    import __graft_entry__ as g
    shd = g.import_package().sharding
    for k, world in ((4096, 2), (11008, 8), (512, 4)):
        cols = [shd.input_shard_cols(k, r, world) for r in range(world)]
        assert np.array_equal(np.concatenate(cols), np.arange(k))
        assert all(len(c) == k // world for c in cols)
