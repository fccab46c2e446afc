"""Column-sharded decode step on two GPUs vs the same model on one GPU (skipped with fewer than
two devices).  Ranks are child processes; the shards come from one global model definition."""
import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
pytestmark = pytest.mark.gpu


def _model(rng, L, heads, ffn, T):
    d = heads * 128
    layers = []
    for _ in range(L):
        layer = {n: (rng.standard_normal(shape) * 0.02).astype(np.float32)
                 for n, shape in (("qkv", (3 * d, d)), ("o", (d, d)), ("gu", (2 * ffn, d)), ("down", (d, ffn)))}
        layer["norm1"] = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float16)
        layer["norm2"] = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float16)
        layers.append(layer)
    kc = rng.standard_normal((L, T, d)).astype(np.float16)
    vc = rng.standard_normal((L, T, d)).astype(np.float16)
    return layers, kc, vc


def _make_decoder(mld, layers, kc, vc, heads, ffn, T, rank, world, nccl_id, shard_layout=0):
    shd = mld.sharding
    d = heads * 128
    dev = torch.device("cuda", torch.cuda.current_device())
    dec = mld.Decoder(len(layers), d, heads, ffn, T, rank=rank, world=world, nccl_id=nccl_id,
                      shard_layout=shard_layout)
    rows = {"qkv": shd.qkv_shard_rows(heads, 128, rank, world), "o": shd.column_shard_rows(d, rank, world),
            "gu": shd.gate_up_shard_rows(ffn, rank, world), "down": shd.column_shard_rows(d, rank, world)}
    in_cols = {"qkv": None, "gu": None, "o": None, "down": None}
    if shard_layout == 1:     # o and down keep all rows and take the input columns of the rank's heads / FFN units
        rows["o"] = rows["down"] = np.arange(d)
        in_cols["o"] = shd.input_shard_cols(d, rank, world)
        in_cols["down"] = shd.input_shard_cols(ffn, rank, world)
    cols = shd.column_shard_rows(d, rank, world)
    keep = []
    for l, layer in enumerate(layers):
        t = {}
        for n in ("qkv", "o", "gu", "down"):
            wn = layer[n][rows[n]]
            if in_cols[n] is not None:
                wn = wn[:, in_cols[n]]
            w = torch.from_numpy(np.ascontiguousarray(wn)).to(dev)
            q, s = mld.quantize_weights(w, 4, 32)
            t["w" + n], _ = mld.pack_weights(q, (w.shape[0], 1, 1, w.shape[1]), 4)
            t["s" + n] = mld.pack_scales(s, True)
        t["norm1"] = torch.from_numpy(layer["norm1"]).to(dev)
        t["norm2"] = torch.from_numpy(layer["norm2"]).to(dev)
        t["kcache"] = torch.from_numpy(np.ascontiguousarray(kc[l][:, cols])).to(dev)
        t["vcache"] = torch.from_numpy(np.ascontiguousarray(vc[l][:, cols])).to(dev)
        dec.set_layer(l, **t)
        keep.append(t)
    return dec, keep


def _worker(rank, world, port, out_dir, exchange):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import __graft_entry__ as g
    mld = g.import_package()
    torch.cuda.set_device(rank)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    nccl_id = None
    # "mega": every rank runs the whole step as one persistent kernel, shards go to the peers with plain
    # stores and the kernel's barriers span the ranks; "peer" / "nccl": the chain of kernels
    os.environ["MLD_DECODER_MODE"] = "mega" if exchange.startswith("mega") else "ops"
    layout = 1 if exchange == "mega_paired" else 0
    if exchange == "nccl":
        idt = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            idt = torch.frombuffer(bytearray(mld.comm_unique_id()), dtype=torch.uint8).clone()
        dist.broadcast(idt, 0)
        nccl_id = idt.numpy().tobytes()
    L, heads, ffn, T, pos = 2, 4, 512, 64, 40
    d = heads * 128
    layers, kc, vc = _model(np.random.default_rng(0), L, heads, ffn, T)
    x = torch.from_numpy(np.random.default_rng(1).standard_normal(d).astype(np.float16)).cuda()
    dec, keep = _make_decoder(mld, layers, kc, vc, heads, ffn, T, rank, world, nccl_id, layout)
    assert dec.single_kernel == exchange.startswith("mega")
    if exchange in ("peer", "mega", "mega_paired"):         # shards go straight into every rank's exchange block
        mine = torch.frombuffer(bytearray(dec.ipc_export()), dtype=torch.uint8).clone()
        table = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(table, mine)
        dec.ipc_import(b"".join(t.numpy().tobytes() for t in table))
        dist.barrier()
    y = torch.empty(d, dtype=torch.float16, device="cuda")
    for _ in range(3):                       # repeated steps reuse the gather buffers
        dec.step(x, y, pos)
    torch.cuda.synchronize()
    agree = torch.zeros(d, dtype=torch.float16)
    agree.copy_(y)
    both = [torch.zeros_like(agree) for _ in range(world)]
    dist.all_gather(both, agree)
    same = all(torch.equal(both[0], b) for b in both)
    dist.barrier()
    assert dec.device_status() == 0
    if rank == 0:
        os.environ["MLD_DECODER_MODE"] = "ops"
        single, keep1 = _make_decoder(mld, layers, kc, vc, heads, ffn, T, 0, 1, None)
        y1 = torch.empty_like(y)
        single.step(x, y1, pos)
        torch.cuda.synchronize()
        err = (y.float() - y1.float()).abs().max().item() / y1.float().abs().max().item()
        with open(os.path.join(out_dir, "result.txt"), "w") as f:
            f.write(f"{err}\n{int(torch.isfinite(y).all())}\n{int(same)}")
        single.close()
    dist.barrier()
    dec.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange", ["nccl", "peer", "mega", "mega_paired"])
def test_two_gpu_sharded_decode_equals_single_gpu(tmp_path, exchange):
    import torch.multiprocessing as mp
    port = 29700 + (os.getpid() % 2000) + {"nccl": 0, "peer": 7, "mega": 13, "mega_paired": 19}[exchange]
    mp.spawn(_worker, args=(2, port, str(tmp_path), exchange), nprocs=2, join=True)
    err, finite, same = open(tmp_path / "result.txt").read().split()
    assert int(finite) == 1
    assert int(same) == 1                    # every rank holds the same gathered output
    assert float(err) < 1e-2
