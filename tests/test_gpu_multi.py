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


def _make_decoder(mld, layers, kc, vc, heads, ffn, T, rank, world, nccl_id, shard_layout=0, **kw):
    shd = mld.sharding
    d = heads * 128
    dev = torch.device("cuda", torch.cuda.current_device())
    dec = mld.Decoder(len(layers), d, heads, ffn, T, rank=rank, world=world, nccl_id=nccl_id,
                      shard_layout=shard_layout, **kw)
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


EXCHANGES = {
    # name: (decoder mode, shard layout, extra descriptor fields, how shards travel)
    "nccl": ("op_chain", 0, {}, "nccl"),                 # chain of kernels, ncclAllGather after each producer
    "peer": ("op_chain", 0, {}, "ipc"),                  # chain of kernels storing shards into every rank's memory
    "mega": ("single", 0, {}, "ipc"),                    # one persistent kernel per rank, tagged words over NVLink
    "mega_barriers": ("single", 0, {"handover": 1}, "ipc"),   # the same with cross-rank grid barriers
    "mega_paired": ("single", 1, {}, "ipc"),             # o / down split by input columns, fp32 partial sums
}
SHAPES = {"small": (2, 4, 512, 64, 40), "wide": (2, 8, 2816, 300, 257)}   # L, heads, ffn, T, pos


def _setup(rank, world, port):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    import __graft_entry__ as g
    mld = g.import_package()
    torch.cuda.set_device(rank)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    dist.init_process_group("gloo", rank=rank, world_size=world)
    return mld, dist


def _sharded_decoder(mld, dist, exchange, model, heads, ffn, T, rank, world, **kw):
    mode_name, layout, extra, travel = EXCHANGES[exchange]
    mode = mld.DECODER_SINGLE_KERNEL if mode_name == "single" else mld.DECODER_OP_CHAIN
    nccl_id = None
    if travel == "nccl":
        idt = torch.zeros(128, dtype=torch.uint8)
        if rank == 0:
            idt = torch.frombuffer(bytearray(mld.comm_unique_id()), dtype=torch.uint8).clone()
        dist.broadcast(idt, 0)
        nccl_id = idt.numpy().tobytes()
    layers, kc, vc = model
    dec, keep = _make_decoder(mld, layers, kc, vc, heads, ffn, T, rank, world, nccl_id, layout, mode=mode,
                              **dict(extra, **kw))
    assert dec.single_kernel == (mode_name == "single")
    if travel == "ipc":         # shards go straight into every rank's exchange block
        mine = torch.frombuffer(bytearray(dec.ipc_export()), dtype=torch.uint8).clone()
        table = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
        dist.all_gather(table, mine)
        dec.ipc_import(b"".join(t.numpy().tobytes() for t in table))
        dist.barrier()
    return dec, keep


def _worker(rank, world, port, out_dir, exchange, shape):
    mld, dist = _setup(rank, world, port)
    L, heads, ffn, T, pos = SHAPES[shape]
    d = heads * 128
    model = _model(np.random.default_rng(0), L, heads, ffn, T)
    x = torch.from_numpy(np.random.default_rng(1).standard_normal(d).astype(np.float16)).cuda()
    dec, keep = _sharded_decoder(mld, dist, exchange, model, heads, ffn, T, rank, world)
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
        layers, kc, vc = model
        single, keep1 = _make_decoder(mld, layers, kc, vc, heads, ffn, T, 0, 1, None, mode=mld.DECODER_OP_CHAIN)
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


def _port(offset):
    return 29700 + (os.getpid() % 2000) + offset


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange,shape", [("nccl", "small"), ("peer", "small"), ("mega", "small"), ("mega", "wide"),
                                            ("mega_barriers", "small"), ("mega_paired", "small")])
def test_two_gpu_sharded_decode_equals_single_gpu(tmp_path, exchange, shape):
    import torch.multiprocessing as mp
    port = _port(list(EXCHANGES).index(exchange) * 7 + (3 if shape == "wide" else 0))
    mp.spawn(_worker, args=(2, port, str(tmp_path), exchange, shape), nprocs=2, join=True)
    err, finite, same = open(tmp_path / "result.txt").read().split()
    assert int(finite) == 1
    assert int(same) == 1                    # every rank holds the same gathered output
    assert float(err) < 1e-2


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs four GPUs")
@pytest.mark.parametrize("exchange", ["mega", "peer"])
def test_four_gpu_sharded_decode_equals_single_gpu(tmp_path, exchange):
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(4, _port(61 + list(EXCHANGES).index(exchange)), str(tmp_path), exchange, "wide"),
             nprocs=4, join=True)
    err, finite, same = open(tmp_path / "result.txt").read().split()
    assert int(finite) == 1 and int(same) == 1
    assert float(err) < 1e-2


def _late_rank_worker(rank, world, port, out_dir, exchange):
    """Rank 1 sits out one step (it stays alive and launches nothing): rank 0's step must give up within
    its wait limit, tell the host, and leave both GPUs usable; after both ranks have reset their
    decoders the next step, taken together, is right."""
    mld, dist = _setup(rank, world, port)
    L, heads, ffn, T, pos = SHAPES["small"]
    d = heads * 128
    model = _model(np.random.default_rng(0), L, heads, ffn, T)
    x = np.random.default_rng(1).standard_normal(d).astype(np.float16)
    dec, keep = _sharded_decoder(mld, dist, exchange, model, heads, ffn, T, rank, world, wait_limit_us=200000)
    xh = torch.from_numpy(x).pin_memory()
    yh = torch.empty(d, dtype=torch.float16).pin_memory()
    dec.step_host(xh, yh, pos)                 # a good step together
    dist.barrier()
    status = 0
    if rank == 0:
        try:
            dec.step_host(xh, yh, pos)             # alone: the other rank's shards never come
        except mld.MldError as e:
            status = e.status
    dist.barrier()                             # rank 1 waited here, on the host
    code = dec.device_status() if rank == 0 else 0
    dec.reset()                                # both ranks, nothing in flight
    dist.barrier()
    dec.step_host(xh, yh, pos)
    dist.barrier()
    ok = dec.device_status() == 0
    if rank == 0:
        layers, kc, vc = model
        single, keep1 = _make_decoder(mld, layers, kc, vc, heads, ffn, T, 0, 1, None, mode=mld.DECODER_OP_CHAIN)
        y1 = torch.empty(d, dtype=torch.float16, device="cuda")
        single.step(torch.from_numpy(x).cuda(), y1, pos)
        torch.cuda.synchronize()
        err = (yh.float() - y1.float().cpu()).abs().max().item() / y1.float().abs().max().item()
        with open(os.path.join(out_dir, "result.txt"), "w") as f:
            f.write(f"{status}\n{code}\n{int(ok)}\n{err}")
        single.close()
    dist.barrier()
    dec.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("exchange", ["peer", "mega"])
def test_two_gpu_step_without_the_other_rank_times_out_and_recovers(tmp_path, exchange):
    import torch.multiprocessing as mp
    mp.spawn(_late_rank_worker, args=(2, _port(90 + list(EXCHANGES).index(exchange)), str(tmp_path), exchange),
             nprocs=2, join=True)
    status, code, ok, err = open(tmp_path / "result.txt").read().split()
    assert int(status) == 5                   # MLD_TIMEOUT from mld_decoder_step_host
    assert int(code) != 0
    assert int(ok) == 1
    assert float(err) < 1e-2


# ------------------------------------------------------------------ one operator split over the ranks
def _sharded_fc_worker(rank, world, port, out_dir):
    """Every rank holds the rows [rank n, (rank + 1) n) of one FullyConnected node; the gathered output on
    every rank must equal the unsharded operator's, bit for bit (same per-output arithmetic), for both
    ways of gathering and for the prefill GEMM, the int8-activation GEMM and the decode kernel."""
    mld, dist = _setup(rank, world, port)
    dev = torch.device("cuda", rank)
    rng = np.random.default_rng(3)
    nccl_id = torch.zeros(128, dtype=torch.uint8)
    if rank == 0:
        nccl_id = torch.frombuffer(bytearray(mld.comm_unique_id()), dtype=torch.uint8).clone()
    dist.broadcast(nccl_id, 0)
    results = []
    cases = [("int4_prefill", 4, 300, 1024, 520, 0), ("w8a8_asym", 8, 300, 1024, 520, 2), ("w8a8_sym", 8, 130, 2048, 264, 1),
             ("int4_decode", 4, 1, 1024, 520, 0), ("int4_prefill_converted", 4, 600, 512, 264, 0)]
    group = mld.ShardGroup(rank, world, 2 * 1024 * 1024, nccl_id=nccl_id.numpy().tobytes())
    mine = torch.frombuffer(bytearray(group.ipc_export()), dtype=torch.uint8).clone()
    table = [torch.zeros(64, dtype=torch.uint8) for _ in range(world)]
    dist.all_gather(table, mine)
    group.ipc_import(b"".join(t.numpy().tobytes() for t in table))
    dist.barrier()
    for name, bits, M, K, n, aq in cases:
        N = n * world
        w = torch.from_numpy((rng.standard_normal((N, K)) * 0.02).astype(np.float32)).to(dev)
        x = torch.from_numpy((rng.standard_normal((M, K)) + (0.4 if aq == 2 else 0.0)).astype(np.float16)).to(dev)
        xs = x.reshape(M, K // 4, 4).permute(1, 0, 2).contiguous()
        block = 32 if bits == 4 else 0

        def make(wm):
            q, s = mld.quantize_weights(wm, bits, block)
            packed, wsum = mld.pack_weights(q, (wm.shape[0], 1, 1, K), bits, want_sum=True)
            return packed, mld.pack_scales(s, True), wsum

        def plan_for(rows):
            return mld.FullyConnectedPlan(rows, K, bits, scale_mode=mld.SCALE_BLOCK if bits == 4 else mld.SCALE_PER_CHANNEL,
                                          groups=K // 32 if bits == 4 else 1, precision=mld.F32F16, max_tokens=M,
                                          prefill_act_quant=aq, force_path=mld.PATH_GEMV if M == 1 else mld.PATH_GEMM)
        pw, ps, psum = make(w[rank * n:(rank + 1) * n].contiguous())
        plan = plan_for(n)
        if aq == 2:
            plan.set_weights_sum(psum)
        outs = {}
        for gname, gather in (("nccl", mld.GATHER_NCCL), ("peer", mld.GATHER_PEER_STORES)):
            y = group.output(N * M, dev)
            y.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            for _ in range(2):                       # twice: the second run overwrites a consumed tensor
                group.run(plan, xs, pw, ps, M, gather)
            torch.cuda.synchronize()
            assert group.device_status() == 0
            outs[gname] = y.clone()
            dist.barrier()
        plan.close()
        fw, fs, fsum = make(w)
        full = plan_for(N)
        if aq == 2:
            full.set_weights_sum(fsum)
        yf = torch.empty(N * M, dtype=torch.float16, device=dev)
        full.run(xs, fw, fs, yf, M)
        torch.cuda.synchronize()
        full.close()
        def same(a):
            if M == 1:      # the decode kernel's split of K over CTAs depends on the row count: fp32 summation order
                return bool((a.float() - yf.float()).abs().max() <= 1e-3 * yf.float().abs().max())
            return bool(torch.equal(a, yf))
        results.append((name, same(outs["nccl"]), same(outs["peer"])))
    gathered = [None] * world
    dist.all_gather_object(gathered, results)
    if rank == 0:
        with open(os.path.join(out_dir, "result.txt"), "w") as f:
            f.write(repr(gathered))
    dist.barrier()
    group.close()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_sharded_operator_gathers_the_unsharded_output(tmp_path):
    import torch.multiprocessing as mp
    mp.spawn(_sharded_fc_worker, args=(2, _port(120), str(tmp_path)), nprocs=2, join=True)
    gathered = eval(open(tmp_path / "result.txt").read())
    for rank_results in gathered:
        for name, nccl_ok, peer_ok in rank_results:
            assert nccl_ok, name
            assert peer_ok, name
