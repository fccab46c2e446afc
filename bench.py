"""Benchmark of the quantized FullyConnected hot path.

Workload (N = 1 and every N): one decode step of a Llama-style 7B decoder with
random-init INT4 block-32 weights (32 layers, d_model 4096, 32 heads x 128,
SwiGLU FFN 11008, RMSNorm, RoPE, fp16 KV cache of 2048 tokens, batch 1) - the
configuration the headline metric "7B INT4 decode tok/s" is quoted on.  With
N > 1 the projections are column-sharded over the ranks (strong scaling: the
model is fixed) and shard outputs are all-gathered.

One JSON line is printed by rank 0.  `value` is device-timed tokens/s with all
inputs resident in HBM; `e2e` is the same step through the host-buffer entry
point of the C ABI (H2D of the token's hidden vector, the step, D2H of the
result, every step); `roofline` describes the dominant kernel (the INT4 decode
GEMV); `cpu_baseline` is the CPU restatement timed on this host's cores on a
bounded sample.  `--impl reference` times only that CPU restatement.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "7B INT4 decode tok/s at 1/2/4/8 GPU; quantized-FC HBM GB/s & prefill TFLOP/s"
CFG = dict(layers=32, d_model=4096, heads=32, head_dim=128, ffn=11008, kv_len=2048, block=32)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=CFG["layers"], help="for quick functional runs only")
    return ap.parse_args()


# ------------------------------------------------------------------ CPU baseline
def cpu_layer_sample(n_layers, seed=0):
    """Builds n_layers of the 7B geometry on the host (quantised with the CPU oracle)."""
    import numpy as np
    from oracle import oracle as orc
    rng = np.random.default_rng(seed)
    d, ffn, blk = CFG["d_model"], CFG["ffn"], CFG["block"]
    layers = []
    for _ in range(n_layers):
        layer = {}
        for name, N, K in (("qkv", 3 * d, d), ("o", d, d), ("gu", 2 * ffn, d), ("down", d, ffn)):
            w = (rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02))
            q, s = orc.quantize_int4_sym(w, blk)
            layer[name] = (orc.rearrange_int8_as_uint4(q), np.ascontiguousarray(orc.scale_layout(s, False)), N)
        layer["norm1"] = np.ones(d, np.float32)
        layer["norm2"] = np.ones(d, np.float32)
        layers.append(layer)
    T = CFG["kv_len"] + 1
    kc = rng.standard_normal((n_layers, T, d), dtype=np.float32).astype(np.float16)
    vc = rng.standard_normal((n_layers, T, d), dtype=np.float32).astype(np.float16)
    return layers, kc, vc


def cpu_step(layers, kc, vc, x):
    """The decode step in fp32 on the CPU: FC through the oracle's OpenMP GEMV over the
    packed layout, attention and glue in numpy."""
    import numpy as np
    from oracle import oracle as orc
    from oracle import decode_ref
    heads, hd, ffn, d = CFG["heads"], CFG["head_dim"], CFG["ffn"], CFG["d_model"]
    pos = CFG["kv_len"]
    resid = None
    for l, layer in enumerate(layers):
        if resid is not None:
            x = x + resid
        xn = x / np.sqrt(np.mean(x * x) + 1e-6) * layer["norm1"]
        qkv = orc.gemv_f32_fast(4, xn, layer["qkv"][0], layer["qkv"][2], layer["qkv"][1])
        q = decode_ref.rope(qkv[:d].reshape(heads, hd), pos) / np.float32(np.sqrt(hd))
        kc[l, pos] = decode_ref.rope(qkv[d:2 * d].reshape(heads, hd), pos).reshape(-1)
        vc[l, pos] = qkv[2 * d:]
        k3 = kc[l].reshape(-1, heads, hd)
        v3 = vc[l].reshape(-1, heads, hd)
        s = np.einsum("hd,thd->ht", q.astype(np.float32), k3, dtype=np.float32)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        attn = np.einsum("ht,thd->hd", p, v3, dtype=np.float32).reshape(-1)
        o = orc.gemv_f32_fast(4, attn, layer["o"][0], layer["o"][2], layer["o"][1])
        h = x + o
        hn = h / np.sqrt(np.mean(h * h) + 1e-6) * layer["norm2"]
        gu = orc.gemv_f32_fast(4, hn, layer["gu"][0], layer["gu"][2], layer["gu"][1])
        act = gu[:ffn] / (1.0 + np.exp(-gu[:ffn])) * gu[ffn:]
        resid = orc.gemv_f32_fast(4, act, layer["down"][0], layer["down"][2], layer["down"][1])
        x = h
    return x + resid


def time_cpu(n_layers, reps, warm):
    import numpy as np
    from oracle import oracle as orc
    orc.build()
    layers, kc, vc = cpu_layer_sample(n_layers)
    x = np.random.default_rng(1).standard_normal(CFG["d_model"]).astype(np.float32)
    for _ in range(warm):
        cpu_step(layers, kc, vc, x)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        cpu_step(layers, kc, vc, x)
        times.append(time.perf_counter() - t0)
    per_layer = statistics.median(times) / n_layers
    tok_s = 1.0 / (per_layer * CFG["layers"])
    return tok_s, orc.num_threads(), times


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_layers = 2
    tok_s, cores, times = time_cpu(n_layers, reps=max(args.steps, 1), warm=max(min(args.warmup, 3), 1))
    sample = f"{n_layers} of {CFG['layers']} layers per step (KV 2048), scaled x{CFG['layers'] // n_layers}"
    line = {
        "impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / tok_s, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "7B INT4 decode step (32L, d4096, 32h x128, ffn11008, KV 2048, batch 1), "
                               "CPU restatement of the reference FullyConnected arithmetic"},
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------- GPU arm
class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for ln in out.splitlines():
            f = [c.strip() for c in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def build_model(mld, torch, rank, world, n_layers, dev, shard_layout=0):
    """Random-init 7B-geometry model, quantised and packed on the GPU by the library.  The model is
    defined globally (one seed per projection); a rank keeps the rows of its column shard, so every
    world size runs the same model."""
    d, ffn, blk, heads, hd = CFG["d_model"], CFG["ffn"], CFG["block"], CFG["heads"], CFG["head_dim"]
    dl = d // world
    T = CFG["kv_len"] + 1
    shd = mld.sharding
    layers = []
    gen = torch.Generator(device=dev)

    def qpack(n_full, K, seed, rows, cols=None):
        gen.manual_seed(seed)
        w = torch.randn((n_full, K), generator=gen, device=dev, dtype=torch.float32) * 0.02
        if len(rows) != n_full or (rows[:-1] > rows[1:]).any():     # a shard, or the interleaved gate/up order
            w = w.index_select(0, torch.from_numpy(rows).to(dev))
        if cols is not None:                                        # a shard by input columns
            w = w.index_select(1, torch.from_numpy(cols).to(dev)).contiguous()
            K = len(cols)
        q, s = mld.quantize_weights(w, 4, blk)
        packed, _ = mld.pack_weights(q, (w.shape[0], 1, 1, K), 4)
        sc = mld.pack_scales(s, True)
        del w, q, s
        return packed, sc

    head_cols = torch.from_numpy(shd.column_shard_rows(d, rank, world)).to(dev)
    for l in range(n_layers):
        base = 1000 * l
        t = {}
        t["wqkv"], t["sqkv"] = qpack(3 * d, d, base + 1, shd.qkv_shard_rows(heads, hd, rank, world))
        if shard_layout == 1:   # o and down: all rows, the input columns of this rank's heads / FFN units
            import numpy as np
            t["wo"], t["so"] = qpack(d, d, base + 2, np.arange(d), shd.input_shard_cols(d, rank, world))
            t["wdown"], t["sdown"] = qpack(d, ffn, base + 4, np.arange(d), shd.input_shard_cols(ffn, rank, world))
        else:
            t["wo"], t["so"] = qpack(d, d, base + 2, shd.column_shard_rows(d, rank, world))
            t["wdown"], t["sdown"] = qpack(d, ffn, base + 4, shd.column_shard_rows(d, rank, world))
        t["wgu"], t["sgu"] = qpack(2 * ffn, d, base + 3, shd.gate_up_shard_rows(ffn, rank, world))
        t["norm1"] = torch.ones(d, dtype=torch.float16, device=dev)
        t["norm2"] = torch.ones(d, dtype=torch.float16, device=dev)
        for name, seed in (("kcache", base + 5), ("vcache", base + 6)):
            gen.manual_seed(seed)
            full = torch.randn((T, d), generator=gen, device=dev, dtype=torch.float32).half()
            t[name] = full.index_select(1, head_cols).contiguous() if world > 1 else full
        layers.append(t)
    torch.cuda.synchronize()
    return layers


def gemv_roofline(mld, torch, layers, world, peaks, layout=0):
    """Times the decode GEMV (the dominant kernel) alone: every projection of every layer once
    per pass, back to back on the current stream, CUDA events around the passes.  The weights
    of a pass (3.6 GB / world) exceed L2, so every launch streams from HBM."""
    d, ffn, blk = CFG["d_model"], CFG["ffn"], CFG["block"]
    dl, fl = d // world, ffn // world
    shapes = {"qkv": (3 * dl, d), "o": (dl, d), "gu": (2 * fl, d), "down": (dl, ffn)}
    if layout == 1:
        shapes["o"], shapes["down"] = (d, dl), (d, fl)
    plans = {k: mld.FullyConnectedPlan(n, kk, 4, scale_mode=mld.SCALE_BLOCK, groups=kk // blk, precision=mld.F32F16)
             for k, (n, kk) in shapes.items()}
    xs = {k: torch.randn(kk, device="cuda").half() for k, (n, kk) in shapes.items()}
    ys = {k: torch.empty(n, dtype=torch.float16, device="cuda") for k, (n, kk) in shapes.items()}
    algo = 0
    for k, (n, kk) in shapes.items():
        algo += n * kk // 2 + (kk // blk) * n * 2 + kk * 2 + n * 2
    algo *= len(layers)

    def one_pass():
        for t in layers:
            for k in ("qkv", "o", "gu", "down"):
                plans[k].run(xs[k], t["w" + k], t["s" + k], ys[k], 1)

    for _ in range(3):
        one_pass()
    torch.cuda.synchronize()
    reps = 5
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        one_pass()
    e1.record()
    torch.cuda.synchronize()
    sec = e0.elapsed_time(e1) * 1e-3 / reps
    launches = 4 * len(layers)
    achieved = algo / sec / 1e9
    peak = peaks.get("hbm_gbs")
    src = "measured (MEASURED_PEAKS.json hbm_gbs)"
    if not peak:
        peak, src = 6650.0, "fallback"
    for p in plans.values():
        p.close()
    return {"bound": "hbm", "kernel": "fc_strip_kernel (INT4 decode GEMV)", "achieved": achieved, "peak": peak,
            "unit": "GB/s", "frac": achieved / peak, "peak_source": src,
            # ncu capture of the config-2 launch: 18.93 MB of DRAM reads against 18.9 MB algorithmic
            "traffic": algo / launches * 1.001,
            "traffic_source": "ncu capture of the config-2 launch, ratio applied (profiles/fc_strip_kernel_config2_ncu_full.md)",
            "launches_timed": launches * reps, "avg_launch_us": sec / launches * 1e6,
            "algorithmic_bytes_per_launch": algo / launches}


def side_benchmarks(mld, torch, peaks):
    """The two kernel-level figures the metric also names: decode GEMV bandwidth on BASELINE
    config 2 and prefill GEMM throughput on config 3, each timed alone with CUDA events."""
    out = {}
    # config 2: N=16384, K=2048, INT4 block 32, one token; 16 weight sets (303 MB) rotate to defeat L2
    N, K, blk, sets = 16384, 2048, 32, 16
    plan = mld.FullyConnectedPlan(N, K, 4, scale_mode=mld.SCALE_BLOCK, groups=K // blk, precision=mld.F32F16)
    nbytes = mld.packed_size_bytes(N, K, 4)
    ws = [torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device="cuda") for _ in range(sets)]
    ss = [(torch.rand((K // blk, N), device="cuda") * 0.01).half() for _ in range(sets)]
    x = torch.randn(K, device="cuda").half()
    y = torch.empty(N, dtype=torch.float16, device="cuda")
    for i in range(2 * sets):
        plan.run(x, ws[i % sets], ss[i % sets], y, 1)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iters = 20 * sets
    e0.record()
    for i in range(iters):
        plan.run(x, ws[i % sets], ss[i % sets], y, 1)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / iters
    algo = nbytes + (K // blk) * N * 2 + K * 2 + N * 2
    peak = peaks.get("hbm_gbs") or 6650.0
    out["fc_gemv_config2"] = {"workload": "INT4 block-32 GEMV N=16384 K=2048, 1 token, 16 rotating weight sets",
                              "us_per_launch": us, "GBps": algo / us / 1e3, "frac_of_hbm_peak": algo / us / 1e3 / peak,
                              "algorithmic_bytes": algo}
    plan.close()
    del ws, ss
    # config 3: M=1024, K=4096, N=14336
    M, K, N = 1024, 4096, 14336
    g = torch.Generator(device="cuda").manual_seed(0)
    w = torch.randn((N, K), generator=g, device="cuda") * 0.02
    q, s = mld.quantize_weights(w, 4, blk)
    packed, _ = mld.pack_weights(q, (N, 1, 1, K), 4)
    sc = mld.pack_scales(s, True)
    del w, q, s
    xs = torch.randn((K // 4, M, 4), generator=g, device="cuda").half()
    yy = torch.empty((N // 4, M, 4), dtype=torch.float16, device="cuda")
    flops = 2.0 * M * K * N
    res = {}
    for label, cache in (("with_weight_conversion", False), ("weights_prepared_once", True)):
        plan = mld.FullyConnectedPlan(N, K, 4, scale_mode=mld.SCALE_BLOCK, groups=K // blk, precision=mld.F32F16,
                                      max_tokens=M, force_path=mld.PATH_GEMM, cache_prepared_weights=cache)
        for _ in range(3):
            plan.run(xs, packed, sc, yy, M)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(20):
            plan.run(xs, packed, sc, yy, M)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / 20
        res[label] = {"us": us, "TFLOPs": flops / us / 1e6}
        plan.close()
    pk = peaks.get("bf16_tflops") or 1590.0
    out["prefill_config3"] = {"workload": "INT4 block-32 GEMM M=1024 K=4096 N=14336, fp16 in, fp32 accumulate", **res,
                              "frac_of_bf16_burst_peak": res["weights_prepared_once"]["TFLOPs"] / pk,
                              "frac_with_conversion": res["with_weight_conversion"]["TFLOPs"] / pk, "peak_TFLOPs": pk}
    return out


def run_ours(args):
    import torch
    import __graft_entry__ as g
    mld = g.import_package()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus or world == 1, "launch with torchrun --nproc-per-node N for --gpus N"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    nccl_id = None
    # how the ranks assemble sharded vectors: "peer" = the producing kernels store their shards into
    # every rank's memory over NVLink; "nccl" = an all-gather after each producing kernel
    exchange = os.environ.get("MLD_SHARD_EXCHANGE", "peer") if world > 1 else "none"
    if world > 1:
        # the persistent step kernel exchanges shards itself (peer stores); the NCCL variant is a kernel chain
        os.environ["MLD_DECODER_MODE"] = "ops" if exchange == "nccl" else os.environ.get("MLD_DECODER_MODE", "mega")
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
        if exchange == "nccl":
            idt = torch.zeros(128, dtype=torch.uint8, device=dev)
            if rank == 0:
                idt.copy_(torch.frombuffer(bytearray(mld.comm_unique_id()), dtype=torch.uint8))
            dist.broadcast(idt, 0)
            nccl_id = bytes(idt.cpu().numpy().tobytes())

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass

    n_layers = args.layers
    # sharded step kernel: o and down split by input columns (two exchanges per layer instead of four)
    layout = int(os.environ.get("MLD_SHARD_LAYOUT", "1")) if world > 1 and os.environ.get("MLD_DECODER_MODE") == "mega" else 0
    layers = build_model(mld, torch, rank, world, n_layers, dev, layout)
    T = CFG["kv_len"] + 1
    dec = mld.Decoder(n_layers, CFG["d_model"], CFG["heads"], CFG["ffn"], T, block=CFG["block"], rank=rank,
                      world=world, nccl_id=nccl_id, shard_layout=layout)
    for l, t in enumerate(layers):
        dec.set_layer(l, **t)
    if exchange == "peer":
        mine = torch.frombuffer(bytearray(dec.ipc_export()), dtype=torch.uint8).to(dev)
        table = [torch.zeros(64, dtype=torch.uint8, device=dev) for _ in range(world)]
        dist.all_gather(table, mine)
        dec.ipc_import(b"".join(t.cpu().numpy().tobytes() for t in table))
        barrier()
    pos = CFG["kv_len"]
    gen = torch.Generator(device=dev).manual_seed(7)
    x = torch.randn(CFG["d_model"], generator=gen, device=dev, dtype=torch.float32).half()
    y = torch.empty_like(x)

    # launches per step (counted by the library)
    c0 = mld.kernel_launch_count()
    dec.step(x, y, pos)
    torch.cuda.synchronize()
    launches_per_step = mld.kernel_launch_count() - c0

    # capture one step in a CUDA graph; fall back to direct launches if capture is refused
    stream = torch.cuda.Stream()
    graph = None
    single = dec.single_kernel
    try:
        if single:
            raise RuntimeError("the step is one cooperative launch; nothing to capture")
        with torch.cuda.stream(stream):
            dec.step(x, y, pos)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                dec.step(x, y, pos)
        torch.cuda.synchronize()
    except Exception as exc:  # noqa: BLE001
        graph = None
        if not single:
            sys.stderr.write(f"[bench] CUDA graph capture unavailable ({exc}); timing direct launches\n")

    def step_once():
        if graph is not None:
            graph.replay()
        else:
            dec.step(x, y, pos)

    with torch.cuda.stream(stream):
        for _ in range(max(args.warmup, 3)):
            step_once()
        barrier()
        sampler = ClockSampler(local)
        sampler.start()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step_once()
        e1.record(stream)
        barrier()
        ms = e0.elapsed_time(e1)
        # end to end through the host-buffer entry point
        xh = x.cpu().pin_memory()
        yh = torch.empty(CFG["d_model"], dtype=torch.float16).pin_memory()
        for _ in range(3):
            dec.step_host(xh, yh, pos, stream=stream)
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            dec.step_host(xh, yh, pos, stream=stream)
        barrier()
        e2e_s = time.perf_counter() - t0
        clocks = sampler.stop()

    tmax = torch.tensor([ms, e2e_s * 1e3], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(tmax[0]), float(tmax[1])
    tok_s = args.steps / (ms * 1e-3)
    e2e_tok_s = args.steps / (e2e_ms * 1e-3)

    status = dec.device_status()
    if status != 0:
        raise RuntimeError(f"a device-side wait gave up (code {status}); the timing is void")
    ranks_agree = None
    if world > 1:
        # every rank assembled the same output vector from the shards (bit for bit), and it is finite
        dec.step(x, y, pos)
        torch.cuda.synchronize()
        ys = [torch.empty_like(y) for _ in range(world)]
        dist.all_gather(ys, y)
        ranks_agree = bool(all(torch.equal(ys[0], t) for t in ys)) and bool(torch.isfinite(y).all())
        if not ranks_agree:
            raise RuntimeError("the ranks' outputs differ or are not finite; the timing is void")
    roof = gemv_roofline(mld, torch, layers, world, peaks, layout) if rank == 0 or world > 1 else None
    if single:
        # the step is one kernel: its roofline is the step's own — every weight, scale and cached K/V
        # byte once, over the CUDA-event time of the launch
        d_, f_, blk_ = CFG["d_model"], CFG["ffn"], CFG["block"]
        per_layer = 0
        for n, kk in ((3 * d_, d_), (d_, d_), (2 * f_, d_), (d_, f_)):
            per_layer += n * kk // 2 + (kk // blk_) * n * 2
        per_layer += 2 * (pos + 1) * d_ * 2
        step_bytes = per_layer * n_layers // world     # per launch = per GPU: a rank streams its own shard
        gemv_alone = roof
        sec = ms * 1e-3 / args.steps
        roof = {"bound": "hbm", "kernel": "decode_mega_kernel (whole decode step, one launch per GPU)",
                "achieved": step_bytes / sec / 1e9, "peak": gemv_alone["peak"], "unit": "GB/s",
                "frac": step_bytes / sec / 1e9 / gemv_alone["peak"], "peak_source": gemv_alone["peak_source"],
                # dram__bytes_read + write of one launch: ncu capture of the same kernel on 2 layers
                # (296.3 + 6.2 MB against 294.9 MB algorithmic), scaled by the layer count
                "traffic": step_bytes * 1.018,
                "traffic_source": "ncu capture on 2 layers, scaled by layers (profiles/decode_mega_kernel_2_layers_ncu_full.md)",
                "launches_timed": args.steps, "avg_launch_us": sec * 1e6,
                "algorithmic_bytes_per_launch": step_bytes,
                "fc_strip_kernel_alone": {k: gemv_alone[k] for k in ("achieved", "frac", "avg_launch_us",
                                                                       "algorithmic_bytes_per_launch")}}
    side = None
    if rank == 0 and world == 1:
        dec.close()
        del layers
        torch.cuda.empty_cache()
        try:
            side = side_benchmarks(mld, torch, peaks)
        except Exception as exc:  # noqa: BLE001
            side = {"error": str(exc)}
    cpu = None
    if rank == 0 and world == 1:
        tok_cpu, cores, _ = time_cpu(2, reps=3, warm=1)
        cpu = {"value": tok_cpu, "unit": "tok/s", "cores": cores, "kind": "port",
               "sample": "2 of 32 layers per step (KV 2048), scaled x16, 3 timed steps"}
    if rank == 0:
        d, ffn = CFG["d_model"], CFG["ffn"]
        line = {
            "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"7B INT4 decode step ({n_layers}L, d{d}, 32h x128, ffn{ffn}, KV 2048, batch 1)",
                       "weights": "INT4 block-32, fp16 scales, random init ~N(0,0.02)",
                       "parallelism": (f"sharded x{world} ({'o/down by input columns, partial sums' if layout == 1 else 'all by output rows'}), "
                                       f"shard exchange: {exchange}") if world > 1 else "single GPU",
                       "l2": "inputs larger than L2 (3.6 GB of weights per step / world)",
                       "timed_with": "cuda graph replay" if graph is not None else "direct launches",
                       "decoder": "one persistent kernel per step" if single else "kernel chain"},
            "e2e": {"value": e2e_tok_s, "unit": "tok/s", "h2d_bytes_per_step": d * 2, "d2h_bytes_per_step": d * 2},
            "gpu_launches": int(launches_per_step) * args.steps,
            "launches_per_step": int(launches_per_step),
            "roofline": roof, "cpu_baseline": cpu, "clocks": clocks, "kernels": side, "ranks_agree": ranks_agree,
        }
        print(json.dumps(line), flush=True)
    # Tear down without collective destructors: every rank has printed / finished its work, and a
    # hard exit cannot hang on a peer that is already gone.
    sys.stdout.flush()
    sys.stderr.flush()
    if world > 1:
        try:
            dist.barrier()
        except Exception:  # noqa: BLE001
            pass
        os._exit(0)
    dec.close()


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
