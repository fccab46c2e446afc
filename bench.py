"""Benchmark of the quantized FullyConnected hot path.

Workload (N = 1 and every N): one decode step of a Llama-style 7B decoder with
random-init INT4 block-32 weights (32 layers, d_model 4096, 32 heads x 128,
SwiGLU FFN 11008, RMSNorm, RoPE, fp16 KV cache of 2048 tokens, batch 1) - the
configuration the headline metric "7B INT4 decode tok/s" is quoted on.  With
N > 1 every projection is split by output rows over the ranks (strong scaling:
the model is fixed) and the shard outputs are gathered on every rank.

One JSON line is printed by rank 0.  `value` is device-timed tokens/s with all
inputs resident in HBM; `e2e` is the same step through the host-buffer entry
point of the C ABI (H2D of the token's hidden vector, the step, D2H of the
result, every step); `roofline` describes the dominant kernel; `parity` is the
error of the timed decoder's output against the CPU restatement (N = 1) or
against a single-GPU decoder of the same model (N > 1); `kernels` holds the
kernel-level figures the metric also names (decode GEMV GB/s, prefill GEMM
TFLOP/s, W8A8 prefill TOP/s, weight conversion GB/s) with the CPU restatement
timed beside them; `cpu_baseline` is the CPU restatement of the step timed on
this host's cores on a bounded sample.  `--impl reference` times only that CPU
restatement.

Environment switches of this script (not of the library): MLD_SHARD_EXCHANGE =
tagged (default: one persistent kernel per rank, shards travel as tagged words
over NVLink) | barriers (the same kernel with cross-rank grid barriers) | paired
(o / down split by input columns, fp32 partial sums) | peer (kernel chain, peer
stores + flags) | nccl (kernel chain, ncclAllGather after each producer).
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
PARITY_TOL = 1e-2   # max |y - ref| / max |ref|, the bound stated for fp16 activations


def workload_name(n_layers):
    return (f"7B INT4 decode step ({n_layers}L, d{CFG['d_model']}, 32h x128, ffn{CFG['ffn']}, "
            f"KV {CFG['kv_len']}, batch 1)")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=CFG["layers"], help="for quick functional runs only")
    ap.add_argument("--no-kernels", action="store_true", help="skip the kernel-level side measurements")
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


def use_all_host_cores():
    """The CPU restatement runs on every core this process may use, whatever OMP_NUM_THREADS a launcher
    exported (torchrun sets it to 1)."""
    from oracle import oracle as orc
    orc.build()
    orc.set_num_threads(orc.host_cores())
    return orc.num_threads()


def time_cpu(n_layers, reps, warm):
    import numpy as np
    cores = use_all_host_cores()
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
    return tok_s, cores, times


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    n_layers = 2
    tok_s, cores, times = time_cpu(n_layers, reps=max(args.steps, 1), warm=max(min(args.warmup, 3), 1))
    sample = (f"each timed step runs {n_layers} of the {CFG['layers']} layers (all layers are alike: same shapes, "
              f"KV 2048); tok/s = 1 / (median step time x {CFG['layers'] // n_layers})")
    line = {
        "impl": "reference", "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / tok_s, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(CFG["layers"])},
        "arm": "CPU restatement of the reference FullyConnected arithmetic (the reference's own OpenCL CPU run is "
               "unavailable on this box)",
        "measured_ms_per_sample_step": statistics.median(times) * 1e3,
        "cpu_baseline": {"value": tok_s, "unit": "tok/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tok_s, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------- GPU arm
class ClockSampler:
    """nvidia-smi in loop mode beside the run (read-only queries, 20 ms apart).  It is started before the warm-up so
    that it is already sampling when the timed region begins; `mark()` brackets the timed region, and only the
    samples whose time stamps fall inside it count (all samples of the run when the region was too short to
    catch one, which `window` then says)."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.t0 = self.t1 = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def mark(self):
        import datetime
        now = datetime.datetime.now()
        if self.t0 is None:
            self.t0 = now
        else:
            self.t1 = now

    def stop(self):
        import datetime
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        rows = []
        for ln in out.splitlines():
            f = [c.strip() for c in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                when = datetime.datetime.strptime(f[0], "%Y/%m/%d %H:%M:%S.%f")
                rows.append((when, float(f[1]), float(f[2]), f[5:9]))
            except ValueError:
                continue
        inside = [r for r in rows if self.t0 is not None and self.t1 is not None and self.t0 <= r[0] <= self.t1]
        window = "timed region"
        if not inside:
            inside, window = rows, "whole run (no sample fell inside the timed region)"
        reasons = set()
        for r in inside:
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm, mx = [r[1] for r in inside], [r[2] for r in inside]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "window": window, "reasons": sorted(reasons)}


def build_model(mld, torch, rank, world, n_layers, dev, shard_layout=0):
    """Random-init 7B-geometry model, quantised and packed on the GPU by the library.  The model is
    defined globally (one seed per projection); a rank keeps the rows of its column shard, so every
    world size runs the same model."""
    import numpy as np
    d, ffn, blk, heads, hd = CFG["d_model"], CFG["ffn"], CFG["block"], CFG["heads"], CFG["head_dim"]
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


def parity_vs_oracle(mld, torch, layers, x, n_check=2):
    """The first n_check layers of the timed model through a fresh decoder, against the CPU restatement
    on the same packed bytes (copied back from the device).  Returns the error figures."""
    import numpy as np
    from oracle import oracle as orc
    from oracle import decode_ref
    use_all_host_cores()
    d, ffn, heads, blk = CFG["d_model"], CFG["ffn"], CFG["heads"], CFG["block"]
    pos, T = CFG["kv_len"], CFG["kv_len"] + 1
    n_check = min(n_check, len(layers))
    ref_layers, dev_layers = [], []
    for t in layers[:n_check]:
        rl = {}
        for name in ("qkv", "o", "gu", "down"):
            sc = t["s" + name].cpu().numpy()                       # [G][N] fp16, the device layout
            rl[name] = {"packed": t["w" + name].cpu().numpy(), "scale": np.ascontiguousarray(sc.T.astype(np.float32))}
        rl["norm1"] = t["norm1"].float().cpu().numpy()
        rl["norm2"] = t["norm2"].float().cpu().numpy()
        ref_layers.append(rl)
        dl = dict(t)
        dl["kcache"], dl["vcache"] = t["kcache"].clone(), t["vcache"].clone()
        dev_layers.append(dl)
    kref = np.stack([t["kcache"].float().cpu().numpy() for t in layers[:n_check]])
    vref = np.stack([t["vcache"].float().cpu().numpy() for t in layers[:n_check]])
    dec = mld.Decoder(n_check, d, heads, ffn, T, block=blk)
    for l, t in enumerate(dev_layers):
        dec.set_layer(l, **t)
    y = torch.empty_like(x)
    dec.step(x, y, pos)
    torch.cuda.synchronize()
    status = dec.device_status()
    single = dec.single_kernel
    dec.close()
    xf = x.float().cpu().numpy()
    ref = decode_ref.decode_step(xf, ref_layers, kref, vref, pos, heads, CFG["head_dim"], ffn, block=blk,
                                 interleaved_gate_up=True)
    got = y.float().cpu().numpy()
    err = float(np.max(np.abs(got - ref)) / np.max(np.abs(ref)))
    contrib = float(np.max(np.abs((got - xf) - (ref - xf))) / np.max(np.abs(ref - xf)))
    return {"against": f"CPU restatement of the step on the first {n_check} layers of the timed model "
                       f"(same packed bytes, same KV cache, position {pos})",
            "max_abs_err_over_max_abs_ref": err, "err_of_the_step_contribution_y_minus_x": contrib,
            "tolerance": PARITY_TOL, "device_status": status, "single_kernel": bool(single),
            "ok": bool(status == 0 and np.isfinite(got).all() and err < PARITY_TOL)}


def parity_vs_single_gpu(mld, torch, dev, n_layers, x, y_sharded):
    """Rank 0 builds the whole model on its own GPU (world = 1), steps it once and compares."""
    layers1 = build_model(mld, torch, 0, 1, n_layers, dev, 0)
    T = CFG["kv_len"] + 1
    dec = mld.Decoder(n_layers, CFG["d_model"], CFG["heads"], CFG["ffn"], T, block=CFG["block"])
    for l, t in enumerate(layers1):
        dec.set_layer(l, **t)
    y1 = torch.empty_like(x)
    dec.step(x, y1, CFG["kv_len"])
    torch.cuda.synchronize()
    status = dec.device_status()
    dec.close()
    del layers1
    torch.cuda.empty_cache()
    ref = y1.float()
    err = float((y_sharded.float() - ref).abs().max() / ref.abs().max())
    return {"against": f"the same {n_layers}-layer model stepped by a single-GPU decoder on rank 0",
            "max_abs_err_over_max_abs_ref": err, "tolerance": PARITY_TOL, "device_status": status,
            "ok": bool(status == 0 and bool(torch.isfinite(y_sharded).all()) and err < PARITY_TOL)}


def gemv_roofline(mld, torch, layers, world, peaks, layout=0):
    """Times the decode GEMV alone: every projection of every layer once per pass, back to back on the
    current stream, CUDA events around the passes.  The weights of a pass (3.6 GB / world) exceed L2,
    so every launch streams from HBM."""
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
            "unit": "GB/s", "frac": achieved / peak, "peak_source": src, "traffic": None,
            "traffic_source": "not measured in this run",
            "launches_timed": launches * reps, "avg_launch_us": sec / launches * 1e6,
            "algorithmic_bytes_per_launch": algo / launches}


# DRAM bytes of one step-kernel launch over the algorithmic bytes, from the ncu capture of a 2-layer run of
# this script (dram__bytes_read.sum + dram__bytes_write.sum per launch; traffic grows with the layer
# count because every layer streams its own weights and cache once).
STEP_KERNEL_TRAFFIC_RATIO = 1.018


def time_in_graph(torch, launch, n_launches, replays=7):
    """Captures n_launches calls of launch(i) in one CUDA graph and replays it: per-launch time without
    the host in the loop.  Returns (median_us, best_us) per launch, or None when capture is refused."""
    stream = torch.cuda.Stream()
    try:
        with torch.cuda.stream(stream):
            for i in range(min(n_launches, 32)):
                launch(i)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for i in range(n_launches):
                    launch(i)
            torch.cuda.synchronize()
            times = []
            for _ in range(2):
                graph.replay()
            torch.cuda.synchronize()
            for _ in range(replays):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                graph.replay()
                e1.record(stream)
                torch.cuda.synchronize()
                times.append(e0.elapsed_time(e1) * 1e3 / n_launches)
        return statistics.median(times), min(times)
    except Exception as exc:  # noqa: BLE001
        sys.stderr.write(f"[bench] CUDA graph timing unavailable ({exc})\n")
        torch.cuda.synchronize()
        return None


def cpu_best_of(fn, reps=10, warm=3, budget_s=8.0):
    for _ in range(warm):
        fn()
    best, t_start = float("inf"), time.perf_counter()
    for _ in range(reps):
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
        if time.perf_counter() - t_start > budget_s:
            break
    return best


def side_benchmarks(mld, torch, peaks):
    """The kernel-level figures the metric also names, each kernel timed alone with CUDA events, with
    the CPU restatement of the same operation timed on the host's cores beside it."""
    import numpy as np
    from oracle import oracle as orc
    cores = use_all_host_cores()
    out = {"cpu_cores": cores}
    hbm = peaks.get("hbm_gbs") or 6650.0
    blk = 32
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    # ---- decode GEMV, INT4 block 32: N=16384, K=2048, one token; 16 weight sets (303 MB) rotate to defeat L2
    N, K, sets = 16384, 2048, 16
    plan = mld.FullyConnectedPlan(N, K, 4, scale_mode=mld.SCALE_BLOCK, groups=K // blk, precision=mld.F32F16)
    nbytes = mld.packed_size_bytes(N, K, 4)
    ws = [torch.randint(0, 256, (nbytes,), dtype=torch.uint8, device="cuda") for _ in range(sets)]
    ss = [(torch.rand((K // blk, N), device="cuda") * 0.01).half() for _ in range(sets)]
    x = torch.randn(K, device="cuda").half()
    y = torch.empty(N, dtype=torch.float16, device="cuda")
    for i in range(2 * sets):
        plan.run(x, ws[i % sets], ss[i % sets], y, 1)
    torch.cuda.synchronize()
    iters = 20 * sets
    e0.record()
    for i in range(iters):
        plan.run(x, ws[i % sets], ss[i % sets], y, 1)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / iters
    algo = nbytes + (K // blk) * N * 2 + K * 2 + N * 2
    entry = {"workload": "INT4 block-32 GEMV N=16384 K=2048, 1 token, 16 rotating weight sets (303 MB > L2)",
             "algorithmic_bytes": algo,
             "launched_from_the_host": {"us_per_launch": us, "GBps": algo / us / 1e3, "frac_of_hbm_peak": algo / us / 1e3 / hbm,
                                        "timed_with": "320 launches back to back on one stream, CUDA events"}}
    g_dep = time_in_graph(torch, lambda i: plan.run(x, ws[i % sets], ss[i % sets], y, 1), 256)
    plan.close()
    # The launches of this benchmark do not depend on one another (each reads the same x and writes one of four
    # rotating outputs), as the q / k / v or gate / up projections of one input do not: the plan says so
    # (independent_io) and consecutive launches overlap completely.  That is the headline of this entry; the
    # same launches through a plan that assumes each consumes what the one before it wrote (a chain of
    # decoder ops: hand-over at the activation load) are reported beside it.
    plan = mld.FullyConnectedPlan(N, K, 4, scale_mode=mld.SCALE_BLOCK, groups=K // blk, precision=mld.F32F16,
                                  independent_io=True)
    ys = [torch.empty(N, dtype=torch.float16, device="cuda") for _ in range(4)]
    g = time_in_graph(torch, lambda i: plan.run(x, ws[i % sets], ss[i % sets], ys[i % 4], 1), 256)
    plan.close()
    if g is not None:
        entry.update({"us_per_launch": g[0], "best_us_per_launch": g[1], "GBps": algo / g[0] / 1e3,
                      "frac_of_hbm_peak": algo / g[0] / 1e3 / hbm, "frac_of_hbm_peak_best": algo / g[1] / 1e3 / hbm,
                      "timed_with": "256 launches per replay of one CUDA graph, median of 7 replays, CUDA events; "
                                    "independent launches (plan flag independent_io)"})
    else:
        entry.update({"us_per_launch": us, "GBps": algo / us / 1e3, "frac_of_hbm_peak": algo / us / 1e3 / hbm,
                      "timed_with": "320 launches back to back on one stream, CUDA events"})
    if g_dep is not None:
        entry["in_cuda_graph_as_a_dependent_chain"] = {
            "launches_per_replay": 256, "median_us_per_launch": g_dep[0], "best_us_per_launch": g_dep[1],
            "GBps_median": algo / g_dep[0] / 1e3, "frac_of_hbm_peak_median": algo / g_dep[0] / 1e3 / hbm,
            "frac_of_hbm_peak_best": algo / g_dep[1] / 1e3 / hbm,
            "note": "every launch waits for the one before it to finish before it reads its activations"}
    # CPU restatement of the same GEMV (OpenMP over output slices), one of the sets copied back
    wh, sh = ws[0].cpu().numpy(), np.ascontiguousarray(ss[0].float().cpu().numpy())
    xh = x.float().cpu().numpy()
    t_cpu = cpu_best_of(lambda: orc.gemv_f32_fast(4, xh, wh, N, sh))
    entry["cpu"] = {"us": t_cpu * 1e6, "GBps": algo / t_cpu / 1e9, "cores": cores, "kind": "port"}
    out["fc_gemv_int4"] = entry
    del ws, ss

    # ---- the W8 per-output-channel case: N=2048, K=2048, fp32 activations, bias (runs on the CPU baseline;
    # on the GPU for completeness: it is L2-resident after the first launch, which the entry says)
    N1 = K1 = 2048
    rng = np.random.default_rng(0)
    w1 = (rng.standard_normal((N1, K1)) * 0.02).astype(np.float32)
    x1 = rng.standard_normal((1, K1)).astype(np.float32)
    b1 = (rng.standard_normal(N1) * 0.01).astype(np.float32)
    q1, s1 = orc.quantize_int8_sym(w1)
    p1 = orc.rearrange_int8_as_uint8(q1)
    algo1 = N1 * K1 + N1 * 4 * 2 + K1 * 4 + N1 * 4
    s1gn = np.ascontiguousarray(orc.scale_layout(s1, False))
    t_cpu = cpu_best_of(lambda: orc.gemv_f32_fast(8, x1[0], p1, N1, s1gn, bias=b1))
    plan = mld.FullyConnectedPlan(N1, K1, 8, scale_mode=mld.SCALE_PER_CHANNEL, has_bias=True, precision=mld.F32)
    dw, dsc = torch.from_numpy(p1).cuda(), torch.from_numpy(s1gn).cuda()
    dx, db = torch.from_numpy(x1[0]).cuda(), torch.from_numpy(b1).cuda()
    dy = torch.empty(N1, dtype=torch.float32, device="cuda")
    for _ in range(5):
        plan.run(dx, dw, dsc, dy, 1, bias=db)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(100):
        plan.run(dx, dw, dsc, dy, 1, bias=db)
    e1.record()
    torch.cuda.synchronize()
    us1 = e0.elapsed_time(e1) * 1e3 / 100
    g1 = time_in_graph(torch, lambda i: plan.run(dx, dw, dsc, dy, 1, bias=db), 256)
    plan.close()
    gpu1 = {"us_per_launch": us1, "GBps": algo1 / us1 / 1e3, "timed_with": "100 launches from the host, CUDA events",
            "note": "4 MB of weights stay in L2 between launches: not an HBM figure"}
    if g1 is not None:
        gpu1["in_cuda_graph"] = {"launches_per_replay": 256, "median_us_per_launch": g1[0], "best_us_per_launch": g1[1]}
    out["fc_gemv_int8_f32"] = {"workload": "INT8 per-channel GEMV N=2048 K=2048, fp32 activations + bias, seed 0",
                               "algorithmic_bytes": algo1,
                               "cpu": {"us": t_cpu * 1e6, "GBps": algo1 / t_cpu / 1e9, "cores": cores, "kind": "port"},
                               "gpu": gpu1}

    # ---- weight conversion: quantise + pack a 16384 x 2048 matrix (GPU kernels) next to the CPU restatement
    # (quantiser on all cores; the rearrangement is the reference's single-threaded loop order)
    gen = torch.Generator(device="cuda").manual_seed(0)
    w = torch.randn((N, K), generator=gen, device="cuda") * 0.02
    q, s = mld.quantize_weights(w, 4, blk)
    packed, _ = mld.pack_weights(q, (N, 1, 1, K), 4)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(10):
        q, s = mld.quantize_weights(w, 4, blk)
    e1.record()
    torch.cuda.synchronize()
    us_q = e0.elapsed_time(e1) * 1e3 / 10
    e0.record()
    for _ in range(10):
        packed, _ = mld.pack_weights(q, (N, 1, 1, K), 4)
    e1.record()
    torch.cuda.synchronize()
    us_p = e0.elapsed_time(e1) * 1e3 / 10
    wh32 = w.cpu().numpy()
    t_q = cpu_best_of(lambda: orc.quantize_int4_sym(wh32, blk), reps=5, warm=1)
    qh = q.cpu().numpy()
    t_p = cpu_best_of(lambda: orc.rearrange_int8_as_uint4(qh), reps=5, warm=1)
    bytes_q = N * K * 5 + (K // blk) * N * 4          # fp32 read, int8 + scales written
    bytes_p = N * K + N * K // 2                       # int8 read, nibbles written
    out["weight_conversion_int4"] = {
        "workload": "16384 x 2048 fp32 -> INT4 block 32: quantise, then rearrange into the packed layout",
        "quantize": {"gpu_us": us_q, "gpu_GBps": bytes_q / us_q / 1e3, "cpu_us": t_q * 1e6,
                     "cpu_GBps": bytes_q / t_q / 1e9, "cpu_cores": cores},
        "pack": {"gpu_us": us_p, "gpu_GBps": bytes_p / us_p / 1e3, "cpu_us": t_p * 1e6,
                 "cpu_GBps": bytes_p / t_p / 1e9, "cpu_cores": 1}}
    del w, q, s, packed

    # ---- prefill GEMM, INT4 block 32: M=1024, K=4096, N=14336, fp16 in, fp32 accumulate, fp16 out
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
    # the three ways the operator serves a prefill call: the weights dequantised inside the GEMM (route 1),
    # a conversion pass before a plain GEMM on every call (route 0: what the conversion-cost rule picks at
    # this M), and the converted copy kept between calls
    ROUTES = (("dequantised_inside_gemm", 1, False), ("with_weight_conversion", 0, False),
              ("weights_prepared_once", 0, True))
    for label, route, cache in ROUTES:
        plan = mld.FullyConnectedPlan(N, K, 4, scale_mode=mld.SCALE_BLOCK, groups=K // blk, precision=mld.F32F16,
                                      max_tokens=M, force_path=mld.PATH_GEMM, cache_prepared_weights=cache,
                                      prefill_route=route)
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
    # CPU restatement on a sample of the tokens (the work is linear in M)
    m_cpu = 16
    xrow = np.ascontiguousarray(xs.permute(1, 0, 2).reshape(M, K)[:m_cpu].cpu().numpy()).view(np.uint16)
    ph, sch = packed.cpu().numpy(), np.ascontiguousarray(sc.cpu().numpy()).view(np.uint16)
    t_cpu = cpu_best_of(lambda: orc.prefill_gemm_int4(xrow, ph, sch, N), reps=3, warm=1)
    out["prefill_gemm_int4"] = {"workload": "INT4 block-32 GEMM M=1024 K=4096 N=14336, fp16 in, fp32 accumulate", **res,
                                "frac_of_bf16_burst_peak": res["weights_prepared_once"]["TFLOPs"] / pk,
                                "frac_with_conversion": res["with_weight_conversion"]["TFLOPs"] / pk, "peak_TFLOPs": pk,
                                "cpu": {"TFLOPs": 2.0 * m_cpu * K * N / t_cpu / 1e12, "cores": cores, "kind": "port",
                                        "sample": f"{m_cpu} of {M} tokens"}}
    del packed, sc, xs, yy

    # ---- W8A8 prefill, one rank's shard of the 8-way split: M=2048, K=8192, N=3584 (of 28672)
    M, K, N = 2048, 8192, 3584
    w = torch.randn((N, K), generator=g, device="cuda") * 0.02
    q, s = mld.quantize_weights(w, 8)
    packed, w_sum = mld.pack_weights(q, (N, 1, 1, K), 8, want_sum=True)
    sc = mld.pack_scales(s, True)
    del w, q, s
    xs = torch.randn((K // 4, M, 4), generator=g, device="cuda").half()
    yy = torch.empty((N // 4, M, 4), dtype=torch.float16, device="cuda")
    ops = 2.0 * M * K * N
    res = {}
    for label, route, cache in ROUTES:
        plan = mld.FullyConnectedPlan(N, K, 8, scale_mode=mld.SCALE_PER_CHANNEL, precision=mld.F32F16, max_tokens=M,
                                      force_path=mld.PATH_GEMM, prefill_act_quant=2, cache_prepared_weights=cache,
                                      prefill_route=route)
        plan.set_weights_sum(w_sum)
        for _ in range(3):
            plan.run(xs, packed, sc, yy, M)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(20):
            plan.run(xs, packed, sc, yy, M)
        e1.record()
        torch.cuda.synchronize()
        us = e0.elapsed_time(e1) * 1e3 / 20
        res[label] = {"us": us, "TOPs": ops / us / 1e6}
        plan.close()
    out["prefill_gemm_w8a8_shard"] = {
        "workload": "W8A8 GEMM M=2048 K=8192 N=3584 (one rank's eighth of N=28672): asymmetric per-token int8 "
                    "activations (quantised inside the call), int32 accumulate, fp16 out", **res,
        "nominal_int8_dense_peak_TOPs": 4500.0,
        "frac_of_nominal_int8_peak": res["weights_prepared_once"]["TOPs"] / 4500.0,
        "vs_measured_bf16_burst_TFLOPs": res["weights_prepared_once"]["TOPs"] / pk}
    return out


def sharded_prefill_benchmark(mld, torch, dist, rank, world, dev, nccl_id):
    """The W8A8 prefill case split over the ranks by output rows: M=2048, K=8192, N=28672 (N / world rows
    per rank), asymmetric per-token int8 activations, gather of Y on every rank.  Reports the GEMM alone,
    GEMM + ncclAllGather, and the GEMM whose epilogue stores into every rank's tensor (max over ranks)."""
    M, K, N = 2048, 8192, 28672
    n = N // world

    def all_ok(flag):   # the ranks agree on whether to go on, so that no rank enters a collective alone
        t = torch.tensor([1 if flag else 0], dtype=torch.int32, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return bool(t[0])

    failure = None
    try:
        g = torch.Generator(device=dev).manual_seed(100 + rank)
        w = torch.randn((n, K), generator=g, device=dev) * 0.02
        q, s = mld.quantize_weights(w, 8)
        packed, w_sum = mld.pack_weights(q, (n, 1, 1, K), 8, want_sum=True)
        sc = mld.pack_scales(s, True)
        del w, q, s
        gx = torch.Generator(device=dev).manual_seed(99)
        xs = (torch.randn((K // 4, M, 4), generator=gx, device=dev) + 0.2).half()
        plan = mld.FullyConnectedPlan(n, K, 8, scale_mode=mld.SCALE_PER_CHANNEL, precision=mld.F32F16, max_tokens=M,
                                      force_path=mld.PATH_GEMM, prefill_act_quant=2)
        plan.set_weights_sum(w_sum)
        y_local = torch.empty((n // 4, M, 4), dtype=torch.float16, device=dev)
    except Exception as exc:  # noqa: BLE001
        failure = f"{type(exc).__name__}: {exc}"
    if not all_ok(failure is None):
        return {"error": failure or "another rank failed to set up"}
    group = mld.ShardGroup(rank, world, N * M * 2, nccl_id=nccl_id)      # collective (NCCL communicator)
    mine = torch.frombuffer(bytearray(group.ipc_export()), dtype=torch.uint8).to(dev)
    table = [torch.zeros(64, dtype=torch.uint8, device=dev) for _ in range(world)]
    dist.all_gather(table, mine)
    try:
        group.ipc_import(b"".join(t.cpu().numpy().tobytes() for t in table))
    except Exception as exc:  # noqa: BLE001
        failure = f"{type(exc).__name__}: {exc}"
    if not all_ok(failure is None):
        return {"error": failure or "another rank failed to import the exchange blocks"}
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def timed(fn, iters=10):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / iters], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])

    us_gemm = timed(lambda: plan.run(xs, packed, sc, y_local, M))
    us_nccl = timed(lambda: group.run(plan, xs, packed, sc, M, mld.GATHER_NCCL))
    y_nccl = group.output(N * M, dev).clone()
    us_peer = timed(lambda: group.run(plan, xs, packed, sc, M, mld.GATHER_PEER_STORES))
    y_peer = group.output(N * M, dev)
    status = group.device_status()
    same = bool(torch.equal(y_nccl, y_peer)) and status == 0
    own = y_peer.view(N // 4, M, 4)[rank * (n // 4):(rank + 1) * (n // 4)]
    own_ok = bool(torch.equal(own, y_local))
    ops = 2.0 * M * K * N
    plan.close()
    return {"workload": f"W8A8 GEMM M={M} K={K} N={N} split {world} ways by output rows ({n} per rank), asymmetric "
                        "per-token int8 activations, Y gathered on every rank (fp16, 117 MB)",
            "gemm_only_us": us_gemm, "gemm_plus_nccl_allgather_us": us_nccl, "gemm_storing_into_every_rank_us": us_peer,
            "whole_job_TOPs_nccl": ops / us_nccl / 1e6, "whole_job_TOPs_peer_stores": ops / us_peer / 1e6,
            "gather_bytes_per_rank_out": (world - 1) * n * M * 2,
            "peer_stores_equal_nccl": same, "own_block_equals_unsharded_kernel_output": own_ok,
            "timing": "10 runs after 3 warm-ups, CUDA events, max over ranks"}


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
    exchange = os.environ.get("MLD_SHARD_EXCHANGE", "tagged") if world > 1 else "none"
    assert exchange in ("none", "tagged", "barriers", "paired", "peer", "nccl")
    single_kernel = exchange in ("none", "tagged", "barriers", "paired")
    layout = 1 if exchange == "paired" else 0
    if world > 1:
        import torch.distributed as dist
        import datetime
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(minutes=10))
        ids = torch.zeros(2, 128, dtype=torch.uint8, device=dev)   # one for the decoder, one for the operator group
        if rank == 0:
            for i in range(2):
                ids[i].copy_(torch.frombuffer(bytearray(mld.comm_unique_id()), dtype=torch.uint8))
        dist.broadcast(ids, 0)
        if exchange == "nccl":
            nccl_id = bytes(ids[0].cpu().numpy().tobytes())
        group_id = bytes(ids[1].cpu().numpy().tobytes())

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
    layers = build_model(mld, torch, rank, world, n_layers, dev, layout)
    T = CFG["kv_len"] + 1
    mode = mld.DECODER_AUTO if world == 1 else (mld.DECODER_SINGLE_KERNEL if single_kernel else mld.DECODER_OP_CHAIN)
    dec = mld.Decoder(n_layers, CFG["d_model"], CFG["heads"], CFG["ffn"], T, block=CFG["block"], rank=rank,
                      world=world, nccl_id=nccl_id, shard_layout=layout, mode=mode,
                      handover=mld.HANDOVER_BARRIERS if exchange == "barriers" else mld.HANDOVER_TAGGED)
    for l, t in enumerate(layers):
        dec.set_layer(l, **t)
    if world > 1 and exchange != "nccl":
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
        sampler = ClockSampler(local)
        sampler.start()
        for _ in range(max(args.warmup, 3)):
            step_once()
        barrier()
        sampler.mark()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step_once()
        e1.record(stream)
        barrier()
        sampler.mark()
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
    parity = None
    sharded_side = None
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
        # the step is one kernel: its roofline is the step's own - every weight, scale and cached K/V
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
                "traffic": step_bytes * STEP_KERNEL_TRAFFIC_RATIO if world == 1 else None,
                "traffic_source": ("ncu capture of a 2-layer single-GPU run (dram bytes read + written per launch), "
                                   "scaled by the layer count; not measured in this run") if world == 1
                else "not measured in this run",
                "launches_timed": args.steps, "avg_launch_us": sec * 1e6,
                "algorithmic_bytes_per_launch": step_bytes,
                "fc_strip_kernel_alone": {k: gemv_alone[k] for k in ("achieved", "frac", "avg_launch_us",
                                                                       "algorithmic_bytes_per_launch")}}
    if world == 1:
        parity = parity_vs_oracle(mld, torch, layers, x)
        dec.close()
        del layers
        torch.cuda.empty_cache()
    else:
        # (the sharded decoder stays open until the process exits: tearing a communicator down is a
        # collective matter, and the other ranks are waiting at the barrier below)
        if rank == 0:
            parity = parity_vs_single_gpu(mld, torch, dev, n_layers, x, y)
        barrier()
        if not args.no_kernels:
            del layers
            torch.cuda.empty_cache()
            try:
                sharded_side = sharded_prefill_benchmark(mld, torch, dist, rank, world, dev, group_id)
            except Exception as exc:  # noqa: BLE001
                sharded_side = {"error": f"{type(exc).__name__}: {exc}"}
    if parity is not None and not parity["ok"]:
        raise RuntimeError(f"parity check failed: {parity}")
    side = None if world == 1 else ({"prefill_gemm_w8a8_sharded": sharded_side} if sharded_side is not None else None)
    cpu = None
    if rank == 0 and world == 1:
        if not args.no_kernels:
            try:
                side = side_benchmarks(mld, torch, peaks)
            except Exception as exc:  # noqa: BLE001
                side = {"error": f"{type(exc).__name__}: {exc}"}
        tok_cpu, cores, _ = time_cpu(2, reps=3, warm=1)
        cpu = {"value": tok_cpu, "unit": "tok/s", "cores": cores, "kind": "port",
               "sample": "each timed step runs 2 of the 32 layers (all layers alike, KV 2048); "
                         "tok/s = 1 / (median of 3 step times x 16)"}
    if rank == 0:
        d, ffn = CFG["d_model"], CFG["ffn"]
        par = {"none": "single GPU",
               "tagged": f"sharded x{world}, every projection split by output rows; one persistent kernel per rank, "
                         "shard outputs stored into every rank's memory as self-validating words (no collective call)",
               "barriers": f"sharded x{world}, every projection split by output rows; one persistent kernel per rank, "
                           "peer stores + cross-rank grid barriers",
               "paired": f"sharded x{world}, o/down split by input columns (fp32 partial sums), cross-rank barriers",
               "peer": f"sharded x{world} by output rows, kernel chain, peer stores + completion flags",
               "nccl": f"sharded x{world} by output rows, kernel chain, ncclAllGather after each producer"}[exchange]
        line = {
            "metric": METRIC, "value": tok_s, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": workload_name(n_layers),
                       "weights": "INT4 block-32, fp16 scales, random init ~N(0,0.02)",
                       "parallelism": par,
                       "l2": "inputs larger than L2 (3.6 GB of weights per step / world)",
                       "timed_with": "cuda graph replay" if graph is not None else "direct launches",
                       "decoder": "one persistent kernel per step" if single else "kernel chain"},
            "e2e": {"value": e2e_tok_s, "unit": "tok/s", "h2d_bytes_per_step": d * 2, "d2h_bytes_per_step": d * 2},
            "gpu_launches": int(launches_per_step) * args.steps,
            "launches_per_step": int(launches_per_step),
            "roofline": roof, "cpu_baseline": cpu, "clocks": clocks, "parity": parity, "kernels": side,
            "ranks_agree": ranks_agree,
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


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
