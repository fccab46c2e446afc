"""One decode step through the C ABI vs the CPU restatement, on a small decoder
of the same structure as the 7B benchmark model."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mld():
    import __graft_entry__ as g
    return g.import_package()


def _dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).cuda()
    return t if dtype is None else t.to(dtype)


def build_small_decoder(mld, oracle, rng, L, heads, ffn, T, pos, world=1, rank=0, block=32):
    d = heads * 128
    layers_ref, dec_tensors = [], []
    for _ in range(L):
        layer = {}
        dev = {}
        for name, N, K in (("qkv", 3 * d, d), ("o", d, d), ("gu", 2 * ffn, d), ("down", d, ffn)):
            w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
            q, s = oracle.quantize_int4_sym(w, block)
            layer[name] = {"packed": oracle.rearrange_int8_as_uint4(q), "scale": s}
            if name == "gu":   # the device matrix interleaves gate_i, up_i rows for the fused SiLU*mul write
                order = mld.sharding.gate_up_shard_rows(ffn, 0, 1)
                q, s = q[order], s[order]
            dev["w" + name] = _dev(oracle.rearrange_int8_as_uint4(q))
            dev["s" + name] = _dev(oracle.scale_layout(s, True).view(np.float16))
        for n in ("norm1", "norm2"):
            g = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float16)
            layer[n] = g.astype(np.float32)
            dev[n] = _dev(g)
        layers_ref.append(layer)
        dec_tensors.append(dev)
    kc = rng.standard_normal((L, T, d)).astype(np.float16)
    vc = rng.standard_normal((L, T, d)).astype(np.float16)
    return layers_ref, dec_tensors, kc, vc


MODES = {"ops": 1, "mega": 2}   # mld_decoder_mode: op chain / single kernel


def _make(mld, mode, L, d, heads, ffn, T, block, dec_tensors, kcd, vcd, **tuning):
    """mode: "ops" (chain of kernels), "mega" (single kernel, tagged hand-over) or "mega_barriers"."""
    if mode == "mega_barriers":
        tuning = dict(tuning, handover=mld.HANDOVER_BARRIERS)
    dec = mld.Decoder(L, d, heads, ffn, T, block=block, mode=MODES[mode.split("_")[0]], **tuning)
    assert dec.single_kernel == mode.startswith("mega")
    for l in range(L):
        t = dec_tensors[l]
        dec.set_layer(l, wqkv=t["wqkv"], sqkv=t["sqkv"], wo=t["wo"], so=t["so"], wgu=t["wgu"], sgu=t["sgu"],
                      wdown=t["wdown"], sdown=t["sdown"], norm1=t["norm1"], norm2=t["norm2"],
                      kcache=kcd[l], vcache=vcd[l])
    return dec


# "ops": a chain of FullyConnected / attention kernels; "mega": the whole step as one persistent kernel.
# Shapes cover a ragged last k-stage (ffn 1408 -> 352 k-slices), one- and many-tile attention, the first
# position, tile boundaries, and coarser scale blocks.
@pytest.mark.parametrize("mode,L,heads,ffn,T,pos,block", [
    ("ops", 2, 2, 384, 96, 70, 32),
    ("mega", 2, 2, 384, 96, 70, 32),
    ("mega_barriers", 2, 2, 384, 96, 70, 32),
    ("mega_barriers", 3, 4, 1408, 200, 31, 32),
    ("mega", 3, 4, 1408, 200, 0, 32),
    ("mega", 3, 4, 1408, 200, 31, 32),
    ("mega", 2, 4, 1408, 200, 32, 32),
    ("mega", 2, 4, 1408, 200, 199, 32),
    ("mega", 1, 8, 2816, 1100, 1030, 32),
    ("mega", 2, 2, 512, 96, 64, 128),
    ("mega", 2, 2, 256, 96, 65, 256),
])
def test_decode_step_matches_oracle(mld, oracle, mode, L, heads, ffn, T, pos, block):
    from oracle import decode_ref
    rng = np.random.default_rng(0)
    d = heads * 128
    layers_ref, dec_tensors, kc, vc = build_small_decoder(mld, oracle, rng, L, heads, ffn, T, pos, block=block)
    x = rng.standard_normal(d).astype(np.float16)
    kcd, vcd = _dev(kc), _dev(vc)
    dec = _make(mld, mode, L, d, heads, ffn, T, block, dec_tensors, kcd, vcd)
    xd = _dev(x)
    y = torch.empty(d, dtype=torch.float16, device="cuda")
    dec.step(xd, y, pos)
    torch.cuda.synchronize()
    assert dec.device_status() == 0
    kref, vref = kc.astype(np.float32), vc.astype(np.float32)
    ref = decode_ref.decode_step(x.astype(np.float32), layers_ref, kref, vref, pos, heads, 128, ffn, block=block)
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) < 1e-2
    # the new token's K/V rows were written to the cache
    assert np.max(np.abs(kcd[:, pos].float().cpu().numpy() - kref[:, pos])) < 2e-2
    assert np.max(np.abs(vcd[:, pos].float().cpu().numpy() - vref[:, pos])) < 2e-2
    # a second step at the next position is reproducible
    if pos + 1 < T:
        y2 = torch.empty_like(y)
        dec.step(xd, y2, pos + 1)
        y3 = torch.empty_like(y)
        dec.step(xd, y3, pos + 1)
        torch.cuda.synchronize()
        assert dec.device_status() == 0
        assert torch.equal(y2, y3)
    dec.close()


# Small grids reach the work splits a full B200 grid does not: fewer CTAs than heads (heads shared out
# item by item, several heads per CTA, ticketed merge), a handful of CTAs per head, one CTA for everything;
# and the last row of the cache (its tile is cut off by the end of the tensor).
@pytest.mark.parametrize("grid,heads,ffn,T,pos", [
    (3, 4, 512, 200, 130),
    (2, 2, 256, 96, 95),
    (8, 2, 384, 160, 159),
    (37, 4, 1408, 300, 299),
])
def test_single_kernel_step_on_small_grids(mld, oracle, grid, heads, ffn, T, pos):
    from oracle import decode_ref
    rng = np.random.default_rng(grid)
    L, d = 2, heads * 128
    layers_ref, dec_tensors, kc, vc = build_small_decoder(mld, oracle, rng, L, heads, ffn, T, pos)
    x = rng.standard_normal(d).astype(np.float16)
    kcd, vcd = _dev(kc), _dev(vc)
    dec = _make(mld, "mega", L, d, heads, ffn, T, 32, dec_tensors, kcd, vcd, grid_limit=grid)
    y = torch.empty(d, dtype=torch.float16, device="cuda")
    dec.step(_dev(x), y, pos)
    torch.cuda.synchronize()
    assert dec.device_status() == 0
    kref, vref = kc.astype(np.float32), vc.astype(np.float32)
    ref = decode_ref.decode_step(x.astype(np.float32), layers_ref, kref, vref, pos, heads, 128, ffn)
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) < 1e-2
    assert np.max(np.abs(kcd[:, pos].float().cpu().numpy() - kref[:, pos])) < 2e-2
    dec.close()


@pytest.mark.parametrize("stages", [12, 16, 20])
def test_single_kernel_step_with_a_short_ring(mld, oracle, stages):
    """Rings shorter than two stages per consumer warp (large vectors leave that little shared memory)
    put fewer warps on attention and must give the same step; the step is run several times so that
    consecutive launches, whose vectors carry different tags, are covered too."""
    from oracle import decode_ref
    rng = np.random.default_rng(stages)
    L, heads, ffn, T, pos = 2, 4, 1408, 1024, 1000
    d = heads * 128
    layers_ref, dec_tensors, kc, vc = build_small_decoder(mld, oracle, rng, L, heads, ffn, T, pos)
    x = rng.standard_normal(d).astype(np.float16)
    kcd, vcd = _dev(kc), _dev(vc)
    dec = _make(mld, "mega", L, d, heads, ffn, T, 32, dec_tensors, kcd, vcd, ring_stages=stages)
    y = torch.empty(d, dtype=torch.float16, device="cuda")
    xd = _dev(x)
    outs = []
    for _ in range(3):
        dec.step(xd, y, pos)
        torch.cuda.synchronize()
        assert dec.device_status() == 0
        outs.append(y.float().cpu().numpy().copy())
    kref, vref = kc.astype(np.float32), vc.astype(np.float32)
    ref = decode_ref.decode_step(x.astype(np.float32), layers_ref, kref, vref, pos, heads, 128, ffn)
    for got in outs:
        assert np.isfinite(got).all()
        assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) < 1e-2
    assert np.array_equal(outs[0], outs[1]) and np.array_equal(outs[1], outs[2])
    dec.close()


def test_single_kernel_step_ignores_uninitialised_cache_rows(mld, oracle):
    """Rows of the cache past the current position may hold anything (NaN included): they must not reach
    the result."""
    from oracle import decode_ref
    rng = np.random.default_rng(11)
    L, heads, ffn, T, pos = 1, 2, 256, 128, 37
    d = heads * 128
    layers_ref, dec_tensors, kc, vc = build_small_decoder(mld, oracle, rng, L, heads, ffn, T, pos)
    x = rng.standard_normal(d).astype(np.float16)
    kbad, vbad = kc.copy(), vc.copy()
    kbad[:, pos + 1:] = np.nan
    vbad[:, pos + 1:] = np.nan
    kcd, vcd = _dev(kbad), _dev(vbad)
    dec = _make(mld, "mega", L, d, heads, ffn, T, 32, dec_tensors, kcd, vcd)
    y = torch.empty(d, dtype=torch.float16, device="cuda")
    dec.step(_dev(x), y, pos)
    torch.cuda.synchronize()
    assert dec.device_status() == 0
    ref = decode_ref.decode_step(x.astype(np.float32), layers_ref, kc.astype(np.float32), vc.astype(np.float32),
                                 pos, heads, 128, ffn)
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all()
    assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) < 1e-2
    dec.close()


def test_single_kernel_step_agrees_with_op_chain(mld, oracle):
    """Both decoders on the same model and cache: same result within fp16 rounding of the partial sums'
    different order, same cache rows."""
    rng = np.random.default_rng(3)
    L, heads, ffn, T, pos = 4, 4, 1024, 300, 257
    d = heads * 128
    _, dec_tensors, kc, vc = build_small_decoder(mld, oracle, rng, L, heads, ffn, T, pos)
    xd = _dev(rng.standard_normal(d).astype(np.float16))
    outs, caches = [], []
    for mode in ("ops", "mega"):
        kcd, vcd = _dev(kc), _dev(vc)
        dec = _make(mld, mode, L, d, heads, ffn, T, 32, dec_tensors, kcd, vcd)
        y = torch.empty(d, dtype=torch.float16, device="cuda")
        for p in (pos, pos + 1, pos + 2):        # three consecutive steps share the cache
            dec.step(xd, y, p)
        torch.cuda.synchronize()
        assert dec.device_status() == 0
        outs.append(y.float())
        caches.append((kcd[:, pos:pos + 3].float(), vcd[:, pos:pos + 3].float()))
        dec.close()
    scale = outs[0].abs().max().item()
    assert (outs[0] - outs[1]).abs().max().item() / scale < 1e-2
    assert (caches[0][0] - caches[1][0]).abs().max().item() < 2e-2
    assert (caches[0][1] - caches[1][1]).abs().max().item() < 2e-2


# ------------------------------------------------------------------ the benchmark's own geometry
# Two layers at the full width of the 7B decoder the headline number is measured on (d_model 4096, 32
# heads, FFN 11008, 2048 cached tokens, position 2048): the shapes take paths no smaller decoder
# reaches (an input vector that exactly fills the register path of the vector load, four CTAs per
# head with idle CTAs left over, eleven boxes per strip of the down projection).
WIDE = dict(L=2, heads=32, ffn=11008, T=2049, pos=2048)


@pytest.fixture(scope="module")
def wide_model(mld, oracle):
    rng = np.random.default_rng(42)
    L, heads, ffn, T = WIDE["L"], WIDE["heads"], WIDE["ffn"], WIDE["T"]
    d = heads * 128
    layers_ref, dec_tensors = [], []
    for _ in range(L):
        layer, dev = {}, {}
        for name, N, K in (("qkv", 3 * d, d), ("o", d, d), ("gu", 2 * ffn, d), ("down", d, ffn)):
            w = rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)
            q, sc = oracle.quantize_int4_sym(w, 32)
            del w
            layer[name] = {"packed": oracle.rearrange_int8_as_uint4(q), "scale": sc}
            if name == "gu":
                order = mld.sharding.gate_up_shard_rows(ffn, 0, 1)
                q, sc = q[order], sc[order]
                dev["w" + name] = _dev(oracle.rearrange_int8_as_uint4(q))
            else:
                dev["w" + name] = _dev(layer[name]["packed"])
            dev["s" + name] = _dev(oracle.scale_layout(sc, True).view(np.float16))
            del q
        layers_ref.append(layer)
        dec_tensors.append(dev)
    kc = rng.standard_normal((L, T, d), dtype=np.float32).astype(np.float16)
    vc = rng.standard_normal((L, T, d), dtype=np.float32).astype(np.float16)
    return layers_ref, dec_tensors, kc, vc


def _wide_inputs(case):
    """x and the two RMSNorm weight vectors.  "outliers": three channels of x at 300 sigma and one
    channel of each gamma at 50 times the rest - what the hidden states of real language models look
    like, and what a coarse fixed-point input format would not survive."""
    rng = np.random.default_rng(7)
    d = WIDE["heads"] * 128
    x = rng.standard_normal(d).astype(np.float32)
    g1 = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    g2 = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32)
    if case == "outliers":
        x[[5, 1777, 4000]] = [300.0, -300.0, 300.0]
        g1[1234] = 50.0
        g2[77] = 50.0
    return x.astype(np.float16), g1.astype(np.float16), g2.astype(np.float16)


def _fp16_ulp(v):
    v = np.maximum(np.abs(v).astype(np.float32), 2.0 ** -14)
    return 2.0 ** (np.floor(np.log2(v)) - 10)


@pytest.mark.parametrize("mode,case", [("mega", "gaussian"), ("mega", "outliers"), ("mega_barriers", "gaussian"),
                                       ("ops", "gaussian"), ("ops", "outliers")])
def test_full_width_step_matches_oracle(mld, oracle, wide_model, mode, case):
    from oracle import decode_ref
    layers_ref, dec_tensors, kc, vc = wide_model
    L, heads, ffn, T, pos = (WIDE[k] for k in ("L", "heads", "ffn", "T", "pos"))
    d = heads * 128
    x, g1, g2 = _wide_inputs(case)
    for l in range(L):
        layers_ref[l]["norm1"], layers_ref[l]["norm2"] = g1.astype(np.float32), g2.astype(np.float32)
        dec_tensors[l]["norm1"], dec_tensors[l]["norm2"] = _dev(g1), _dev(g2)
    kcd, vcd = _dev(kc), _dev(vc)
    dec = _make(mld, mode, L, d, heads, ffn, T, 32, dec_tensors, kcd, vcd)
    y = torch.empty(d, dtype=torch.float16, device="cuda")
    dec.step(_dev(x), y, pos)
    torch.cuda.synchronize()
    assert dec.device_status() == 0
    kref, vref = kc.astype(np.float32), vc.astype(np.float32)
    xf = x.astype(np.float32)
    ref = decode_ref.decode_step(xf, layers_ref, kref, vref, pos, heads, 128, ffn)
    got = y.float().cpu().numpy()
    assert np.isfinite(got).all()
    # The step's own contribution is y - x; with outlier channels the residual dwarfs it, so the bound is
    # stated against the contribution (1e-2 of its largest element) plus the fp16 rounding of the stored
    # output itself (2 ulp), element by element.
    contrib = np.max(np.abs(ref - xf))
    tol = 1e-2 * contrib + 2.0 * _fp16_ulp(ref)
    assert np.all(np.abs(got - ref) <= tol), float(np.max(np.abs(got - ref) / tol))
    assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) < 1e-2
    # the new token's cache rows: rotated k and v of both layers (inputs of later steps)
    kgot, vgot = kcd[:, pos].float().cpu().numpy(), vcd[:, pos].float().cpu().numpy()
    assert np.max(np.abs(kgot - kref[:, pos])) <= 1e-2 * np.max(np.abs(kref[:, pos])) + 1e-3
    assert np.max(np.abs(vgot - vref[:, pos])) <= 1e-2 * np.max(np.abs(vref[:, pos])) + 1e-3
    dec.close()


def test_outlier_channels_in_a_small_decoder(mld, oracle):
    """The outlier case on a decoder small enough to check every projection output of the first layer
    through the cache rows: k and v of the new token are plain projection outputs (v untouched, k only
    rotated), so their error is the projection's, measured against the projection's own magnitude."""
    from oracle import decode_ref
    rng = np.random.default_rng(5)
    L, heads, ffn, T, pos = 1, 8, 2816, 64, 40
    d = heads * 128
    layers_ref, dec_tensors, kc, vc = build_small_decoder(mld, oracle, rng, L, heads, ffn, T, pos)
    x = rng.standard_normal(d).astype(np.float32)
    x[[3, 500, 901]] = [300.0, 300.0, -300.0]
    g = layers_ref[0]["norm1"].copy()
    g[17] = 50.0
    layers_ref[0]["norm1"] = g.astype(np.float16).astype(np.float32)
    dec_tensors[0]["norm1"] = _dev(g.astype(np.float16))
    x = x.astype(np.float16)
    for mode in ("mega", "ops"):
        kcd, vcd = _dev(kc), _dev(vc)
        dec = _make(mld, mode, L, d, heads, ffn, T, 32, dec_tensors, kcd, vcd)
        y = torch.empty(d, dtype=torch.float16, device="cuda")
        dec.step(_dev(x), y, pos)
        torch.cuda.synchronize()
        assert dec.device_status() == 0
        kref, vref = kc.astype(np.float32), vc.astype(np.float32)
        decode_ref.decode_step(x.astype(np.float32), layers_ref, kref, vref, pos, heads, 128, ffn)
        for got, ref in ((kcd[0, pos], kref[0, pos]), (vcd[0, pos], vref[0, pos])):
            got = got.float().cpu().numpy()
            # fp32-accumulate bound of the FullyConnected path: 1e-3 of the output's scale, plus the fp16
            # rounding of the stored value
            assert np.all(np.abs(got - ref) <= 1e-3 * np.max(np.abs(ref)) + 1.0 * _fp16_ulp(ref)), mode
        dec.close()


def test_step_after_a_wait_that_ran_out(mld, oracle):
    """A step whose device-side waits are given one microsecond gives up somewhere (the first weight box
    takes longer than that to arrive), reports it to the host and leaves the GPU usable; after the
    status has been read the decoder works again and a step matches the oracle - nothing written by the
    abandoned step passes for data of the next one."""
    from oracle import decode_ref
    rng = np.random.default_rng(9)
    L, heads, ffn, T, pos = 2, 4, 1408, 200, 150
    d = heads * 128
    layers_ref, dec_tensors, kc, vc = build_small_decoder(mld, oracle, rng, L, heads, ffn, T, pos)
    x = rng.standard_normal(d).astype(np.float16)
    kref, vref = kc.astype(np.float32), vc.astype(np.float32)
    ref = decode_ref.decode_step(x.astype(np.float32), layers_ref, kref, vref, pos, heads, 128, ffn)
    kcd, vcd = _dev(kc), _dev(vc)
    dec = _make(mld, "mega", L, d, heads, ffn, T, 32, dec_tensors, kcd, vcd)
    xd = _dev(x)
    y = torch.empty(d, dtype=torch.float16, device="cuda")
    dec.step(xd, y, pos)                      # one good step first: its tagged words stay in memory
    torch.cuda.synchronize()
    assert dec.device_status() == 0
    dec.set_wait_limit(1)
    xh = x.copy()
    xt = torch.from_numpy(xh).pin_memory()
    yt = torch.empty(d, dtype=torch.float16).pin_memory()
    failed = 0
    for _ in range(3):
        try:
            dec.step_host(xt, yt, pos)
        except mld.MldError as e:
            assert e.status == mld.TIMEOUT
            failed += 1
            assert dec.device_status() != 0     # reads, clears and resets the hand-over state
    dec.set_wait_limit(0)
    assert dec.device_status() == 0
    kcd.copy_(_dev(kc))
    vcd.copy_(_dev(vc))
    for _ in range(2):
        dec.step(xd, y, pos)
        torch.cuda.synchronize()
        assert dec.device_status() == 0
        got = y.float().cpu().numpy()
        assert np.max(np.abs(got - ref)) / np.max(np.abs(ref)) < 1e-2
    if failed == 0:
        pytest.skip("no wait exceeded one microsecond on this run; recovery path not exercised")
    dec.close()


@pytest.mark.parametrize("heads,n_tokens", [(2, 1), (2, 70), (32, 2049), (4, 515), (64, 33)])
def test_attention_decode_matches_softmax(mld, heads, n_tokens):
    rng = np.random.default_rng(heads * 1000 + n_tokens)
    q = (rng.standard_normal((heads, 128)) / np.sqrt(128)).astype(np.float16)
    k = rng.standard_normal((n_tokens, heads, 128)).astype(np.float16)
    v = rng.standard_normal((n_tokens, heads, 128)).astype(np.float16)
    out = torch.empty((heads, 128), dtype=torch.float16, device="cuda")
    mld.attn_decode(_dev(q), _dev(k), _dev(v), out, heads, n_tokens)
    torch.cuda.synchronize()
    s = np.einsum("hd,thd->ht", q.astype(np.float64), k.astype(np.float64))
    p = np.exp(s - s.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    ref = np.einsum("ht,thd->hd", p, v.astype(np.float64))
    got = out.float().cpu().numpy()
    assert np.max(np.abs(got - ref)) <= 2e-3 * max(1.0, np.max(np.abs(ref)))
