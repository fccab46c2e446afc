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


def _make(mld, monkeypatch, mode, L, d, heads, ffn, T, block, dec_tensors, kcd, vcd):
    monkeypatch.setenv("MLD_DECODER_MODE", mode)    # read when the decoder is created
    dec = mld.Decoder(L, d, heads, ffn, T, block=block)
    assert dec.single_kernel == (mode == "mega")
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
    ("mega", 3, 4, 1408, 200, 0, 32),
    ("mega", 3, 4, 1408, 200, 31, 32),
    ("mega", 2, 4, 1408, 200, 32, 32),
    ("mega", 2, 4, 1408, 200, 199, 32),
    ("mega", 1, 8, 2816, 1100, 1030, 32),
    ("mega", 2, 2, 512, 96, 64, 128),
    ("mega", 2, 2, 256, 96, 65, 256),
])
def test_decode_step_matches_oracle(mld, oracle, monkeypatch, mode, L, heads, ffn, T, pos, block):
    from oracle import decode_ref
    rng = np.random.default_rng(0)
    d = heads * 128
    layers_ref, dec_tensors, kc, vc = build_small_decoder(mld, oracle, rng, L, heads, ffn, T, pos, block=block)
    x = rng.standard_normal(d).astype(np.float16)
    kcd, vcd = _dev(kc), _dev(vc)
    dec = _make(mld, monkeypatch, mode, L, d, heads, ffn, T, block, dec_tensors, kcd, vcd)
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
def test_single_kernel_step_on_small_grids(mld, oracle, monkeypatch, grid, heads, ffn, T, pos):
    from oracle import decode_ref
    monkeypatch.setenv("MLD_MEGA_GRID", str(grid))
    rng = np.random.default_rng(grid)
    L, d = 2, heads * 128
    layers_ref, dec_tensors, kc, vc = build_small_decoder(mld, oracle, rng, L, heads, ffn, T, pos)
    x = rng.standard_normal(d).astype(np.float16)
    kcd, vcd = _dev(kc), _dev(vc)
    dec = _make(mld, monkeypatch, "mega", L, d, heads, ffn, T, 32, dec_tensors, kcd, vcd)
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
def test_single_kernel_step_with_a_short_ring(mld, oracle, monkeypatch, stages):
    """Rings shorter than two stages per consumer warp (large vectors leave that little shared memory)
    put fewer warps on attention and must give the same step; the step is run several times so that
    consecutive launches, whose vectors carry different tags, are covered too."""
    from oracle import decode_ref
    monkeypatch.setenv("MLD_MEGA_STAGES", str(stages))
    rng = np.random.default_rng(stages)
    L, heads, ffn, T, pos = 2, 4, 1408, 1024, 1000
    d = heads * 128
    layers_ref, dec_tensors, kc, vc = build_small_decoder(mld, oracle, rng, L, heads, ffn, T, pos)
    x = rng.standard_normal(d).astype(np.float16)
    kcd, vcd = _dev(kc), _dev(vc)
    dec = _make(mld, monkeypatch, "mega", L, d, heads, ffn, T, 32, dec_tensors, kcd, vcd)
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


def test_single_kernel_step_ignores_uninitialised_cache_rows(mld, oracle, monkeypatch):
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
    dec = _make(mld, monkeypatch, "mega", L, d, heads, ffn, T, 32, dec_tensors, kcd, vcd)
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


def test_single_kernel_step_agrees_with_op_chain(mld, oracle, monkeypatch):
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
        dec = _make(mld, monkeypatch, mode, L, d, heads, ffn, T, 32, dec_tensors, kcd, vcd)
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
