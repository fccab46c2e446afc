"""Quantised embedding lookup and the lm_head projection over one packed table, through the C ABI."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mld():
    import __graft_entry__ as g
    return g.import_package()


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_reference_known_answers_on_the_gpu(mld, oracle):
    # ml_drift/common/kernels/tests/embedding_lookup_test_util.cc:133-310
    table8 = np.arange(1, 17, dtype=np.int8).reshape(4, 4)
    out = torch.empty(4, dtype=torch.float32, device="cuda")
    mld.embedding_lookup(_dev(np.int32([1])), _dev(oracle.rearrange_int8_as_uint8(table8)), _dev(np.ones(4, np.float32)),
                         out, 4, 4, 8, zero_point=_dev(np.zeros(4, np.float32)), f16=False)
    assert out.cpu().tolist() == [5.0, 6.0, 7.0, 8.0]
    table4 = np.int8([[0, 1, 2, 3], [4, 5, 6, 7], [0, -1, -2, -3], [-4, -5, -6, -7]])
    packed = _dev(oracle.rearrange_int8_as_uint4(table4))
    for idx, want in ((1, [4.0, 5.0, 6.0, 7.0]), (3, [-4.0, -5.0, -6.0, -7.0])):
        mld.embedding_lookup(_dev(np.int32([idx])), packed, _dev(np.ones(4, np.float32)), out, 4, 4, 4,
                             zero_point=_dev(np.zeros(4, np.float32)), f16=False)
        assert out.cpu().tolist() == want


@pytest.mark.parametrize("bits,vocab,dim,block,f16,layout", [
    (4, 1000, 512, 32, True, "row"), (4, 37, 64, 0, False, "row"), (8, 533, 172, 0, True, "sliced"),
    (4, 4096, 4096, 32, True, "sliced"), (8, 100, 256, 0, False, "row"),
])
def test_lookup_matches_oracle(mld, oracle, bits, vocab, dim, block, f16, layout):
    rng = np.random.default_rng(vocab + dim)
    w = (rng.standard_normal((vocab, dim)) * 0.02).astype(np.float32)
    if bits == 4:
        q, s = oracle.quantize_int4_sym(w, block)
        packed = oracle.rearrange_int8_as_uint4(q)
    else:
        q, s = oracle.quantize_int8_sym(w)
        packed = oracle.rearrange_int8_as_uint8(q)
    s = s.reshape(vocab, -1)
    G = s.shape[1]
    sl = oracle.scale_layout(s, f16)
    s_used = oracle.f16_bits_to_f32(oracle.f32_to_f16_bits(s)) if f16 else s
    ids = np.int32([0, 1, vocab - 1, vocab // 2, 3, 3, vocab + 5, -1] + list(rng.integers(0, vocab, 9)))
    T = len(ids)
    S = (dim + 3) // 4
    lay = mld.LAYOUT_SLICED if layout == "sliced" else mld.LAYOUT_ROW_MAJOR
    dt = torch.float16 if f16 else torch.float32
    out = torch.full((S * T * 4,) if layout == "sliced" else (T * dim,), float("nan"), dtype=dt, device="cuda")
    mld.embedding_lookup(_dev(ids), _dev(packed), _dev(sl.view(np.float16) if f16 else sl), out, vocab, dim, bits,
                         scale_mode=mld.SCALE_BLOCK if G > 1 else mld.SCALE_PER_CHANNEL, groups=G, f16=f16, dst_layout=lay)
    torch.cuda.synchronize()
    got = out.float().cpu().numpy()
    got = oracle.from_sliced(got.reshape(S, T, 4), dim) if layout == "sliced" else got.reshape(T, dim)
    ref = oracle.embedding_lookup(ids, packed, vocab, dim, bits, s_used)
    if f16:
        ref = ref.astype(np.float16).astype(np.float32)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("vocab", [151936, 262144])
def test_lm_head_projection_at_vocabulary_width(mld, oracle, vocab):
    """The lm_head is one more decode GEMV over the embedding table's packed layout: N = vocabulary (151 936
    and 262 144 rows), K = 4096, INT4 block 32.  Weights are quantised and packed on the GPU; sampled
    outputs are checked against exact arithmetic on the same integers, and a looked-up row against the
    same table."""
    K, blk = 4096, 32
    g = torch.Generator(device="cuda").manual_seed(vocab)
    packed = torch.empty(mld.packed_size_bytes(vocab, K, 4), dtype=torch.uint8, device="cuda")
    # quantise in row chunks (the fp32 matrix would take 2.5 - 4.3 GB at once), then pack the whole table
    q = torch.empty((vocab, K), dtype=torch.int8, device="cuda")
    s = torch.empty((vocab, K // blk), dtype=torch.float32, device="cuda")
    for r0 in range(0, vocab, 32768):
        r1 = min(vocab, r0 + 32768)
        w = torch.randn((r1 - r0, K), generator=g, device="cuda") * 0.02
        qc, sc = mld.quantize_weights(w, 4, blk)
        q[r0:r1], s[r0:r1] = qc, sc
    packed, _ = mld.pack_weights(q, (vocab, 1, 1, K), 4)
    scales = mld.pack_scales(s, True)
    x = torch.randn(K, generator=g, device="cuda").half()
    plan = mld.FullyConnectedPlan(vocab, K, 4, scale_mode=mld.SCALE_BLOCK, groups=K // blk, precision=mld.F32F16)
    y = torch.full((vocab,), float("nan"), dtype=torch.float16, device="cuda")
    plan.run(x, packed, scales, y, 1)
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    assert bool(torch.isfinite(y).all())
    rows = torch.tensor([0, 1, 2, 3, 63, 64, 1000, vocab // 2, vocab - 65, vocab - 2, vocab - 1] +
                        list(np.random.default_rng(0).integers(0, vocab, 200)), device="cuda")
    s16 = scales.t()[rows].double()                                    # [rows][G], as stored (fp16)
    qd = q[rows].double().reshape(len(rows), K // blk, blk)
    ref = ((qd * x.double().reshape(1, K // blk, blk)).sum(-1) * s16).sum(-1)
    got = y[rows].double()
    assert float((got - ref).abs().max()) <= 1e-3 * float(ref.abs().max()) + 1e-3 * float(y.float().abs().max())
    # the lookup of a token returns the row the projection multiplied with
    ids = rows[:16].int()
    emb = torch.empty((16, K), dtype=torch.float16, device="cuda")
    mld.embedding_lookup(ids, packed, scales, emb, vocab, K, 4, scale_mode=mld.SCALE_BLOCK, groups=K // blk)
    torch.cuda.synchronize()
    want = (q[rows[:16]].float().reshape(16, K // blk, blk) * scales.t()[rows[:16]].float()[:, :, None]).reshape(16, K)
    assert float((emb.float() - want).abs().max()) <= 2 ** -11 * float(want.abs().max())
    plan.close()
