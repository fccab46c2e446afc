"""Decode dequant-GEMV through the C ABI vs the CPU oracle.

Tolerances, as max |y - ref| / max |ref|:
  * against the restated kernel in the same precision mode: 1e-3 for fp32
    tensors, 1e-2 for fp16 tensors (the restated kF16/kF32F16 kernels round
    every dequantised weight and every product to half, so they sit up to
    ~1.5e-3 away from exact arithmetic themselves);
  * against the exact-arithmetic reference (FullyConnectedReference over
    MakeWeightsFromInt8, what the reference's own big tests compare with):
    1e-3, since the CUDA kernels accumulate in fp32;
  * plus the reference's own bound GetEpsilon(precision) * (K + 1) * 2
    (ml_drift/common/task/testing_util.cc:328-331) on its ragged shapes."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

REL_TOL = {"F32": 1e-3, "F32F16": 1e-2, "F16": 1e-2}


@pytest.fixture(scope="module")
def mld():
    import __graft_entry__ as g
    return g.import_package()


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _run(mld, oracle, precision, bits, x, packed, N, K, scale=None, zp=None, bias=None, mode=None, G=1,
         scalar_scale=0.0, scalar_zp=None, layout="sliced", force_generic=False, exact_operands=False):
    """Runs mld_fc_run on logical float inputs; returns [M][N] float32."""
    prec = getattr(mld, precision)
    half = precision != "F32"
    M = x.shape[0]
    dt = np.float16 if half else np.float32
    if layout == "sliced":
        xs = oracle.to_sliced(x).astype(dt)
    else:
        xs = x.astype(dt)
    sc = zpd = bd = None
    if mode != mld.SCALE_SCALAR:
        sc = oracle.scale_layout(scale, half)
        sc = _dev(sc.view(np.float16) if half else sc)
        if zp is not None:
            z = oracle.scale_layout(zp, half)
            zpd = _dev(z.view(np.float16) if half else z)
    if bias is not None:
        b = oracle.scale_layout(np.asarray(bias, np.float32), half)
        bd = _dev(b.view(np.float16) if half else b)
    lay = mld.LAYOUT_SLICED if layout == "sliced" else mld.LAYOUT_ROW_MAJOR
    plan = mld.FullyConnectedPlan(N, K, bits, scale_mode=mode, groups=G, scalar_scale=scalar_scale,
                                  scalar_zero_point=0.0 if scalar_zp is None else scalar_zp,
                                  has_zero_point=(zp is not None or scalar_zp is not None),
                                  has_bias=bias is not None, precision=prec, src_layout=lay, dst_layout=lay,
                                  max_tokens=M, force_path=mld.PATH_GEMV, exact_operands=exact_operands)
    if force_generic:
        plan_ws = plan.workspace_bytes()
    S = (N + 3) // 4
    tdt = torch.float16 if half else torch.float32
    y = torch.full((S * M * 4,) if layout == "sliced" else (M * N,), float("nan"), dtype=tdt, device="cuda")
    plan.run(_dev(xs), _dev(packed), sc, y, M, zero_point=zpd, bias=bd)
    torch.cuda.synchronize()
    out = y.float().cpu().numpy()
    plan.close()
    if layout == "sliced":
        return oracle.from_sliced(out.reshape(S, M, 4), N)
    return out.reshape(M, N)


def _rel(a, b):
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


# ------------------------------------------------------------- known answers
@pytest.mark.parametrize("precision", ["F32", "F16", "F32F16"])
def test_reference_known_answers(mld, oracle, precision):
    # ml_drift/common/kernels/tests/fully_connected_test_util.cc
    f32 = precision == "F32"
    # :49-103 INT8, scalar scale 0.5, bias -> {20.5, 15.5}
    q = np.array([[2, 4, 6, 8], [10, 12, -14, 16]], np.int8)
    y = _run(mld, oracle, precision, 8, np.float32([[0, 1, 2, 3]]), oracle.rearrange_int8_as_uint8(q), 2, 4,
             bias=np.float32([0.5, -0.5]), mode=mld.SCALE_SCALAR, scalar_scale=0.5)
    assert np.allclose(y, [[20.5, 15.5]], atol=1e-6 if f32 else 1e-3, rtol=0)
    # :105-175 INT8 block-wise, 2 groups -> {91.0, 26.8}
    q = np.array([[1, 1, 1, 1, 2, 2, 2, 2], [3, 3, 3, 3, 4, 4, 4, 4]], np.int8)
    y = _run(mld, oracle, precision, 8, np.arange(8, dtype=np.float32)[None], oracle.rearrange_int8_as_uint8(q), 2, 8,
             scale=np.float32([[0.5, 2.0], [1.0, 0.1]]), bias=np.float32([0, 0]), mode=mld.SCALE_BLOCK, G=2)
    assert np.allclose(y, [[91.0, 26.8]], atol=1e-5 if f32 else 0.05, rtol=0)
    # :177-249 block-wise + zero points -> {509.0, -121.4}
    q = np.array([[1, 2, 3, 4, 5, 6, 7, 8], [-8, -7, -6, -5, -4, -3, -2, -1]], np.int8)
    y = _run(mld, oracle, precision, 8, np.arange(1, 9, dtype=np.float32)[None], oracle.rearrange_int8_as_uint8(q), 2, 8,
             scale=np.float32([[0.5, 2.0], [1.5, 0.1]]), zp=np.float32([[2, -3], [1, 4]]), bias=np.float32([0, 0]),
             mode=mld.SCALE_BLOCK, G=2)
    assert np.allclose(y, [[509.0, -121.4]], atol=1e-5 if f32 else 0.1, rtol=0)
    # :1541-1614 INT4 block-wise all ones -> 8.0
    q = np.ones((4, 16), np.int8)
    y = _run(mld, oracle, precision, 4, np.ones((1, 16), np.float32), oracle.rearrange_int8_as_uint4(q), 4, 16,
             scale=np.full((4, 2), 0.5, np.float32), bias=np.zeros(4, np.float32), mode=mld.SCALE_BLOCK, G=2)
    assert np.allclose(y, 8.0, atol=1e-6 if f32 else 1e-2, rtol=0)


# ------------------------------------------- the reference's ragged big tests
def _uniform(rng, shape):
    return rng.uniform(-1.0, 1.0, size=shape).astype(np.float32)


@pytest.mark.parametrize("precision", ["F32", "F16", "F32F16"])
@pytest.mark.parametrize("bits,K,N,G,M,use_zp", [
    (8, 171, 533, 1, 1, False), (8, 171, 533, 1, 15, False), (8, 171, 533, 1, 2, False),
    (8, 364, 533, 13, 1, False), (4, 171, 533, 1, 1, False), (4, 364, 533, 13, 1, False),
    (4, 364, 533, 7, 1, True), (4, 171, 533, 1, 4, False), (8, 171, 533, 1, 10, False),
])
def test_ragged_shapes_vs_oracle(mld, oracle, precision, bits, K, N, G, M, use_zp):
    rng = np.random.default_rng(bits * 7919 + K + N + G + M)
    wf = _uniform(rng, (N, K))
    if bits == 8:
        q = (np.clip(((wf + 1.0) * 256.0).astype(np.int32), 0, 255) - 128).astype(np.int8)
        scale = _uniform(rng, (N, G)) / 128.0
        packed = oracle.rearrange_int8_as_uint8(q)
    else:
        q = (np.clip(((wf + 1.0) * 16.0).astype(np.int32), 0, 15) - 8).astype(np.int8)
        scale = _uniform(rng, (N, G)) / 8.0
        packed = oracle.rearrange_int8_as_uint4(q)
    zp = rng.integers(-3, 4, size=(N, G)).astype(np.float32) if use_zp else None
    bias = _uniform(rng, (N,))
    x = _uniform(rng, (M, K))
    if precision != "F32":
        x = x.astype(np.float16).astype(np.float32)
    mode = mld.SCALE_BLOCK if G > 1 else mld.SCALE_PER_CHANNEL
    y = _run(mld, oracle, precision, bits, x, packed, N, K, scale=scale, zp=zp, bias=bias, mode=mode, G=G)
    ref = oracle.fc_forward(getattr(oracle, precision), bits, x, packed, N=N, K=K, scale=scale, zp=zp, bias=bias,
                            scale_mode=oracle.SCALE_BLOCK if G > 1 else oracle.SCALE_CHANNEL, G=G)
    assert _rel(y, ref) <= REL_TOL[precision]
    plain = oracle.fc_plain_reference(q, scale, x, zp=zp, bias=bias)
    eps = (1.1920929e-07 if precision == "F32" else 9.7656e-4) * (K + 1) * 2
    assert np.max(np.abs(y - plain)) <= eps


# ------------------------------------------------------- the streaming kernel
def _quantised_case(oracle, rng, bits, K, N, block):
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    if bits == 4:
        q, s = oracle.quantize_int4_sym(w, block)
        packed = oracle.rearrange_int8_as_uint4(q)
    else:
        q, s = oracle.quantize_int8_sym(w)
        s = s.reshape(-1, 1)
        packed = oracle.rearrange_int8_as_uint8(q)
    return q, s, packed


STREAM_CASES = [
    # bits, K, N, block, M
    (4, 2048, 16384, 32, 1),     # the decode GEMV benchmark case (FFN up-projection)
    (4, 4096, 4096, 32, 1),      # 7B attention projection
    (4, 11008, 4096, 32, 1),     # 7B down projection: ragged last K chunk, split-K
    (4, 4096, 11008, 32, 1),     # 7B up projection: ragged last tile
    (4, 512, 64, 32, 1),         # one tile
    (4, 8192, 64, 32, 1),        # one tile split over many CTAs
    (4, 2048, 1024, 32, 2), (4, 2048, 1024, 32, 5), (4, 2048, 1024, 32, 8),
    (4, 2048, 1024, 32, 9), (4, 2048, 1024, 32, 16),
    (4, 2048, 1024, 64, 1), (4, 2048, 1024, 128, 3), (4, 2048, 1024, 256, 1), (4, 2048, 1024, 512, 1),
    (4, 2048, 1024, 1024, 1), (4, 2048, 1024, 0, 1),
    (8, 2048, 2048, 0, 1),       # the W8 per-channel case with fp16 tensors
    (8, 4096, 1000, 0, 4), (8, 1024, 3584, 0, 16),
    (4, 512, 65536, 32, 1),      # strips wider than four boxes: several column passes per CTA
    (4, 1024, 40000, 128, 2),    # multi-pass with ragged last strip
    (8, 8192, 3584, 0, 1),       # one rank's shard of the W8A8 prefill case, one token
    (4, 256, 4096, 32, 1),       # K too short to split: narrow strips, one CTA each
    (4, 1024, 8, 32, 1), (4, 1024, 16, 32, 3), (8, 1024, 8, 0, 1),   # a single chunk / unit
]


@pytest.mark.parametrize("operands", ["subnormal", "exact"])
@pytest.mark.parametrize("bits,K,N,block,M", STREAM_CASES)
def test_streaming_gemv_vs_oracle(mld, oracle, operands, bits, K, N, block, M):
    rng = np.random.default_rng(bits + K + N + block + M)
    q, s, packed = _quantised_case(oracle, rng, bits, K, N, block)
    G = s.shape[1]
    x = rng.standard_normal((M, K)).astype(np.float16).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.01).astype(np.float32) if (N % 3 == 0) else None
    mode = mld.SCALE_BLOCK if G > 1 else mld.SCALE_PER_CHANNEL
    y = _run(mld, oracle, "F32F16", bits, x, packed, N, K, scale=s, bias=bias, mode=mode, G=G,
             exact_operands=operands == "exact")
    assert not np.isnan(y).any()
    plain = oracle.fc_plain_reference(q, oracle.f16_bits_to_f32(oracle.f32_to_f16_bits(s)), x,
                                      bias=None if bias is None else bias.astype(np.float16).astype(np.float32))
    assert _rel(y, plain) <= 1e-3
    if K * N * M <= 2048 * 16384:
        ref = oracle.fc_forward(oracle.F32F16, bits, x, packed, N=N, K=K, scale=s, bias=bias,
                                scale_mode=oracle.SCALE_BLOCK if G > 1 else oracle.SCALE_CHANNEL, G=G)
        assert _rel(y, ref) <= REL_TOL["F32F16"]


def test_streaming_gemv_kf16_request(mld, oracle):
    # kF16 tensors are served by the same kernel; compare with the half-accumulating oracle at 1e-2
    rng = np.random.default_rng(3)
    K, N = 512, 256
    q, s, packed = _quantised_case(oracle, rng, 4, K, N, 32)
    x = rng.standard_normal((1, K)).astype(np.float16).astype(np.float32)
    y = _run(mld, oracle, "F16", 4, x, packed, N, K, scale=s, mode=mld.SCALE_BLOCK, G=K // 32)
    ref = oracle.fc_forward(oracle.F16, 4, x, packed, N=N, K=K, scale=s, scale_mode=oracle.SCALE_BLOCK, G=K // 32)
    assert _rel(y, ref) <= 1e-2


def test_streaming_gemv_is_deterministic_and_reusable(mld, oracle):
    rng = np.random.default_rng(5)
    K, N = 8192, 192                      # tiles split over several CTAs -> ticketed reduction
    q, s, packed = _quantised_case(oracle, rng, 4, K, N, 32)
    x = rng.standard_normal((1, K)).astype(np.float16)
    plan = mld.FullyConnectedPlan(N, K, 4, scale_mode=mld.SCALE_BLOCK, groups=K // 32, precision=mld.F32F16)
    xd, pd = _dev(x.reshape(-1)), _dev(packed)
    sd = _dev(oracle.scale_layout(s, True).view(np.float16))
    outs = []
    for _ in range(5):
        y = torch.zeros(N, dtype=torch.float16, device="cuda")
        plan.run(xd, pd, sd, y, 1)
        outs.append(y)
    torch.cuda.synchronize()
    for o in outs[1:]:
        assert torch.equal(o, outs[0])
    plain = oracle.fc_plain_reference(q, oracle.f16_bits_to_f32(oracle.f32_to_f16_bits(s)), x.astype(np.float32))
    assert _rel(outs[0].float().cpu().numpy()[None], plain) <= 1e-3


def test_independent_launches_overlap_and_finish_in_stream_order(mld, oracle):
    """independent_io: the launches do not wait for one another at the activation load.  Their results equal
    the ordinary plan's bit for bit, and a kernel queued behind them on the stream sees all of them."""
    rng = np.random.default_rng(15)
    K, N = 2048, 4096
    sets = []
    for i in range(6):
        q, s, packed = _quantised_case(oracle, rng, 4, K, N, 32)
        sets.append((_dev(packed), _dev(oracle.scale_layout(s, True).view(np.float16))))
    x = _dev(rng.standard_normal(K).astype(np.float16))
    ref_plan = mld.FullyConnectedPlan(N, K, 4, scale_mode=mld.SCALE_BLOCK, groups=K // 32, precision=mld.F32F16)
    plan = mld.FullyConnectedPlan(N, K, 4, scale_mode=mld.SCALE_BLOCK, groups=K // 32, precision=mld.F32F16,
                                  independent_io=True)
    want = [torch.zeros(N, dtype=torch.float16, device="cuda") for _ in sets]
    for (w, sc), y in zip(sets, want):
        ref_plan.run(x, w, sc, y, 1)
    torch.cuda.synchronize()
    for _ in range(3):
        got = [torch.zeros(N, dtype=torch.float16, device="cuda") for _ in sets]
        for (w, sc), y in zip(sets, got):
            plan.run(x, w, sc, y, 1)
        total = torch.stack(got).float().sum(0)        # queued behind the six launches, no synchronisation between
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            assert torch.equal(a, b)
        assert torch.equal(total, torch.stack(want).float().sum(0))
    assert plan.device_status() == 0
    plan.close()
    ref_plan.close()


@pytest.mark.parametrize("K,N,block", [(2048, 1024, 32), (40, 64, 0), (200, 328, 0), (4096, 512, 64), (1032, 1160, 0),
                                       (11008, 256, 128)])
@pytest.mark.parametrize("outliers", [False, True])
def test_one_token_int4_digit_route(mld, oracle, K, N, block, outliers):
    """4-bit weights with one token take integer MMAs on the activations as 16-bit fixed point, one
    power-of-two scale per 32 inputs: K tails inside a unit and inside a stage, several scale groupings,
    channels at 300 sigma, all against the plain dequantised product and against the fp16 route."""
    rng = np.random.default_rng(K * 3 + N + block)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    if block:
        q, s = oracle.quantize_int4_sym(w, block)
        mode, G = mld.SCALE_BLOCK, K // block
    else:
        q, s = oracle.quantize_int4_sym(w, 0)
        mode, G = mld.SCALE_PER_CHANNEL, 1
    packed = oracle.rearrange_int8_as_uint4(q)
    x = rng.standard_normal((1, K)).astype(np.float32)
    if outliers:
        x[0, rng.choice(K, 3, replace=False)] *= 300.0
    x = x.astype(np.float16).astype(np.float32)
    s16 = oracle.f16_bits_to_f32(oracle.f32_to_f16_bits(s))
    plain = oracle.fc_plain_reference(q, s16, x)
    y = _run(mld, oracle, "F32F16", 4, x, packed, N, K, scale=s, mode=mode, G=G)
    exact = _run(mld, oracle, "F32F16", 4, x, packed, N, K, scale=s, mode=mode, G=G, exact_operands=True)
    assert _rel(exact, plain) <= 1e-3
    assert _rel(y, plain) <= 1e-3
    assert _rel(y, exact) <= 1e-3
    if outliers:  # an infinity among the inputs must not come out as finite numbers
        x[0, K // 2] = np.inf
        y = _run(mld, oracle, "F32F16", 4, x, packed, N, K, scale=s, mode=mode, G=G)
        assert not np.isfinite(y).any()


def test_row_major_single_token(mld, oracle):
    rng = np.random.default_rng(6)
    K, N = 1024, 512
    q, s, packed = _quantised_case(oracle, rng, 4, K, N, 32)
    x = rng.standard_normal((1, K)).astype(np.float16).astype(np.float32)
    y = _run(mld, oracle, "F32F16", 4, x, packed, N, K, scale=s, mode=mld.SCALE_BLOCK, G=K // 32, layout="row")
    plain = oracle.fc_plain_reference(q, oracle.f16_bits_to_f32(oracle.f32_to_f16_bits(s)), x)
    assert _rel(y, plain) <= 1e-3


def test_config1_f32_int8(mld, oracle):
    # the W8 per-channel CPU-runnable case: N=2048, K=2048, INT8, fp32 activations and bias, seed 0
    rng = np.random.default_rng(0)
    K = N = 2048
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    x = rng.standard_normal((1, K)).astype(np.float32)
    bias = (rng.standard_normal(N) * 0.01).astype(np.float32)
    q, s = oracle.quantize_int8_sym(w)
    packed = oracle.rearrange_int8_as_uint8(q)
    y = _run(mld, oracle, "F32", 8, x, packed, N, K, scale=s, bias=bias, mode=mld.SCALE_PER_CHANNEL)
    ref = oracle.fc_forward(oracle.F32, 8, x, packed, N=N, K=K, scale=s, bias=bias, scale_mode=oracle.SCALE_CHANNEL)
    assert _rel(y, ref) <= 1e-3
    assert np.max(np.abs(y - ref)) <= 1.1920929e-07 * (K + 1) * 2


def test_errors(mld):
    with pytest.raises(mld.MldError) as e:
        mld.FullyConnectedPlan(16, 16, 5)
    assert e.value.status == mld.INVALID_ARGUMENT
    # features of the reference operator that are not built are refused by name
    for kwargs, word in ((dict(weight_bits=2), "INT2"), (dict(weight_bits=4, runtime_channel_bounds=True), "channel bounds"),
                         (dict(weight_bits=4, has_batch_ids=True), "batch ids")):
        with pytest.raises(mld.MldError) as e:
            mld.FullyConnectedPlan(16, 16, **kwargs)
        assert e.value.status == mld.UNIMPLEMENTED and word in str(e.value)
    with pytest.raises(mld.MldError) as e:
        mld.quantize_weights(torch.zeros((4, 32), device="cuda"), 4, 32, optimize_scale=True)
    assert e.value.status == mld.UNIMPLEMENTED and "optimize_scale" in str(e.value)
    plan = mld.FullyConnectedPlan(16, 16, 4, max_tokens=2)
    x = torch.zeros(64, dtype=torch.float16, device="cuda")
    with pytest.raises(mld.MldError):
        plan.run(x, x, x, x, 3)          # more tokens than planned
    with pytest.raises(mld.MldError):
        plan.run(x, x, None, x, 1)       # per-channel scale tensor missing
