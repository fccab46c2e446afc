"""Prefill dequant-GEMM (tcgen05) through the C ABI vs the CPU oracle.

Every case runs on each route: "inline" (the GEMM reads the packed weights and dequantises them in shared
tensor memory - or, "inline_smem", in shared memory; what the cost rule picks up to 512 tokens), "convert" (a conversion pass writes a K-major copy and
a GEMM with both operands loaded by TMA follows; the rule's pick above 512 tokens) and "cached" (the
same with the copy kept between calls).  All apply the same arithmetic to every weight.
Float route: tolerance 1e-3 of max |ref| against the restated WeightsConverter + fp32-accumulate GEMM
(fp16 operands, exact products).  Int8-activation route: the int32 accumulators are exact, so outputs
agree with the restated Quantize -> int GEMM -> Dequantization chain to fp16 rounding."""
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


def _rel(a, b):
    return float(np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30))


ROUTES = [("inline", False), ("inline_smem", False), ("convert", False), ("cached", True)]
ROUTE_CODE = {"inline": 1, "convert": 2, "cached": 0, "auto": 0, "inline_smem": 3}


def _run_gemm(mld, oracle, x16, packed, scale_dev, N, K, bits, mode, G, bias=None, layout="sliced", act_quant=0,
              cache=False, reps=1, w_sum=None, route="auto"):
    M = x16.shape[0]
    lay = mld.LAYOUT_SLICED if layout == "sliced" else mld.LAYOUT_ROW_MAJOR
    xs = oracle.to_sliced(x16.astype(np.float32)).astype(np.float16) if layout == "sliced" else x16
    plan = mld.FullyConnectedPlan(N, K, bits, scale_mode=mode, groups=G, has_bias=bias is not None,
                                  precision=mld.F32F16, src_layout=lay, dst_layout=lay, max_tokens=M,
                                  force_path=mld.PATH_GEMM, prefill_act_quant=act_quant, cache_prepared_weights=cache,
                                  prefill_route=ROUTE_CODE[route])
    S = (N + 3) // 4
    y = torch.full((S * M * 4,) if layout == "sliced" else (M * N,), float("nan"), dtype=torch.float16, device="cuda")
    bd = None if bias is None else _dev(oracle.scale_layout(bias, True).view(np.float16))
    xd, pd = _dev(xs), _dev(packed)
    if w_sum is not None:
        plan.set_weights_sum(_dev(np.asarray(w_sum, np.int32)))
    for _ in range(reps):
        plan.run(xd, pd, scale_dev, y, M, bias=bd)
    torch.cuda.synchronize()
    assert plan.device_status() == 0
    out = y.float().cpu().numpy()
    plan.close()
    return oracle.from_sliced(out.reshape(S, M, 4), N) if layout == "sliced" else out.reshape(M, N)


@pytest.mark.parametrize("route,cache", ROUTES)
@pytest.mark.parametrize("M,K,N,block,layout", [
    (128, 128, 64, 32, "sliced"), (128, 256, 256, 32, "sliced"), (17, 64, 16, 32, "sliced"),
    (100, 200, 72, 0, "sliced"), (300, 512, 520, 32, "row"), (256, 1024, 1000, 128, "sliced"),
    (1024, 512, 2048, 32, "sliced"),
    (257, 320, 20, 32, "sliced"),       # a weight row pitch no tensor map can express: served by the prepared route
    (700, 4096, 1200, 64, "sliced"),    # several tiles per SM pair, two scale groups per stage
    (40, 2048, 6000, 32, "row"),        # few tokens: the pair's second CTA holds no rows
    (2048, 320, 2560, 32, "sliced"),    # 80 tiles on 74 SM pairs: neighbouring pairs share tiles along K
])
def test_int4_prefill_gemm_vs_oracle(mld, oracle, route, cache, M, K, N, block, layout):
    rng = np.random.default_rng(M + K + N)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    q, s = oracle.quantize_int4_sym(w, block)
    packed = oracle.rearrange_int8_as_uint4(q)
    G = s.shape[1]
    sgn = oracle.scale_layout(s, True)
    x16 = rng.standard_normal((M, K)).astype(np.float16)
    bias = (rng.standard_normal(N) * 0.01).astype(np.float32) if N % 3 == 0 else None
    y = _run_gemm(mld, oracle, x16, packed, _dev(sgn.view(np.float16)), N, K, 4,
                  mld.SCALE_BLOCK if G > 1 else mld.SCALE_PER_CHANNEL, G, bias=bias, layout=layout, cache=cache, reps=2,
                  route=route)
    assert not np.isnan(y).any()
    ref = oracle.f16_bits_to_f32(oracle.prefill_gemm_int4(x16.view(np.uint16), packed, sgn, N))
    if bias is not None:
        ref = (ref.astype(np.float16) + bias.astype(np.float16)).astype(np.float32)
    assert _rel(y, ref) <= 1e-3


@pytest.mark.parametrize("route,cache", ROUTES)
@pytest.mark.parametrize("M,K,N", [(64, 256, 96), (300, 1024, 520)])
def test_int8_weights_float_route(mld, oracle, route, cache, M, K, N):
    rng = np.random.default_rng(8)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    q, s = oracle.quantize_int8_sym(w)
    packed = oracle.rearrange_int8_as_uint8(q)
    sgn = oracle.scale_layout(s, True)
    x16 = rng.standard_normal((M, K)).astype(np.float16)
    y = _run_gemm(mld, oracle, x16, packed, _dev(sgn.view(np.float16)), N, K, 8, mld.SCALE_PER_CHANNEL, 1, cache=cache,
                  route=route)
    ref = oracle.f16_bits_to_f32(oracle.prefill_gemm_int4(x16.view(np.uint16), packed, sgn, N, bits=8))
    assert _rel(y, ref) <= 1e-3


@pytest.mark.parametrize("rule,route,cache", [("symmetric", "inline", False), ("symmetric", "cached", True),
                                              ("asymmetric", "inline", False), ("asymmetric", "convert", False)])
@pytest.mark.parametrize("M,K,N", [(64, 128, 32), (256, 512, 128), (130, 1040, 264), (32, 8192, 96), (300, 2048, 520),
                                   (1100, 384, 4608)])   # the last: 90 tiles on 74 SM pairs, tiles shared along K
def test_w8a8_prefill_vs_oracle(mld, oracle, rule, route, cache, M, K, N):
    rng = np.random.default_rng(M * 3 + K + N)
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    q, s = oracle.quantize_int8_sym(w)
    packed = oracle.rearrange_int8_as_uint8(q)
    s16 = oracle.scale_layout(s, True)                          # the operator stores scales in fp16
    x16 = rng.standard_normal((M, K)).astype(np.float16)
    sym = rule == "symmetric"
    if not sym:
        x16 = (x16.astype(np.float32) + 0.6).astype(np.float16)   # a shifted distribution: the offset term matters
    w_sum = oracle.weights_sum_i(q)
    y = _run_gemm(mld, oracle, x16, packed, _dev(s16.view(np.float16)), N, K, 8, mld.SCALE_PER_CHANNEL, 1,
                  act_quant=1 if sym else 2, cache=cache, w_sum=None if sym else w_sum, route=route)
    quantise = oracle.quantize_act_sym if sym else oracle.quantize_act_asym
    xq, params = quantise(x16.view(np.uint16), src_f16=True)
    acc = oracle.gemm_s8s8_s32(xq, q)
    ws = oracle.f16_bits_to_f32(s16).reshape(-1)[:N]
    ref = oracle.f16_bits_to_f32(oracle.dequant_epilogue(acc, params, ws, w_sum))
    assert not np.isnan(y).any()
    assert np.max(np.abs(y - ref)) <= 2 * np.finfo(np.float16).eps * np.max(np.abs(ref))
    # and close to the float product it approximates
    assert _rel(y, x16.astype(np.float32) @ w.T) < 3e-2


def test_w8a8_shard_of_the_eight_way_split(mld, oracle):
    """One rank's share of the W8A8 prefill case that is split eight ways over N: M=2048, K=8192,
    N=3584 of 28672, asymmetric per-token activations.  Sampled tokens against the restated chain: the
    int32 accumulators over K=8192 are exact, the outputs agree to fp16 rounding."""
    M, K, N = 2048, 8192, 3584
    g = torch.Generator(device="cuda").manual_seed(5)
    w = torch.randn((N, K), generator=g, device="cuda") * 0.02
    q, s = mld.quantize_weights(w, 8)
    packed, w_sum = mld.pack_weights(q, (N, 1, 1, K), 8, want_sum=True)
    sc = mld.pack_scales(s, True)
    x = (torch.randn((M, K), generator=g, device="cuda") + 0.3).half()
    xs = x.reshape(M, K // 4, 4).permute(1, 0, 2).contiguous()
    rows = [0, 1, 127, 128, 255, 256, 1000, 1500, 2046, 2047]
    qh = q.cpu().numpy()
    ws = sc.float().cpu().numpy().reshape(-1)[:N]
    for rule, aq, route in (("asymmetric", 2, "auto"), ("asymmetric", 2, "inline"), ("symmetric", 1, "auto")):
        plan = mld.FullyConnectedPlan(N, K, 8, scale_mode=mld.SCALE_PER_CHANNEL, precision=mld.F32F16, max_tokens=M,
                                      force_path=mld.PATH_GEMM, prefill_act_quant=aq,
                                      prefill_route=ROUTE_CODE[route])
        if aq == 2:
            plan.set_weights_sum(w_sum)
        y = torch.empty((N // 4, M, 4), dtype=torch.float16, device="cuda")
        plan.run(xs, packed, sc, y, M)
        torch.cuda.synchronize()
        assert plan.device_status() == 0
        got = y.permute(1, 0, 2).reshape(M, N)[rows].float().cpu().numpy()
        quantise = oracle.quantize_act_sym if aq == 1 else oracle.quantize_act_asym
        xq, params = quantise(x[rows].cpu().numpy().view(np.uint16), src_f16=True)
        acc = oracle.gemm_s8s8_s32(xq, qh)
        ref = oracle.f16_bits_to_f32(oracle.dequant_epilogue(acc, params, ws, w_sum.cpu().numpy()))
        assert np.isfinite(got).all(), rule
        assert np.max(np.abs(got - ref)) <= 2 * np.finfo(np.float16).eps * np.max(np.abs(ref)), rule
        plan.close()


def test_prefill_dispatch_threshold_and_cache(mld, oracle):
    # 17 tokens at kF32F16 leave the decode kernel (IsFullyConnectedRecommended) and take the GEMM;
    # a second call with cached prepared weights returns the same bits
    rng = np.random.default_rng(21)
    M, K, N = 17, 256, 128
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    q, s = oracle.quantize_int4_sym(w, 32)
    packed = oracle.rearrange_int8_as_uint4(q)
    sgn = oracle.scale_layout(s, True)
    x16 = rng.standard_normal((M, K)).astype(np.float16)
    xs = oracle.to_sliced(x16.astype(np.float32)).astype(np.float16)
    plan = mld.FullyConnectedPlan(N, K, 4, scale_mode=mld.SCALE_BLOCK, groups=K // 32, precision=mld.F32F16,
                                  max_tokens=M, cache_prepared_weights=True)
    xd, pd, sd = _dev(xs), _dev(packed), _dev(sgn.view(np.float16))
    y1 = torch.zeros(N * M, dtype=torch.float16, device="cuda")
    y2 = torch.zeros_like(y1)
    c0 = mld.kernel_launch_count()
    plan.run(xd, pd, sd, y1, M)
    c1 = mld.kernel_launch_count()
    plan.run(xd, pd, sd, y2, M)
    c2 = mld.kernel_launch_count()
    torch.cuda.synchronize()
    assert c1 - c0 == 2 and c2 - c1 == 2        # conversion (+ transpose in the same launch) + gemm, then transpose + gemm
    assert torch.equal(y1, y2)
    ref = oracle.f16_bits_to_f32(oracle.prefill_gemm_int4(x16.view(np.uint16), packed, sgn, N))
    got = oracle.from_sliced(y1.float().cpu().numpy().reshape(N // 4, M, 4), N)
    assert _rel(got, ref) <= 1e-3


def test_conversion_cost_rule_picks_the_route(mld, oracle):
    # up to 512 tokens the weights are dequantised inside the GEMM; above that a conversion pass runs first (the
    # activations' transposition rides along in its launch); both give the oracle's answer
    rng = np.random.default_rng(33)
    K, N = 512, 256
    w = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    q, s = oracle.quantize_int4_sym(w, 32)
    packed = oracle.rearrange_int8_as_uint4(q)
    sgn = oracle.scale_layout(s, True)
    plan = mld.FullyConnectedPlan(N, K, 4, scale_mode=mld.SCALE_BLOCK, groups=K // 32, precision=mld.F32F16,
                                  max_tokens=600)
    pd, sd = _dev(packed), _dev(sgn.view(np.float16))
    for M, route in ((512, mld.ROUTE_PREFILL_INLINE), (513, mld.ROUTE_PREFILL_CONVERTED)):
        x16 = rng.standard_normal((M, K)).astype(np.float16)
        xd = _dev(oracle.to_sliced(x16.astype(np.float32)).astype(np.float16))
        y = torch.zeros(N * M, dtype=torch.float16, device="cuda")
        c0 = mld.kernel_launch_count()
        plan.run(xd, pd, sd, y, M)
        assert mld.kernel_launch_count() - c0 == 2 and plan.last_route() == route
        torch.cuda.synchronize()
        ref = oracle.f16_bits_to_f32(oracle.prefill_gemm_int4(x16.view(np.uint16), packed, sgn, N))
        got = oracle.from_sliced(y.float().cpu().numpy().reshape(N // 4, M, 4), N)
        assert _rel(got, ref) <= 1e-3
    plan.close()


@pytest.mark.parametrize("route", ["auto", "inline"])
def test_config3_full_size_sampled(mld, oracle, route):
    # the prefill benchmark case: M=1024, K=4096, N=14336, INT4 block 32; the oracle checks 8 sampled tokens
    M, K, N = 1024, 4096, 14336
    g = torch.Generator(device="cuda").manual_seed(0)
    w = torch.randn((N, K), generator=g, device="cuda") * 0.02
    q, s = mld.quantize_weights(w, 4, 32)
    packed, _ = mld.pack_weights(q, (N, 1, 1, K), 4)
    sc = mld.pack_scales(s, True)
    x = torch.randn((M, K), generator=g, device="cuda").half()
    xs = x.reshape(M, K // 4, 4).permute(1, 0, 2).contiguous()      # sliced [K/4][M][4]
    plan = mld.FullyConnectedPlan(N, K, 4, scale_mode=mld.SCALE_BLOCK, groups=K // 32, precision=mld.F32F16,
                                  max_tokens=M, force_path=mld.PATH_GEMM, prefill_route=ROUTE_CODE[route])
    y = torch.empty((N // 4, M, 4), dtype=torch.float16, device="cuda")
    plan.run(xs, packed, sc, y, M)
    torch.cuda.synchronize()
    rows = [0, 1, 127, 128, 500, 777, 1000, 1023]
    got = y.permute(1, 0, 2).reshape(M, N)[rows].float().cpu().numpy()
    ref = oracle.f16_bits_to_f32(oracle.prefill_gemm_int4(
        x[rows].cpu().numpy().view(np.uint16), packed.cpu().numpy(), sc.cpu().numpy().view(np.uint16), N))
    assert _rel(got, ref) <= 1e-3
    # linearity over tokens: a second run on 2x gives exactly 2y wherever y is a normal fp16 number
    # (the fp32 accumulators double exactly; only subnormal results can round differently)
    y2 = torch.empty_like(y)
    plan.run((xs * 2).contiguous(), packed, sc, y2, M)
    torch.cuda.synchronize()
    normal = y.abs() >= 6.2e-5
    assert torch.equal(y2[normal], (y * 2)[normal])
    assert float((y2.float() - 2 * y.float()).abs().max()) <= 2 ** -23
    # and the kernel is deterministic
    y3 = torch.empty_like(y)
    plan.run((xs * 2).contiguous(), packed, sc, y3, M)
    torch.cuda.synchronize()
    assert torch.equal(y2, y3)
    plan.close()
