"""The loader's device half through the C ABI: packed weights, weight sums, scales and zero points read from
the committed file set (tests/golden/loader_fixture) against the CPU packers applied to the same bytes, and a
projection run from loaded tensors against plain arithmetic on the file's contents."""
import os

import numpy as np
import pytest
import torch

from test_loader_files import FIXTURE, P, PROJECTIONS

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mld():
    import __graft_entry__ as g
    return g.import_package()


@pytest.fixture(scope="module")
def loader_ref():
    from oracle import loader_ref
    return loader_ref


def test_int4_weights_and_sums_equal_the_cpu_packer(mld, oracle, loader_ref):
    d = os.path.join(FIXTURE, "int4_block32") + os.sep
    ld = mld.FileTensorLoader(d)
    for name, (o, i) in PROJECTIONS.items():
        packed, sums = ld.load_weights(name, 4, o, i)
        raw = np.fromfile(d + name, dtype=np.uint8)
        want, want_sums = oracle.rearrange_uint4_packed(raw, (o, 1, 1, i))
        assert np.array_equal(packed.cpu().numpy(), want), name
        assert np.array_equal(sums.cpu().numpy(), want_sums), name
        q = loader_ref.int4_file_as_int8(d + name, o * i).reshape(o, i)
        assert np.array_equal(want_sums, oracle.weights_sum_i(q)), name       # and the slow path's sums agree
        assert np.array_equal(want, oracle.rearrange_int8_as_uint4(q)), name  # and its packing
    ld.close()


def test_int8_weights_with_and_without_swapped_dims(mld, oracle, tmp_path):
    d = os.path.join(FIXTURE, "int8") + os.sep
    ld = mld.FileTensorLoader(d)
    name = P + "mlp.down_proj.weight"
    o, i = PROJECTIONS[name]
    q = np.fromfile(d + name, dtype=np.int8).reshape(o, i)
    packed, sums = ld.load_weights(name, 8, o, i)
    assert np.array_equal(packed.cpu().numpy(), oracle.rearrange_int8_as_uint8(q))
    assert np.array_equal(sums.cpu().numpy(), oracle.weights_sum_i(q))
    ld.close()
    # the same matrix stored [i][o], as checkpoints with transposed projections have it
    t = str(tmp_path) + os.sep
    np.ascontiguousarray(q.T).tofile(t + name)
    ld = mld.FileTensorLoader(t)
    packed_t, sums_t = ld.load_weights(name, 8, o, i, swap_dims=True)
    assert torch.equal(packed_t, packed) and torch.equal(sums_t, sums)
    # INT4, stored [i][o]
    d4 = os.path.join(FIXTURE, "int4_block32") + os.sep
    q4 = np.fromfile(d4 + name, dtype=np.uint8)
    from oracle import loader_ref
    v = loader_ref.int4_file_as_int8(d4 + name, o * i).reshape(o, i)
    oracle.pack_int4_dense(np.ascontiguousarray(v.T)).tofile(t + "swapped.weight")
    got, got_sums = ld.load_weights("swapped.weight", 4, o, i, swap_dims=True)
    want, want_sums = oracle.rearrange_uint4_packed(q4, (o, 1, 1, i))
    assert np.array_equal(got.cpu().numpy(), want) and np.array_equal(got_sums.cpu().numpy(), want_sums)
    ld.close()


@pytest.mark.parametrize("f16", [True, False])
def test_scales_in_both_file_forms(mld, oracle, loader_ref, f16, tmp_path):
    d = os.path.join(FIXTURE, "int4_block32") + os.sep
    ld = mld.FileTensorLoader(d)
    dt = np.float16 if f16 else np.float32
    for name, (o, i) in PROJECTIONS.items():
        g = i // 32
        got = ld.load_scale(name + "_quantized_scale", o, g, f16=f16).cpu().numpy()
        s = loader_ref.scale_values(d + name + "_quantized_scale", o, g)
        want = oracle.scale_layout(s, f16).reshape(-1)
        assert np.array_equal(got.view(np.uint16 if f16 else np.float32), want), name
    name = P + "mlp.down_proj.weight_quantized_scale"
    for form in (".grouped_int16", ".grouped_int8"):
        got = ld.load_scale(name + form, 64, 5, f16=f16).cpu().numpy()
        s = loader_ref.scale_values(d + name + form, 64, 5)
        assert np.all(s * 1024 == np.rint(s * 1024))        # whole multiples of 1/1024
        assert np.array_equal(got.view(np.uint16 if f16 else np.float32), oracle.scale_layout(s, f16).reshape(-1))
    with pytest.raises(mld.MldError) as e:
        ld.load_scale("missing_quantized_scale", 8, 1)
    assert e.value.status == mld.NOT_FOUND
    with pytest.raises(mld.MldError) as e:
        ld.load_weights("missing.weight", 4, 8, 8)
    assert e.value.status == mld.NOT_FOUND
    ld.close()
    del dt


def test_zero_points(mld, oracle, loader_ref, tmp_path):
    t = str(tmp_path) + os.sep
    rng = np.random.default_rng(3)
    o, g = 12, 4
    scale = (rng.random((o, g)).astype(np.float32) + 0.5) * 0.01
    scale[2, 1] = 0.0                                         # a zero scale gives a zero result
    zp = rng.integers(-8, 8, (o, g)).astype(np.float32)
    scale.tofile(t + "a.weight_quantized_scale")
    (zp * scale).astype(np.float32).tofile(t + "a.weight_quantized_zp")
    ld = mld.FileTensorLoader(t)
    got = ld.load_zero_point("a.weight_quantized_zp", "a.weight_quantized_scale", o, g, f16=False).cpu().numpy()
    want = loader_ref.zero_point_values(t + "a.weight_quantized_zp", t + "a.weight_quantized_scale", o, g)
    assert want[2, 1] == 0.0
    assert np.array_equal(got, oracle.scale_layout(want, False).reshape(-1))
    none = ld.load_zero_point("b.weight_quantized_zp", "a.weight_quantized_scale", o, g, f16=True)
    assert not none.cpu().numpy().view(np.uint16).any()       # no file: zero points of zero
    ld.close()


def test_projection_from_loaded_files(mld, oracle, loader_ref):
    """gate_proj of the fixture, one token: loader -> operator against plain arithmetic on the file contents."""
    d = os.path.join(FIXTURE, "int4_block32") + os.sep
    name = P + "mlp.gate_proj.weight"
    o, i = PROJECTIONS[name]
    ld = mld.FileTensorLoader(d)
    assert ld.element_bits(name, o * i) == 4
    block = ld.group_size(name, o, i)
    g = i // block
    packed, _ = ld.load_weights(name, 4, o, i)
    scale = ld.load_scale(name + "_quantized_scale", o, g, f16=True)
    ld.close()
    rng = np.random.default_rng(9)
    x = rng.standard_normal((1, i)).astype(np.float16)
    plan = mld.FullyConnectedPlan(o, i, 4, scale_mode=mld.SCALE_BLOCK, groups=g, precision=mld.F32F16)
    y = torch.zeros(o, dtype=torch.float16, device="cuda")
    plan.run(torch.from_numpy(x.reshape(-1)).cuda(), packed, scale, y, 1)
    torch.cuda.synchronize()
    plan.close()
    q = loader_ref.int4_file_as_int8(d + name, o * i).reshape(o, i)
    s = loader_ref.scale_values(d + name + "_quantized_scale", o, g)
    s16 = oracle.f16_bits_to_f32(oracle.f32_to_f16_bits(s))
    ref = oracle.fc_plain_reference(q, s16, x.astype(np.float32))
    got = y.float().cpu().numpy()[None]
    assert np.max(np.abs(got - ref)) <= 1e-3 * np.max(np.abs(ref))


def test_tiny_files_of_the_reference_loader_test(mld, oracle, loader_ref, tmp_path):
    """The int8 (5 x 2) and int4 (8 x 1, the word 0x12345678) files of
    samples/llm/llm_file_tensor_loader_test.cc:96-112: both load, and the packed bytes are the CPU packer's."""
    d = str(tmp_path) + os.sep
    np.arange(1, 11, dtype=np.int8).tofile(d + "model.layers.9.mlp.gate_proj.weight")
    np.array([0x12345678], np.int32).tofile(d + "model.layers.9.mlp.gate_proj.weight_int4")
    ld = mld.FileTensorLoader(d)
    packed, sums = ld.load_weights("model.layers.9.mlp.gate_proj.weight", 8, 5, 2)
    q = np.arange(1, 11, dtype=np.int8).reshape(5, 2)
    assert np.array_equal(packed.cpu().numpy(), oracle.rearrange_int8_as_uint8(q))
    assert np.array_equal(sums.cpu().numpy(), q.astype(np.int32).sum(1))
    packed4, sums4 = ld.load_weights("model.layers.9.mlp.gate_proj.weight_int4", 4, 8, 1)
    raw = np.fromfile(d + "model.layers.9.mlp.gate_proj.weight_int4", dtype=np.uint8)
    want, want_sums = oracle.rearrange_uint4_packed(raw, (8, 1, 1, 1))
    assert np.array_equal(packed4.cpu().numpy(), want) and np.array_equal(sums4.cpu().numpy(), want_sums)
    v = loader_ref.int4_file_as_int8(d + "model.layers.9.mlp.gate_proj.weight_int4", 8)
    assert list(v) == [-8, 7, 6, 5, 4, 3, 2, 1]          # nibbles of 0x12345678, low first, two's complement
    assert np.array_equal(want_sums, v.astype(np.int32))
    ld.close()
