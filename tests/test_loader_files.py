"""The weight-file rules of the loader that need no GPU: which files exist, element widths, group-size
deduction and float reads through the C ABI, against the numpy restatement of the reference's loader and
against the committed file set (tests/golden/loader_fixture, written by the reference's own converter; the
script beside it regenerates it).  The files themselves are also checked against the restated quantiser, run
on the same seeded weights the generating script used."""
import importlib.util
import os

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
FIXTURE = os.path.join(ROOT, "tests", "golden", "loader_fixture")
P = "model.layers.0."
# name -> (O, I)
PROJECTIONS = {
    P + "self_attn.q_proj.weight": (64, 64), P + "self_attn.k_proj.weight": (32, 64),
    P + "self_attn.v_proj.weight": (32, 64), P + "self_attn.o_proj.weight": (64, 64),
    P + "mlp.gate_proj.weight": (160, 64), P + "mlp.up_proj.weight": (160, 64), P + "mlp.down_proj.weight": (64, 160),
}


@pytest.fixture(scope="module")
def mld():
    import __graft_entry__ as g
    return g.import_package()


@pytest.fixture(scope="module")
def loader_ref():
    from oracle import loader_ref
    return loader_ref


@pytest.fixture(scope="module")
def seeded_weights():
    spec = importlib.util.spec_from_file_location("make_loader_fixture",
                                                  os.path.join(ROOT, "tests", "golden", "make_loader_fixture.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return {k: v.float().numpy() for k, v in mod.state_dict(0).items()}


def test_layer_info_lists_every_tensor():
    lines = [l.strip() for l in open(os.path.join(FIXTURE, "int4_block32", "layer_info.txt")) if l.strip()]
    assert f"mdl_vars.{P}mlp.down_proj.weight.int4.64_160" in lines
    assert f"mdl_vars.{P}mlp.down_proj.weight_quantized_scale.float32.64_5" in lines
    assert "mdl_vars.model.embed_tokens.weight.int8.96_64" in lines
    assert f"mdl_vars.{P}input_layernorm.weight.float32.64" in lines


@pytest.mark.parametrize("variant,bits,block", [("int4_block32", 4, 32), ("int8", 8, 0)])
def test_files_are_what_the_restated_quantiser_writes(oracle, seeded_weights, variant, bits, block):
    d = os.path.join(FIXTURE, variant) + os.sep
    for name, (o, i) in PROJECTIONS.items():
        w = seeded_weights[name]
        assert w.shape == (o, i)
        if bits == 4:
            q, s = oracle.quantize_int4_sym(w, block)
            want = oracle.pack_int4_dense(q)
        else:
            q, s = oracle.quantize_int8_sym(w)
            want = q.reshape(-1).view(np.uint8)
        assert np.array_equal(np.fromfile(d + name, dtype=np.uint8), want), name
        assert np.array_equal(np.fromfile(d + name + "_quantized_scale", dtype=np.float32), s.reshape(-1)), name
    # the zero row and the zero block got scale 1
    s = np.fromfile(d + P + "mlp.up_proj.weight_quantized_scale", dtype=np.float32)
    g = 2 if bits == 4 else 1
    assert np.all(s.reshape(160, g)[3] == 1.0)
    if bits == 4:
        assert np.fromfile(d + P + "mlp.gate_proj.weight_quantized_scale", dtype=np.float32).reshape(160, 2)[5, 1] == 1.0


@pytest.mark.parametrize("variant", ["int4_block32", "int8"])
def test_host_side_rules_match_the_restatement(mld, loader_ref, variant):
    d = os.path.join(FIXTURE, variant) + os.sep
    ld = mld.FileTensorLoader(d)
    for name, (o, i) in PROJECTIONS.items():
        assert ld.has_tensor(name) and ld.has_tensor(name + "_quantized_scale")
        assert ld.element_bits(name, o * i) == loader_ref.element_bits(d, name, o * i) == (4 if variant == "int4_block32" else 8)
        assert ld.group_size(name, o, i) == loader_ref.group_size(d, name, o, i) == (32 if variant == "int4_block32" else i)
        assert ld.group_size(name, o, i) == ld.group_size(name, o, i)      # the cached answer
    assert ld.element_bits(P + "input_layernorm.weight", 64) == 32
    assert ld.element_bits("model.embed_tokens.weight", 96 * 64) == 8
    assert ld.group_size("model.embed_tokens.weight", 96, 64) == 64
    assert not ld.has_tensor("model.layers.1.mlp.up_proj.weight")
    assert ld.element_bits("model.layers.1.mlp.up_proj.weight", 10) == 0
    assert ld.element_bits(P + "input_layernorm.weight", 0) == 0
    assert ld.group_size("model.layers.1.mlp.up_proj.weight", 8, 24) == 24   # no scale file: one group
    norm = ld.load_float32(P + "input_layernorm.weight", 64).numpy()
    assert np.array_equal(norm, np.fromfile(d + P + "input_layernorm.weight", dtype=np.float32))
    padded = ld.load_float32(P + "self_attn.q_norm.weight", 20).numpy()     # a short file leaves zeros behind
    assert np.array_equal(padded[:16], np.fromfile(d + P + "self_attn.q_norm.weight", dtype=np.float32))
    assert np.all(padded[16:] == 0.0)
    with pytest.raises(mld.MldError) as e:
        ld.load_float32("missing.weight", 4)
    assert e.value.status == mld.NOT_FOUND
    ld.close()


def test_group_header_scale_files(mld, loader_ref, tmp_path):
    """The second scale form (int32 group size, then int16 or int8 values in units of 1/1024): the group size
    comes from the header when the size is not a whole number of float32 values per output."""
    src = os.path.join(FIXTURE, "int4_block32") + os.sep
    name = P + "mlp.down_proj.weight"
    o, i = PROJECTIONS[name]
    for form in ("grouped_int16", "grouped_int8"):
        d = str(tmp_path / form) + os.sep
        os.makedirs(d)
        raw = open(src + name + "_quantized_scale." + form, "rb").read()
        open(d + name + "_quantized_scale", "wb").write(raw)
        open(d + name, "wb").write(open(src + name, "rb").read())
        ld = mld.FileTensorLoader(d)
        want = loader_ref.group_size(d, name, o, i)
        assert ld.group_size(name, o, i) == want
        # int16: 4 + 2 * 320 = 644 bytes = 161 float32 values, not a multiple of 64 outputs -> header rule (32);
        # int8: 4 + 320 = 324 bytes = 81 values -> header rule as well
        assert want == 32
        assert loader_ref.is_grouped(d + name + "_quantized_scale", o * (i // 32))
        ld.close()


def test_group_size_answers_of_the_reference_loader_test(mld, loader_ref, tmp_path):
    """The two cases of samples/llm/llm_file_tensor_loader_test.cc:196-264, with their caching: the answer
    survives the removal of the scale file."""
    d = str(tmp_path) + os.sep
    ld = mld.FileTensorLoader(d)
    # ten float32 values for OHWI(5, 1, 1, 8): two scales per output -> groups of 4 inputs
    f = d + "model.layers.0.mlp.gate_proj.weight_quantized_scale"
    np.ones(10, np.float32).tofile(f)
    assert loader_ref.group_size(d, "model.layers.0.mlp.gate_proj.weight", 5, 8) == 4
    assert ld.group_size("model.layers.0.mlp.gate_proj.weight", 5, 8) == 4
    os.remove(f)
    assert ld.group_size("model.layers.0.mlp.gate_proj.weight", 5, 8) == 4
    # header 16, then eight int8 values, for OHWI(4, 1, 1, 32): 12 bytes = 3 float32 values, not a multiple of
    # the 4 outputs, so the header decides
    f = d + "model.layers.1.mlp.gate_proj.weight_quantized_scale"
    with open(f, "wb") as fh:
        np.int32(16).tofile(fh)
        np.ones(8, np.int8).tofile(fh)
    assert loader_ref.group_size(d, "model.layers.1.mlp.gate_proj.weight", 4, 32) == 16
    assert ld.group_size("model.layers.1.mlp.gate_proj.weight", 4, 32) == 16
    os.remove(f)
    assert ld.group_size("model.layers.1.mlp.gate_proj.weight", 4, 32) == 16
    # and the float read of the same test (:80-95, 148-154)
    np.arange(1, 11, dtype=np.float32).tofile(d + "model.layers.9.mlp.gate_proj.weight_quantized_scale")
    got = ld.load_float32("model.layers.9.mlp.gate_proj.weight_quantized_scale", 10).numpy()
    assert np.array_equal(got, np.arange(1, 11, dtype=np.float32))
    ld.close()
