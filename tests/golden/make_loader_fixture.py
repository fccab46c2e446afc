"""Generates tests/golden/loader_fixture/: the file set that the reference's own converter
(ml_drift/samples/llm/extract_weights_hf.py: extract_model_weights, with optimize_scale=False) writes
for a seeded random one-layer decoder, which the loader tests then read.

    python tests/golden/make_loader_fixture.py /path/to/ml-drift

The state dict (names as in a Hugging Face Qwen checkpoint; tiny dimensions) is saved as one .safetensors
file in a temporary directory and converted twice: block-wise INT4 (block 32) for the attention and
feed-forward projections with an INT8 embedding into loader_fixture/int4_block32/, and per-channel INT8
for everything into loader_fixture/int8/.  Two files are added by this script itself, because the
converter never writes them but the loader accepts them
(ml_drift/samples/llm/llm_file_tensor_loader.cc:57-96, 399-452): a scale file in the "group header"
form (int32 group size, then int16 values in units of 1/1024) and its int8 twin.  The fixture directory is
committed; tests only read it.
"""
import importlib.util
import os
import shutil
import sys
import tempfile

import numpy as np
import torch

D_MODEL, FFN, VOCAB, HEAD_DIM = 64, 160, 96, 16


def state_dict(seed):
    g = torch.Generator().manual_seed(seed)
    r = lambda *shape: torch.randn(*shape, generator=g) * 0.05
    p = "model.layers.0."
    sd = {
        "model.embed_tokens.weight": r(VOCAB, D_MODEL),
        p + "input_layernorm.weight": 1.0 + r(D_MODEL),
        p + "post_attention_layernorm.weight": 1.0 + r(D_MODEL),
        p + "self_attn.q_proj.weight": r(D_MODEL, D_MODEL),
        p + "self_attn.k_proj.weight": r(D_MODEL // 2, D_MODEL),
        p + "self_attn.v_proj.weight": r(D_MODEL // 2, D_MODEL),
        p + "self_attn.o_proj.weight": r(D_MODEL, D_MODEL),
        p + "self_attn.q_norm.weight": 1.0 + r(HEAD_DIM),
        p + "self_attn.k_norm.weight": 1.0 + r(HEAD_DIM),
        p + "mlp.gate_proj.weight": r(FFN, D_MODEL),
        p + "mlp.up_proj.weight": r(FFN, D_MODEL),
        p + "mlp.down_proj.weight": r(D_MODEL, FFN),
        "model.norm.weight": 1.0 + r(D_MODEL),
    }
    # a zero output row and a zero block, the cases whose scale the quantiser sets to 1
    sd[p + "mlp.up_proj.weight"][3, :] = 0.0
    sd[p + "mlp.gate_proj.weight"][5, 32:64] = 0.0
    return {k: v.contiguous() for k, v in sd.items()}


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_loader_fixture.py /path/to/ml-drift")
    path = os.path.join(sys.argv[1], "ml_drift", "samples", "llm", "extract_weights_hf.py")
    spec = importlib.util.spec_from_file_location("extract_weights_hf", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    from safetensors.torch import save_file

    here = os.path.dirname(os.path.abspath(__file__))
    out_root = os.path.join(here, "loader_fixture")
    shutil.rmtree(out_root, ignore_errors=True)
    with tempfile.TemporaryDirectory() as tmp:
        model = os.path.join(tmp, "model.safetensors")
        save_file(state_dict(0), model)
        mod.extract_model_weights(model, os.path.join(out_root, "int4_block32"), embedding_quant_bits=8,
                                  attention_quant_bits=4, feedforward_quant_bits=4, block_size=32,
                                  optimize_scale=False)
        mod.extract_model_weights(model, os.path.join(out_root, "int8"), embedding_quant_bits=8,
                                  attention_quant_bits=8, feedforward_quant_bits=8, block_size=0,
                                  optimize_scale=False)

    # the "group header" scale forms, derived from the float scales of one projection
    d = os.path.join(out_root, "int4_block32")
    name = "model.layers.0.mlp.down_proj.weight_quantized_scale"
    s = np.fromfile(os.path.join(d, name), dtype=np.float32)
    for suffix, dtype in ((".grouped_int16", np.int16), (".grouped_int8", np.int8)):
        q = np.clip(np.rint(s * 1024.0), np.iinfo(dtype).min, np.iinfo(dtype).max).astype(dtype)
        with open(os.path.join(d, name + suffix), "wb") as f:
            np.int32(32).tofile(f)
            q.tofile(f)
    for root, _, files in os.walk(out_root):
        for fn in sorted(files):
            print(os.path.relpath(os.path.join(root, fn), out_root), os.path.getsize(os.path.join(root, fn)))


if __name__ == "__main__":
    main()
