"""Generates tests/golden/quantiser_vectors.npz by running the reference's own
quantiser functions (ml_drift/samples/llm/extract_weights_hf.py:
quantize_tensor_int8_sym, quantize_tensor_int4_sym, pack_int4; all with
optimize_scale=False) on seeded inputs.

Run where the reference checkout is available:
    python tests/golden/make_quantiser_vectors.py /path/to/ml-drift
The .npz it writes is committed; tests only read the .npz.
"""
import importlib.util
import os
import sys

import numpy as np


def main():
    if len(sys.argv) != 2:
        sys.exit("usage: make_quantiser_vectors.py /path/to/ml-drift")
    ref_root = sys.argv[1]
    path = os.path.join(ref_root, "ml_drift", "samples", "llm", "extract_weights_hf.py")
    spec = importlib.util.spec_from_file_location("extract_weights_hf", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    rng = np.random.default_rng(0)
    out = {}
    # (name, O, I, sigma)
    cases = [("a", 8, 64, 0.02), ("b", 5, 96, 1.0), ("c", 12, 128, 0.02)]
    for name, O, I, sigma in cases:
        w = (rng.standard_normal((O, I)) * sigma).astype(np.float32)
        if name == "b":
            w[1, :] = 0.0          # zero row -> scale 1
            w[2, 32:64] = 0.0      # zero block
            w[3, 0] = 0.5 * w[3, 1]  # exercise ties-ish values
        out[f"{name}_w"] = w
        q8, s8 = mod.quantize_tensor_int8_sym(w, quant_axis=1, optimize_scale=False)
        out[f"{name}_q8"], out[f"{name}_s8"] = q8, s8
        q4c, s4c = mod.quantize_tensor_int4_sym(w, quant_axis=1, block_size=0, optimize_scale=False)
        out[f"{name}_q4c"], out[f"{name}_s4c"] = q4c, s4c
        q4b, s4b = mod.quantize_tensor_int4_sym(w, quant_axis=1, block_size=32, optimize_scale=False)
        out[f"{name}_q4b"], out[f"{name}_s4b"] = q4b, s4b
        out[f"{name}_p4b"] = mod.pack_int4(q4b)
    # exact half-way cases for round-half-to-even: w/scale = k + 0.5
    w = np.array([[7.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5] + [0.0] * 24], np.float32)
    q, s = mod.quantize_tensor_int4_sym(w, quant_axis=1, block_size=32, optimize_scale=False)
    out["tie_w"], out["tie_q4b"], out["tie_s4b"] = w, q, s
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "quantiser_vectors.npz")
    np.savez_compressed(dst, **out)
    print("wrote", dst, os.path.getsize(dst), "bytes")


if __name__ == "__main__":
    main()
