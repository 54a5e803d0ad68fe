"""Generates tests/golden/tf_tiny_layer.npz from the reference's own Python model of the fp8 transformer layer
(zkllm-src/transformer_ref.py: TinyLayer, seq 4, d 64, 2 heads of 32, d_ff 128, rng seed 20260703 as its --dump-layer):
weights, gains, RoPE tables, the input and every traced activation.  Run where the reference tree is present:

    python tests/golden/make_tf_layer_golden.py /path/to/zkllm-src
"""
import contextlib
import io
import os
import sys

import numpy as np


def main(src):
    sys.path.insert(0, src)
    with contextlib.redirect_stdout(io.StringIO()):
        import transformer_ref as R
    rng = np.random.default_rng(20260703)
    layer = R.TinyLayer(np.random.default_rng(20260703))
    x = np.array([[R.bf_from_f64(v) for v in row] for row in rng.normal(0, 1.0, (4, 64))], np.uint16)
    tr = {}
    out = layer.forward(x, tr)
    data = {"x0": x, "out": np.asarray(out, dtype=np.uint16), "g1": layer.g1, "g2": layer.g2, "cos": layer.cos, "sin": layer.sin}
    for name, (codes, sc) in zip("qkvogud", (layer.Wq, layer.Wk, layer.Wv, layer.Wo, layer.Wg, layer.Wu, layer.Wd)):
        data["w%s_codes" % name] = codes.astype(np.uint8)
        data["w%s_scales" % name] = sc.view(np.uint32)
    for k, v in tr.items():
        data["trace_" + k] = np.asarray(v, dtype=np.uint16)
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "tf_tiny_layer.npz"), **data)
    print("wrote", sorted(data))


if __name__ == "__main__":
    _repo = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    main(sys.argv[1] if len(sys.argv) > 1 else
         os.path.join(os.environ.get("ZKH_REFERENCE") or os.path.join(os.path.dirname(_repo), "reference"), "zkllm-src"))
