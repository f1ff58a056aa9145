"""Test helper: a random-init model whose Q4_K matrices are QUANTISED GAUSSIANS (zero-mean
weights, quantised with the oracle's restatement of the reference quantizer).  Unlike the
uniform-random blocks of the benchmark generator this keeps activations moderate, so greedy
decoding visits many different tokens and token identity is a discriminating check."""
import numpy as np

from doppler_b200 import synthetic
from oracle import oracle as O


def gaussian_model_weights(cfg: dict, seed: int) -> dict:
    shapes = synthetic.layer_shapes(cfg)
    layers = []
    for l in range(cfg["n_layers"]):
        lw = {}
        for j, (name, (n, k)) in enumerate(shapes.items()):
            w = synthetic.normal_f32(synthetic.key(seed, 5000 + l * 16 + j), n * k, sigma=1.0 / np.sqrt(k))
            lw[name] = O.q4k_quantize_rowwise(w, n, k)
        for j, name in enumerate(("in_norm", "post_norm", "q_norm", "k_norm")):
            size = cfg["head_dim"] if name in ("q_norm", "k_norm") else cfg["hidden"]
            lw[name] = synthetic.normal_f32(synthetic.key(seed, 5000 + l * 16 + 8 + j), size, 0.1, 1.0)
        layers.append(lw)
    return {
        "layers": layers,
        "embed": synthetic.normal_f16(synthetic.key(seed, 4001), cfg["vocab"] * cfg["hidden"], 1.0).reshape(cfg["vocab"], cfg["hidden"]),
        "lm_head": synthetic.normal_f16(synthetic.key(seed, 4002), cfg["vocab"] * cfg["hidden"], 0.05).reshape(cfg["vocab"], cfg["hidden"]),
        "final_norm": synthetic.normal_f32(synthetic.key(seed, 4003), cfg["hidden"], 0.1, 1.0),
    }
