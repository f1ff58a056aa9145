"""Regenerates the committed fixtures under tests/golden/ from the CPU oracle.

    python tests/golden/make_golden.py

Inputs come from the seeded generators of the library (doppler_b200.synthetic) and from the
reference's own LCG test-data generator; outputs are what the oracle computes for them.
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))

from doppler_b200 import synthetic  # noqa: E402
from model_util import gaussian_model_weights  # noqa: E402
from oracle import oracle as O  # noqa: E402


def main():
    # kernels
    blocks = synthetic.q4k_blocks(synthetic.key(2024, 1), 6)
    N, K = 48, 512
    W = synthetic.q4k_matrix(synthetic.key(2024, 2), N, K)
    x = synthetic.normal_f32(synthetic.key(2024, 3), K)
    A = synthetic.normal_f32(synthetic.key(2024, 4), 3 * K)
    H, Hkv, D, kv = 4, 2, 64, 40
    q = synthetic.normal_f32(synthetic.key(2024, 5), H * D)
    k16 = synthetic.normal_f16(synthetic.key(2024, 6), kv * Hkv * D)
    v16 = synthetic.normal_f16(synthetic.key(2024, 7), kv * Hkv * D)
    ref_vals = O.lcg_test_data(512, 1001)
    ref_q = O.q4k_quantize_flat(ref_vals)
    np.savez_compressed(
        os.path.join(HERE, "kernels.npz"),
        blocks=blocks, blocks_dequant=O.q4k_dequant_flat(blocks, 6 * 256),
        W=W, x=x, gemv=O.q4k_gemv(W, N, K, x), A=A, gemm=O.q4k_gemm(W, N, K, A, 3),
        q=q, k16=k16.view(np.uint16), v16=v16.view(np.uint16),
        attn=O.attention_f16kv(q, k16, v16, 1, kv, H, Hkv, D, causal=False),
        ref_suite_vals=ref_vals, ref_suite_q4k=ref_q, ref_suite_dequant=O.q4k_dequant_flat(ref_q, 512),
    )
    # model tokens
    name, seed, prompt_len, steps, max_seq = "tiny", 4321, 20, 64, 128
    cfg = dict(synthetic.MODEL_CONFIGS[name], max_seq=max_seq)
    w = gaussian_model_weights(cfg, seed)
    prompt = synthetic.make_prompt(cfg, prompt_len, seed=seed)
    om = O.OracleModel(cfg, w)
    tok, margin = om.forward(prompt)
    toks, margins = [tok], [margin]
    for _ in range(steps):
        tok, margin = om.forward([tok])
        toks.append(tok)
        margins.append(margin)
    json.dump({"config": name, "seed": seed, "prompt_len": prompt_len, "max_seq": max_seq, "prompt": prompt.tolist(),
               "tokens": toks, "min_margin": float(min(margins))}, open(os.path.join(HERE, "model_tokens.json"), "w"))
    print("wrote fixtures; min top1-top2 margin", min(margins))


if __name__ == "__main__":
    main()
