"""Regenerates the committed fixtures under tests/golden/ from the CPU oracle.

    python tests/golden/make_golden.py

Inputs come from the seeded generators of the library (doppler_b200.synthetic) and from the
reference's own LCG test-data generator; outputs are what the oracle computes for them.

    python tests/golden/make_golden.py --receipt <reference checkout>

copies the reference-held fixture of its 9B gate_proj receipt
(reports/qwen-3-5-9b-metal/2026-07-12/layer0-ffn-gate-oracle/: block-d.f32, block-dmin.f32,
packed-scale-bits.u8, packed-min-bits.u8) into receipt_9b_gate_headers.npz, together with the
sha256 digests the receipt JSON records for the decoded scales and minima the reference computed
from them (artifactFiles.decodedScales / decodedMinima).  Those digests are reference-produced
numbers: tests/test_oracle_pins.py and tests/test_gpu_dequant.py hash what the oracle and the
CUDA dequant kernel decode from the same headers and compare.  The same call copies two manifests of
the reference's model catalog (models/local/<id>/manifest.json) for tests/test_rdrr.py.
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


def receipt(ref_root):
    base = os.path.join(ref_root, "reports", "qwen-3-5-9b-metal", "2026-07-12")
    folder = os.path.join(base, "layer0-ffn-gate-oracle")
    meta = json.load(open(os.path.join(base, "layer0-ffn-gate-oracle.json")))
    d = np.fromfile(os.path.join(folder, "block-d.f32"), np.float32)
    dmin = np.fromfile(os.path.join(folder, "block-dmin.f32"), np.float32)
    sc = np.fromfile(os.path.join(folder, "packed-scale-bits.u8"), np.uint8)
    mn = np.fromfile(os.path.join(folder, "packed-min-bits.u8"), np.uint8)
    d16, dmin16 = d.astype(np.float16), dmin.astype(np.float16)
    # the receipt stores the f16 block scales widened to f32: the narrowing is exact
    assert np.array_equal(d16.astype(np.float32), d) and np.array_equal(dmin16.astype(np.float32), dmin)
    assert sc.size == mn.size == 8 * d.size and int(sc.max()) < 64 and int(mn.max()) < 64
    files = meta["artifactFiles"]
    np.savez_compressed(
        os.path.join(HERE, "receipt_9b_gate_headers.npz"),
        d_f16=d16.view(np.uint16), dmin_f16=dmin16.view(np.uint16), scale_codes=sc, min_codes=mn,
        shape=np.array(meta["artifacts"]["q4"]["tensorDescriptor"]["shape"], np.int64),
        decoded_scales_sha256=np.array(files["decodedScales"]["sha256"]),
        decoded_minima_sha256=np.array(files["decodedMinima"]["sha256"]),
    )
    print("wrote receipt_9b_gate_headers.npz:", d.size, "blocks")


def manifests(ref_root):
    """Two manifests of the reference's model catalog (models/local/*/manifest.json), gzip'd as they are."""
    import gzip

    for name in ("qwen-3-embedding-0-6b-q4k-ehf16-af32", "qwen-3-5-0-8b-q4k-ehaf16"):
        raw = open(os.path.join(ref_root, "models", "local", name, "manifest.json"), "rb").read()
        with gzip.GzipFile(os.path.join(HERE, "manifest__" + name + ".json.gz"), "wb", mtime=0) as f:
            f.write(raw)
        print("wrote manifest__%s.json.gz (%d bytes of JSON)" % (name, len(raw)))


if __name__ == "__main__":
    if "--receipt" in sys.argv:
        receipt(sys.argv[sys.argv.index("--receipt") + 1])
        manifests(sys.argv[sys.argv.index("--receipt") + 1])
    else:
        main()
