"""Committed fixtures (tests/golden/, made by make_golden.py): the oracle must reproduce them
on CPU, and the CUDA kernels must match them on the GPU."""
import json
import os

import numpy as np
import pytest

from doppler_b200 import synthetic
from model_util import gaussian_model_weights
from oracle import oracle as O
from parity import assert_close

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _g():
    return np.load(os.path.join(GOLDEN, "kernels.npz"))


def test_oracle_reproduces_fixtures():
    g = _g()
    assert np.array_equal(synthetic.q4k_blocks(synthetic.key(2024, 1), 6), g["blocks"])  # generator is stable
    assert np.array_equal(O.q4k_dequant_flat(g["blocks"], 1536).view(np.uint32), g["blocks_dequant"].view(np.uint32))
    assert np.array_equal(O.q4k_gemv(g["W"], 48, 512, g["x"]).view(np.uint32), g["gemv"].view(np.uint32))
    assert np.array_equal(O.q4k_gemm(g["W"], 48, 512, g["A"], 3).view(np.uint32), g["gemm"].view(np.uint32))
    a = O.attention_f16kv(g["q"], g["k16"].view(np.float16), g["v16"].view(np.float16), 1, 40, 4, 2, 64, causal=False)
    assert np.array_equal(a.view(np.uint32), g["attn"].view(np.uint32))
    assert np.array_equal(O.lcg_test_data(512, 1001), g["ref_suite_vals"])
    assert np.array_equal(O.q4k_quantize_flat(g["ref_suite_vals"]), g["ref_suite_q4k"])


def test_oracle_model_reproduces_token_fixture():
    g = json.load(open(os.path.join(GOLDEN, "model_tokens.json")))
    cfg = dict(synthetic.MODEL_CONFIGS[g["config"]], max_seq=g["max_seq"])
    om = O.OracleModel(cfg, gaussian_model_weights(cfg, g["seed"]))
    tok, _ = om.forward(np.array(g["prompt"], np.int32))
    toks = [tok]
    for _ in range(12):
        tok, _ = om.forward([tok])
        toks.append(tok)
    assert toks == g["tokens"][:13]


@pytest.mark.gpu
def test_kernels_match_fixtures(dev):
    from doppler_b200 import ops
    g = _g()
    buf = dev.acquire_buffer(g["blocks"].nbytes, "blocks")
    dev.upload_data(buf, g["blocks"])
    t = ops.dequantize(buf, 6)
    assert np.array_equal(dev.read_tensor(t).view(np.uint32), g["blocks_dequant"].view(np.uint32))
    wb = dev.weight_from(g["W"], "q4k", [48, 512])
    xt = dev.tensor_from(g["x"].reshape(1, 512))
    y = ops.run_matmul(xt, wb, 1, 48, 512, output_dtype="f32")
    assert_close(dev.read_tensor(y), g["gemv"], "fixture gemv")
    at = dev.tensor_from(g["A"].reshape(3, 512))
    c = ops.run_matmul(at, wb, 3, 48, 512, output_dtype="f32", exact_weights=True)
    assert_close(dev.read_tensor(c), g["gemm"], "fixture gemm")
    qt = dev.tensor_from(g["q"])
    kt, vt = dev.tensor_from(g["k16"].view(np.float16)), dev.tensor_from(g["v16"].view(np.float16))
    o = ops.run_attention(qt, kt, vt, None, 4, 64, kv_len=40, num_kv_heads=2, causal=False)
    assert_close(dev.read_tensor(o), g["attn"], "fixture attention")
    for x in (t, y, c, o, xt, at, qt, kt, vt, wb):
        dev.release_buffer(x.buffer)
    dev.release_buffer(buf)
