"""The fallback switches (environment variables read once per process, one per op) select the alternative kernels.
Each alternative must stay correct, so a small parity check runs in a child process per setting."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import os, sys
sys.path.insert(0, os.environ["DP_ROOT"]); sys.path.insert(0, os.path.join(os.environ["DP_ROOT"], "tests"))
import numpy as np
from doppler_b200 import ops, synthetic
from doppler_b200.model import DecoderModel
from model_util import gaussian_model_weights
from oracle import oracle as O
from parity import assert_close
dev = ops.Device(0)
for (N, K) in [(3072, 1024), (4096, 4096), (1024, 12288)]:
    W = synthetic.q4k_matrix(synthetic.key(81, N), N, K)
    x = synthetic.normal_f32(synthetic.key(82, K), K)
    y = dev.read_tensor(ops.run_matmul(dev.tensor_from(x.reshape(1, K)), dev.weight_from(W, "q4k", [N, K]), 1, N, K, output_dtype="f32"))
    assert_close(y, O.q4k_gemv(W, N, K, x), f"gemv [{N},{K}]")
M, N, K = 512, 768, 512
W = synthetic.q4k_matrix(synthetic.key(83, 1), N, K)
A = synthetic.normal_f16(synthetic.key(83, 2), M * K)
c = dev.read_tensor(ops.run_matmul(dev.tensor_from(A.reshape(M, K)), dev.weight_from(W, "q4k", [N, K]), M, N, K, output_dtype="f32"))
assert_close(c, O.q4k_gemm(W, N, K, A.astype(np.float32), M), "gemm")
cfg = dict(synthetic.MODEL_CONFIGS["small"])
w = gaussian_model_weights(cfg, 1234)
prompt = synthetic.make_prompt(cfg, 40, seed=1234)
m = DecoderModel(dev, cfg, max_seq=1024)
m.load_all(w)
first = m.prefill(prompt)
out = m.decode([first], 24)[:, 0].tolist()
om = O.OracleModel(dict(cfg, max_seq=1024), w)
tok, _ = om.forward(prompt)
exp, cur = [], tok
for _ in range(24):
    cur, _ = om.forward([cur]); exp.append(cur)
assert first == tok and out == exp, (first, out, tok, exp)
print("ok")
'''


@pytest.mark.parametrize("env", [
    {"DP_GEMV_VARIANT": "0"}, {"DP_ATTN_TC": "0"}, {"DP_PDL": "0"}, {"DP_GEMM_TC": "0"}, {"DP_PREFILL_TC": "0"},
], ids=lambda e: ",".join(f"{k}={v}" for k, v in e.items()))
def test_alternative_kernels_stay_correct(tmp_path, env):
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    p = subprocess.run([sys.executable, str(script)], env=dict(os.environ, DP_ROOT=ROOT, **env), capture_output=True, text=True,
                       timeout=240)
    assert p.returncode == 0 and "ok" in p.stdout, (env, p.stdout[-1500:], p.stderr[-1500:])
