"""Token identity at the BASELINE model sizes (full vocabulary of 151,936, real layer shapes).

  config 3: the whole Qwen3-0.6B-shaped decoder (28 layers, hidden 1024, 16/8 heads, MLP 3072);
  config 4: the 9B shape (hidden 4096, 32/8 heads, MLP 12288) cut to two layers so that the CPU
            oracle finishes in about a minute, at batch 1 and at batch 64 (the oracle of a batch
            is that many independent single-sequence runs: the reference decodes one sequence).

Weights are quantised zero-mean gaussians (see model_util.py), so decoding visits many tokens.
Gate: every greedy token equals the oracle's; prefill logits within the float gate."""
import numpy as np
import pytest

from doppler_b200 import synthetic
from doppler_b200.model import DecoderModel
from model_util import gaussian_model_weights
from oracle import oracle as O
from parity import assert_close

pytestmark = pytest.mark.gpu


def _identity(dev, cfg, w, prompt, steps, max_seq, what):
    m = DecoderModel(dev, cfg, max_seq=max_seq)
    m.load_all(w)
    first = m.prefill(prompt)
    logits_gpu = m.read_logits()
    om = O.OracleModel(dict(cfg, max_seq=max_seq), w)
    tok, margin, logits_cpu = om.forward(prompt, want_logits=True)
    assert_close(logits_gpu, logits_cpu, f"{what}: prefill logits")
    assert first == tok, f"{what}: prefill token {first} vs oracle {tok} (oracle margin {margin:.3e})"
    out = m.decode([first], steps)[:, 0]
    m.destroy()
    cur = tok
    for s in range(steps):
        cur, margin = om.forward([cur])
        assert int(out[s]) == cur, f"{what}: step {s}: GPU token {int(out[s])} vs oracle {cur} (oracle margin {margin:.3e})"
    assert len(set(out.tolist())) > steps // 4, "decoding collapsed; the identity check would be vacuous"


def test_config3_whole_model_64_tokens(dev):
    cfg = dict(synthetic.MODEL_CONFIGS["qwen3-0.6b"])
    w = gaussian_model_weights(cfg, 3003)
    prompt = synthetic.make_prompt(cfg, 96, seed=3003)
    _identity(dev, cfg, w, prompt, 64, 256, "config 3 (0.6B shape, 28 layers, vocab 151936)")


@pytest.fixture(scope="module")
def nine_b_two_layers():
    cfg = dict(synthetic.MODEL_CONFIGS["9b"], n_layers=2)
    return cfg, gaussian_model_weights(cfg, 4004)


def test_config4_shape_batch1_64_tokens(dev, nine_b_two_layers):
    cfg, w = nine_b_two_layers
    prompt = synthetic.make_prompt(cfg, 48, seed=4004)
    _identity(dev, cfg, w, prompt, 64, 128, "config 4 shape (9B, 2 layers, vocab 151936), batch 1")


@pytest.mark.parametrize("B", [64, 12])
def test_config4_shape_batch64(dev, nine_b_two_layers, B):
    """Batch 64 (BASELINE config 4) and batch 12: up to 32 rows the runner folds RMSNorm, silu(gate)*up and the
    residual adds into the small-batch projections, beyond it launches them as kernels of their own."""
    cfg, w = nine_b_two_layers
    steps, max_seq = 12, 32
    lens = [2 + (i * 5) % 8 for i in range(B)]
    m = DecoderModel(dev, cfg, max_seq=max_seq, max_batch=B)
    m.load_all(w)
    prompts = [synthetic.make_prompt(cfg, n, seed=4004, seq=i) for i, n in enumerate(lens)]
    firsts = [m.prefill(p, seq=i) for i, p in enumerate(prompts)]
    out = m.decode(firsts, steps)  # [steps, batch]
    m.destroy()
    seen = set()
    for i, p in enumerate(prompts):
        om = O.OracleModel(dict(cfg, max_seq=max_seq), w)
        tok, margin = om.forward(p)
        assert firsts[i] == tok, f"sequence {i}: prefill token {firsts[i]} vs oracle {tok} (margin {margin:.3e})"
        cur = tok
        for s in range(steps):
            cur, margin = om.forward([cur])
            assert int(out[s, i]) == cur, f"sequence {i} step {s}: {int(out[s, i])} vs oracle {cur} (margin {margin:.3e})"
            seen.add(cur)
    assert len(seen) > B, "the sequences collapsed onto a few tokens; the identity check would be vacuous"
