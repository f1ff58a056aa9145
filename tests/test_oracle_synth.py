"""The oracle's restatement of the seeded input generators (orc_synth_*) produces the same bytes
as the library's host utilities (dp_synth_*): the CPU baseline builds the benchmark model from the
former without loading the CUDA library, and both must describe the same model."""
import numpy as np

from doppler_b200 import synthetic
from oracle import oracle as O


def test_generators_agree_byte_for_byte():
    ours, theirs = synthetic.Generator(), synthetic.Generator(O.SynthBackend())
    for seed, tid in ((synthetic.DEFAULT_SEED, 1), (7, 1003), (2**63 + 5, 4)):
        ka, kb = ours.key(seed, tid), theirs.key(seed, tid)
        assert ka == kb
        assert np.array_equal(ours.normal_f32(ka, 100003, 0.1, 1.0, first=17).view(np.uint32),
                              theirs.normal_f32(kb, 100003, 0.1, 1.0, first=17).view(np.uint32))
        assert np.array_equal(ours.normal_f16(ka, 70001, 0.02, first=5).view(np.uint16), theirs.normal_f16(kb, 70001, 0.02, first=5).view(np.uint16))
        assert np.array_equal(ours.q4k_blocks(ka, 4099, first_block=3), theirs.q4k_blocks(kb, 4099, first_block=3))
        assert np.array_equal(ours.tokens(ka, 999, 151936), theirs.tokens(kb, 999, 151936))


def test_model_builders_agree():
    cfg = dict(synthetic.MODEL_CONFIGS["tiny"])
    a = synthetic.make_model_weights(cfg, 5)
    b = synthetic.make_model_weights(cfg, 5, gen=synthetic.Generator(O.SynthBackend()))
    for la, lb in zip(a["layers"], b["layers"]):
        for k in la:
            assert np.array_equal(la[k].view(np.uint8), lb[k].view(np.uint8)), k
    for k in ("embed", "lm_head", "final_norm"):
        assert np.array_equal(a[k].view(np.uint8), b[k].view(np.uint8)), k
    assert np.array_equal(synthetic.make_prompt(cfg, 33, 5, seq=2), synthetic.make_prompt(cfg, 33, 5, seq=2, gen=synthetic.Generator(O.SynthBackend())))
