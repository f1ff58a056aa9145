"""A device-side wait that runs out returns a status, it does not hang (nothing faults, nothing
spins without a bound).

A loopback group (dp_tp_init_loopback) gives rank 0 of a two-rank group two exchange areas that
both live on this GPU; nobody ever raises rank 1's flag.  With the poll limit set small, every
grid barrier that expects rank 1 gives up after that many polls, the kernels finish, and the decode
call reports DP_ERR_TIMEOUT; the context then runs other work normally."""
import ctypes as C

import numpy as np
import pytest

from doppler_b200 import _lib as L
from doppler_b200 import ops, synthetic
from doppler_b200.model import DecoderModel
from doppler_b200.ops import Device, DopplerError
from model_util import gaussian_model_weights
from oracle import oracle as O
from parity import assert_close

pytestmark = pytest.mark.gpu


def test_exchange_wait_runs_out_and_reports_timeout():
    dev = Device(0)
    try:
        dev.check(dev.lib.dp_ctx_set_wait_limit(dev.h, 10000))
        dev.check(dev.lib.dp_tp_init_loopback(dev.h, 0, 2))
        cfg = dict(synthetic.MODEL_CONFIGS["small"])
        m = DecoderModel(dev, cfg, max_seq=1024, tp_rank=0, tp_size=2)
        m.load_all(gaussian_model_weights(cfg, 5))
        m.set_allreduce_mode(1)
        with pytest.raises(DopplerError) as ei:
            m.decode([7], 2)  # rank 1 never shows up
        assert ei.value.status == L.ERR_TIMEOUT, ei.value
        # the stream is idle again and the status is cleared: the context is usable
        dev.sync()
        N, K = 512, 1024
        W = synthetic.q4k_matrix(synthetic.key(61, 0), N, K)
        x = synthetic.normal_f32(synthetic.key(61, 1), K)
        y = dev.read_tensor(ops.run_matmul(dev.tensor_from(x.reshape(1, K)), dev.weight_from(W, "q4k", [N, K]), 1, N, K, output_dtype="f32"))
        assert_close(y, O.q4k_gemv(W, N, K, x), "gemv after a timed-out decode")
        dev.sync()
        m.destroy()
    finally:
        dev.close()
