"""CPU tests of the checker itself: the C restatement against the golden tensors produced by the
reference's own Cpu code, against that code directly where it is present, and known answers."""
import numpy as np
import pytest

import parity
from oracle import OracleNet, ref_available
from make_golden import run as run_kind


@pytest.mark.parametrize("name", parity.golden_cases())
def test_port_reproduces_reference_golden(name):
    g = parity.load_golden(name)
    got = run_kind("port", g["layers"], g["P"], g["lens"], g["x"], g["tg"], g["weights"])
    # same arithmetic in the same order: exact up to the libm used for expf
    for k, v in got.items():
        np.testing.assert_allclose(v, g[k], rtol=2e-6, atol=1e-7, err_msg="%s %s" % (name, k))
    parity.compare_run(g["layers"], got, g, name, lstm_pad_zero_lens=g["lens"])


@pytest.mark.parametrize("name", ["blstm_ragged_clip", "deep_mixed"])
def test_fp64_arbiter_close_to_reference(name):
    g = parity.load_golden(name)
    got = run_kind("port64", g["layers"], g["P"], g["lens"], g["x"], g["tg"], g["weights"])
    parity.compare_run(g["layers"], got, g, name + " fp64")


@pytest.mark.skipif(not ref_available(), reason="compiled reference library not present")
def test_port_matches_compiled_reference_on_fresh_inputs():
    from b2lstm import workloads
    layers = [dict(type="input", size=11), dict(type="blstm", size=14, bias=1.0), dict(type="lstm", size=7, bias=0.7),
              dict(type="feedforward_tanh", size=6, bias=1.0), dict(type="feedforward_identity", size=4, bias=1.0),
              dict(type="sse", size=4)]
    P, lens = 5, np.array([23, 23, 16, 9, 2], np.int32)
    x, tg = workloads.make_fraction(11, 4, P, lens, 7, 8, binary_dims=4, target_scale=20.0)
    w = workloads.make_weights(layers, 9, 0.2)
    a = run_kind("port", layers, P, lens, x, tg, w)
    b = run_kind("ref", layers, P, lens, x, tg, w)
    for k in b:
        np.testing.assert_allclose(a[k], b[k], rtol=2e-6, atol=1e-7, err_msg=k)


def test_weight_count_known_answers():
    # counts printed by the reference for real networks (its shipped example logs):
    # blstm 256 after a 512-wide layer -> 657152, blstm 10 after 382 inputs -> 15550,
    # feedforward 382 -> 512 -> 196096, feedforward 256 -> 259 -> 66563
    from b2lstm import workloads
    assert workloads.lstm_num_weights(512, 256, True) == 657152
    assert workloads.lstm_num_weights(382, 10, True) == 15550
    L = [dict(type="input", size=382), dict(type="feedforward_tanh", size=512)]
    assert workloads.layer_num_weights(L, 1) == 196096
    L = [dict(type="input", size=256), dict(type="feedforward_identity", size=259)]
    assert workloads.layer_num_weights(L, 1) == 66563
    net = OracleNet([dict(type="input", size=512), dict(type="blstm", size=256), dict(type="sse", size=256)], 1, 1, "port")
    assert net.num_weights(1) == 657152


def test_sgd_update_zeroes_nan_gradients():
    layers = [dict(type="input", size=2), dict(type="feedforward_identity", size=2, bias=1.0), dict(type="sse", size=2)]
    net = OracleNet(layers, 1, 1, "port")
    net.set_weights(1, np.ones(6, np.float32))
    x = np.array([[[np.nan, 1.0]]], np.float32)
    net.load(np.array([1], np.int32), x, np.zeros((1, 1, 2), np.float32))
    net.forward()
    net.backward()
    assert np.isnan(net.weight_updates(1)).any()
    net.sgd_update(0.1, 0.0)
    w = net.get_weights(1)
    assert np.isfinite(w).all()
