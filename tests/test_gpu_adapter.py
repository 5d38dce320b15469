"""The drop-in claim, compiled and run: layers::LstmLayerB200<Gpu> (project-currennt-public_b200/adapter/
LstmLayerB200.hpp), built against the reference toolkit's own headers by oracle/build_ref.sh, takes the place of
layers::LstmLayer<Gpu> with the constructor signature LayerFactory.cu:127-132 uses, between the reference's own
InputLayer<Gpu>, FeedForwardLayer<Gpu, *> and SsePostOutputLayer<Gpu>.  The whole chain runs one fraction on the
GPU (the reference's Thrust and cuBLAS code on either side of the library, on the toolkit's device vectors) and is
compared with the reference's Cpu chain, LstmLayer<Cpu> included."""
import numpy as np
import pytest

import parity
from make_golden import run as run_kind
from oracle import ref_available

pytestmark = pytest.mark.gpu


def L(*spec):
    return [dict(type=t, size=s, **({} if t in ("input", "sse") else {"bias": 1.0})) for t, s in spec]


@pytest.mark.parametrize("layers,P,lens", [
    (L(("input", 6), ("blstm", 16), ("feedforward_identity", 3), ("sse", 3)), 3, [9, 5, 9]),
    (L(("input", 5), ("feedforward_tanh", 7), ("lstm", 9), ("blstm", 12), ("feedforward_identity", 4), ("sse", 4)), 4, [12, 12, 7, 3]),
    (L(("input", 12), ("blstm", 1024), ("feedforward_identity", 5), ("sse", 5)), 16, [10] * 12 + [7, 5, 3, 2]),
    (L(("input", 12), ("blstm", 512), ("feedforward_identity", 5), ("sse", 5)), 6, [14, 14, 11, 9, 4, 2]),
])
def test_reference_gpu_chain_with_the_adapter_in_place_of_its_lstm_layer(layers, P, lens):
    if not (ref_available() and ref_available(adapter=True)):
        pytest.skip("the reference libraries (oracle/_ref) did not travel with the repository")
    from b2lstm import workloads
    lens = np.array(lens, np.int32)
    x, tg = workloads.make_fraction(layers[0]["size"], layers[-1]["size"], P, lens, 71, 72)
    w = workloads.make_weights(layers, 73, 0.1)
    want = run_kind("ref", layers, P, lens, x, tg, w)
    got = run_kind("ref_b200", layers, P, lens, x, tg, w)
    parity.compare_run(layers, got, want, "reference Gpu chain + LstmLayerB200", lstm_pad_zero_lens=lens)
    for i in w:   # the reference's own update on the adapter's gradients
        parity.assert_rel_close(got["wnew%d" % i] - w[i], want["wnew%d" % i] - w[i], "weight step of layer %d" % i)
