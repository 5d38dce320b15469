"""The binary weight dump (NeuralNetwork::printWeightMatrix of the reference): the restatement the GPU test compares
b2_net_save_weights_binary with is pinned here to the reference's own reader, pyTools/ioTools/nnio.py
ReadCURRENNTWeight, where a reference checkout lies beside the repository."""
import os
import sys

import numpy as np
import pytest

import parity

HERE = os.path.dirname(os.path.abspath(__file__))
PYTOOLS = os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference", "pyTools")


def L(*spec):
    return [dict(type=t, size=s, **({} if t in ("input", "sse") else {"bias": 1.0})) for t, s in spec]


LAYERS = L(("input", 7), ("feedforward_tanh", 12), ("blstm", 16), ("lstm", 9), ("feedforward_identity", 3), ("sse", 3))


def make_weights():
    rng = np.random.default_rng(3)
    w = {}
    for i, l in enumerate(LAYERS):
        if l["type"] in ("input", "sse"):
            continue
        pls, ls = LAYERS[i - 1]["size"], l["size"]
        if "lstm" in l["type"]:
            n = ls * (4 * (pls + 1) + (2 if l["type"] == "blstm" else 4) * ls + 3)
        else:
            n = ls * (pls + 1)
        w[i] = rng.standard_normal(n).astype(np.float32)
    return w


def test_layout_of_the_dump():
    w = make_weights()
    raw = np.frombuffer(parity.weight_dump_bytes(LAYERS, w), np.float32)
    assert raw[0] == 4 and raw.size == 1 + 4 * 5 + sum(v.size for v in w.values())
    assert list(raw[1:6]) == [w[1].size, 12, 7, 1, 0]
    assert list(raw[6:11]) == [w[2].size, 16, 12, 4, 2 * 16 + 3]
    assert list(raw[11:16]) == [w[3].size, 9, 16, 4, 4 * 9 + 3]
    assert np.array_equal(raw[21:21 + w[1].size], w[1])
    coded = np.frombuffer(parity.weight_dump_bytes(LAYERS, w, with_type_codes=True), np.float32)
    assert coded.size == raw.size + 4 and [coded[6], coded[12], coded[18], coded[24]] == [0, 5, 4, 2]


@pytest.mark.skipif(not os.path.isdir(PYTOOLS), reason="no reference checkout beside the repository")
def test_the_reference_reader_parses_the_dump(tmp_path):
    sys.path.insert(0, PYTOOLS)
    try:
        import warnings
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            from ioTools import nnio
    finally:
        sys.path.remove(PYTOOLS)
    w = make_weights()
    path = str(tmp_path / "weights.bin")
    with open(path, "wb") as f:
        f.write(parity.weight_dump_bytes(LAYERS, w))
    mats = nnio.ReadCURRENNTWeight(path)
    assert len(mats) == 4
    for (W, b, inter), i in zip(mats, sorted(w)):
        l, pls = LAYERS[i], LAYERS[i - 1]["size"]
        per = 4 if "lstm" in l["type"] else 1
        n_in, n_b = l["size"] * per * pls, l["size"] * per
        assert W.shape == (per * l["size"], pls) and np.array_equal(W.ravel(), w[i][:n_in])
        assert np.array_equal(np.asarray(b).ravel(), w[i][n_in:n_in + n_b])
        assert np.array_equal(np.asarray(inter).ravel(), w[i][n_in + n_b:])
