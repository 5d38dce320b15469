"""Parity metric shared by the CPU and GPU tests.

layer outputs:     |a - b| <= 1e-6 + 1e-5 |b| element-wise (padding frames of (b)lstm layers are exactly 0)
weight gradients:  per block (input, bias, recurrent, peephole): ||a-b||2 / ||b||2 <= 1e-4 and
                   max|a-b| <= 1e-4 max|b|
output errors:     the same relative bound as the gradients
`b` is always the reference side.
"""
import glob
import json
import os

import numpy as np

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
OUT_ATOL, OUT_RTOL, GRAD_RTOL = 1e-6, 1e-5, 1e-4


def golden_cases():
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, "*.npz")))


def load_golden(name):
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    d = {k: z[k] for k in z.files}
    d["layers"] = json.loads(str(d["layers"]))
    d["P"] = int(d["P"])
    d["weights"] = {int(k[1:]): d[k] for k in z.files if k[0] == "w" and k[1:].isdigit()}
    return d


def assert_outputs_close(a, b, what, atol=OUT_ATOL, rtol=OUT_RTOL):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    assert a.shape == b.shape, (what, a.shape, b.shape)
    assert np.isfinite(a).all(), what + ": non-finite values"
    bad = np.abs(a - b) > atol + rtol * np.abs(b)
    if bad.any():
        i = np.unravel_index(np.argmax(np.abs(a - b) - rtol * np.abs(b)), a.shape)
        raise AssertionError("%s: %d of %d elements outside %.0e+%.0e|b|; worst at %s: got %.9g want %.9g"
                             % (what, bad.sum(), a.size, atol, rtol, i, a[i], b[i]))


def assert_rel_close(a, b, what, rtol=GRAD_RTOL):
    a = np.asarray(a, np.float64).ravel()
    b = np.asarray(b, np.float64).ravel()
    assert a.shape == b.shape, (what, a.shape, b.shape)
    assert np.isfinite(a).all(), what + ": non-finite values"
    nb = np.linalg.norm(b)
    if nb == 0:
        assert np.abs(a).max(initial=0.0) <= 1e-7, what + ": reference is all zero, got non-zero"
        return
    rel = np.linalg.norm(a - b) / nb
    mx = np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)
    assert rel <= rtol and mx <= rtol, "%s: rel L2 %.3g, max-abs ratio %.3g (limit %.0e)" % (what, rel, mx, rtol)


def weight_blocks(layers, i):
    """{block name: slice} of layer i's weight vector, per direction for (b)lstm layers."""
    ty, ls, pls = layers[i]["type"], layers[i]["size"], layers[i - 1]["size"]
    if ty.startswith("feedforward"):
        return {"input": slice(0, ls * pls), "bias": slice(ls * pls, ls * pls + ls)}
    bi = ty == "blstm"
    els = ls // 2 if bi else ls
    o_b, o_r, o_p = 4 * ls * pls, 4 * ls * (pls + 1), 4 * ls * (pls + 1) + 4 * ls * els
    blocks = {}
    for d in range(2 if bi else 1):
        idx_in, idx_b, idx_r, idx_p = [], [], [], []
        for g in range(4):
            idx_in.append(np.arange(g * ls * pls + d * els * pls, g * ls * pls + (d + 1) * els * pls))
            idx_b.append(np.arange(o_b + g * ls + d * els, o_b + g * ls + (d + 1) * els))
            idx_r.append(np.arange(o_r + g * ls * els + d * els * els, o_r + g * ls * els + (d + 1) * els * els))
        for q in range(3):
            idx_p.append(np.arange(o_p + q * ls + d * els, o_p + q * ls + (d + 1) * els))
        blocks["input/dir%d" % d] = np.concatenate(idx_in)
        blocks["bias/dir%d" % d] = np.concatenate(idx_b)
        blocks["recurrent/dir%d" % d] = np.concatenate(idx_r)
        blocks["peephole/dir%d" % d] = np.concatenate(idx_p)
    return blocks


def assert_grads_close(layers, i, a, b, what):
    for name, sl in weight_blocks(layers, i).items():
        assert_rel_close(a[sl], b[sl], "%s layer %d %s" % (what, i, name))


def compare_run(layers, got, want, what, lstm_pad_zero_lens=None, P=None, loss_rtol=1e-5):
    """got/want: dicts with loss, out<i>, dyin<i>, dw<i> (want may hold more keys)."""
    assert abs(got["loss"] - want["loss"]) <= loss_rtol * abs(want["loss"]) + 1e-6, (what, got["loss"], want["loss"])
    for i in range(1, len(layers)):
        if layers[i]["type"] == "sse":
            continue
        assert_outputs_close(got["out%d" % i], want["out%d" % i], "%s outputs of layer %d" % (what, i))
        if "dyin%d" % i in got:
            assert_rel_close(got["dyin%d" % i], want["dyin%d" % i], "%s output errors into layer %d" % (what, i))
        if "dw%d" % i in got:
            assert_grads_close(layers, i, got["dw%d" % i], want["dw%d" % i], what)
        if lstm_pad_zero_lens is not None and layers[i]["type"] in ("lstm", "blstm"):
            o = got["out%d" % i]
            for p in range(o.shape[1]):
                Lp = lstm_pad_zero_lens[p] if p < len(lstm_pad_zero_lens) else 0
                # padding frames at or beyond the shortest sequence's length are forced to exact zero
                t0 = max(Lp, min(lstm_pad_zero_lens))
                assert not o[t0:, p].any(), "%s layer %d: non-zero output on padding of sequence %d" % (what, i, p)


def weight_dump_bytes(layers, weights, with_type_codes=False):
    """The file NeuralNetwork::printWeightMatrix writes (NeuralNetwork.cpp:3792-3880 of the reference), restated: native
    floats; the number of layers with weights, per layer {weights, size, preceding size, input weights per block, internal
    weights per block [, type code]}, then the weight vectors.  `weights`: {layer index: flat float32 array}."""
    codes = {"feedforward_tanh": 0, "feedforward_logistic": 1, "feedforward_identity": 2, "feedforward_relu": 3, "lstm": 4, "blstm": 5}
    head, body = [], []
    for i, l in enumerate(layers):
        if i not in weights:
            continue
        lstm = l["type"] in ("lstm", "blstm")
        in_per_block = 4 if lstm else 1
        internal = ((2 if l["type"] == "blstm" else 4) * l["size"] + 3) if lstm else 0
        w = np.asarray(weights[i], np.float32)
        assert w.size == l["size"] * (in_per_block * (layers[i - 1]["size"] + 1) + internal)
        head += [w.size, l["size"], layers[i - 1]["size"], in_per_block, internal]
        if with_type_codes:
            head.append(codes[l["type"]])
        body.append(w)
    n = len(body)
    return np.concatenate([np.array([n] + head, np.float32)] + body).tobytes()
