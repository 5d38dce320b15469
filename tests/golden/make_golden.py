"""Generates tests/golden/*.npz from the reference toolkit's OWN Cpu-device code.

Run in a container that has the reference checkout: `oracle/build_ref.sh` compiles the reference's
layer sources into oracle/_ref/libcurrennt_ref.so, and this script drives that library (kind="ref")
on small seeded cases and stores inputs, weights and every observable result: layer outputs, the
error (SSE), the output errors each layer received, all weight gradients, and the weights after
one steepest-descent update.  The fixtures pin both the C restatement (CPU tests) and the CUDA
kernels (GPU tests) to the reference.

    python tests/golden/make_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, os.path.join(ROOT, "oracle"))
sys.path.insert(0, os.path.join(ROOT, "project-currennt-public_b200"))
from oracle import OracleNet  # noqa: E402
from b2lstm import workloads  # noqa: E402


def L(*spec):
    return [dict(type=t, size=s, **({} if t in ("input", "sse") else {"bias": b})) for t, s, b in spec]


CASES = {
    # name: (layers, P, lens, target_scale, binary_dims)
    "lstm_equal": (L(("input", 5, 0), ("lstm", 8, 1.0), ("feedforward_identity", 3, 1.0), ("sse", 3, 0)), 3, [12, 12, 12], 1.0, 0),
    "blstm_ragged": (L(("input", 5, 0), ("blstm", 8, 1.0), ("feedforward_identity", 3, 1.0), ("sse", 3, 0)), 3, [12, 7, 3], 1.0, 0),
    "lstm_ragged_clip": (L(("input", 6, 0), ("lstm", 9, 1.0), ("feedforward_identity", 4, 1.0), ("sse", 4, 0)), 4, [20, 13, 20, 5], 300.0, 0),
    "blstm_ragged_clip": (L(("input", 6, 0), ("blstm", 10, 0.5), ("feedforward_identity", 4, 1.0), ("sse", 4, 0)), 3, [12, 12, 4], 300.0, 0),
    "blstm_single_seq": (L(("input", 4, 0), ("blstm", 6, 1.0), ("feedforward_identity", 2, 1.0), ("sse", 2, 0)), 1, [30], 1.0, 0),
    "short_fraction": (L(("input", 5, 0), ("blstm", 8, 1.0), ("feedforward_identity", 3, 1.0), ("sse", 3, 0)), 4, [9, 6], 1.0, 0),
    "one_unit_one_step": (L(("input", 3, 0), ("blstm", 2, 1.0), ("lstm", 1, 1.0), ("feedforward_identity", 2, 1.0), ("sse", 2, 0)), 2, [1, 1], 1.0, 0),
    "deep_mixed": (L(("input", 7, 0), ("feedforward_tanh", 9, 1.0), ("blstm", 12, 1.0), ("lstm", 5, 1.0), ("feedforward_logistic", 6, 1.0),
                     ("feedforward_identity", 3, 1.0), ("sse", 3, 0)), 4, [20, 9, 15], 1.0, 3),
    "odd_sizes_33": (L(("input", 33, 0), ("blstm", 66, 1.0), ("blstm", 34, 1.0), ("feedforward_identity", 5, 1.0), ("sse", 5, 0)), 3, [17, 17, 11], 1.0, 0),
    "cfg0_small": (L(("input", 64, 0), ("lstm", 128, 1.0), ("feedforward_identity", 32, 1.0), ("sse", 32, 0)), 4, [40, 40, 40, 40], 1.0, 0),
}


def run(kind, layers, P, lens, x, tg, weights, lr=1e-4, mom=0.9):
    net = OracleNet(layers, P, x.shape[0], kind)
    for i, w in weights.items():
        net.set_weights(i, w)
    net.load(lens, x, tg)
    out = {"loss": np.float64(net.forward())}
    net.backward()
    for i in range(len(layers)):
        out["out%d" % i] = net.outputs(i)
        if i and layers[i]["type"] != "sse":
            out["dyin%d" % i] = net.output_errors_in(i)
        if i in weights:
            out["dw%d" % i] = net.weight_updates(i)
    net.sgd_update(lr, mom)
    for i in weights:
        out["wnew%d" % i] = net.get_weights(i)
    net.close()
    return out


def main():
    for k, (name, (layers, P, lens, tscale, binary)) in enumerate(sorted(CASES.items())):
        lens = np.asarray(lens, np.int32)
        x, tg = workloads.make_fraction(layers[0]["size"], layers[-1]["size"], P, lens, 100 + k, 200 + k, binary, tscale)
        weights = workloads.make_weights(layers, 300 + k, 0.3 if "clip" in name else 0.08)
        res = run("ref", layers, P, lens, x, tg, weights)
        data = {"layers": np.array(json.dumps(layers)), "P": np.int32(P), "lens": lens, "x": x, "tg": tg}
        for i, w in weights.items():
            data["w%d" % i] = w
        data.update(res)
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **data)
        print("%-20s loss %.6g  %d bytes" % (name, res["loss"], os.path.getsize(path)))


if __name__ == "__main__":
    main()
