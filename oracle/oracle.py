"""TEST INFRASTRUCTURE ONLY.  ctypes front-end over the two checkers of the LSTM training path:

* kind="ref" / "ref_omp": the reference toolkit's own Cpu-device layer classes, compiled from
  the reference sources by oracle/build_ref.sh into oracle/_ref/ (serial / OpenMP Thrust host
  backend).  Available only where that library has been built.
* kind="ref_b200": the reference toolkit's own Gpu-device layer classes with layers::LstmLayerB200<Gpu> (the
  adapter class of this repository, compiled against the reference's headers) in place of LstmLayer<Gpu>;
  needs a GPU and the built library.  It is the compiled form of the drop-in claim, not a checker.
* kind="port" / "port64": the plain-C restatement in oracle/currennt_oracle.c (fp32 / fp64).

Only tests/, the smoke check and the CPU-baseline leg of the benchmark may import this module.
All four kinds expose the same calls, in the order the reference's Optimizer drives a fraction
(Optimizer.cu:85-165 of the reference): load -> forward (returns SSE) -> backward -> sgd_update.
"""
import ctypes as C
import json
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
TYPE_CODES = {"input": 0, "feedforward_tanh": 1, "feedforward_logistic": 2,
              "feedforward_identity": 3, "lstm": 4, "blstm": 5, "sse": 6}

_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int)


def _ptr(a, t=_fp):
    return a.ctypes.data_as(t)


def ref_available(omp=False, adapter=False):
    name = "libcurrennt_ref_b200.so" if adapter else ("libcurrennt_ref_omp.so" if omp else "libcurrennt_ref.so")
    return os.path.exists(os.path.join(HERE, "_ref", name))


def _load(kind):
    if kind in ("ref", "ref_omp", "ref_b200"):
        path = os.path.join(HERE, "_ref", "libcurrennt_ref%s.so" % {"ref": "", "ref_omp": "_omp", "ref_b200": "_b200"}[kind])
        if not os.path.exists(path):
            raise FileNotFoundError(path + " (run oracle/build_ref.sh where the reference checkout exists)")
        lib, pre = C.CDLL(path), ("refb200_" if kind == "ref_b200" else "ref_")
    else:
        name = "libcurrennt_oracle%s.so" % ("_f64" if kind == "port64" else "")
        path = os.path.join(HERE, name)
        src = os.path.join(HERE, "currennt_oracle.c")
        if not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
            subprocess.check_call(["make", "-C", HERE, name], stdout=subprocess.DEVNULL)
        lib, pre = C.CDLL(path), "oracle_"
    f = lambda n: getattr(lib, pre + n)
    f("create").restype = C.c_void_p
    f("forward").restype = C.c_double
    for n in ("num_weights", "get_outputs", "get_output_errors", "get_output_errors_in"):
        f(n).restype = C.c_long
    return lib, pre


class _quiet_stdout:
    """The reference's constructors print progress lines with printf; keep them out of the
    caller's stdout (a benchmark prints exactly one JSON line there)."""

    def __enter__(self):
        import sys
        sys.stdout.flush()
        self.saved = os.dup(1)
        null = os.open(os.devnull, os.O_WRONLY)
        os.dup2(null, 1)
        os.close(null)

    def __exit__(self, *a):
        C.CDLL(None).fflush(None)
        os.dup2(self.saved, 1)
        os.close(self.saved)


class OracleNet:
    """layers: list of dicts with keys type, size and (trainable layers) bias, as in network.jsn."""

    def __init__(self, layers, P, maxT, kind="port", weights_section=None):
        """weights_section (reference kinds only): the "weights" object of a network file; the layers then read their
        weights from it, as the reference does when it loads trained_network.jsn"""
        self.kind, self.layers, self.P, self.maxT = kind, layers, P, maxT
        self.lib, self.pre = _load(kind)
        if kind.startswith("ref"):
            doc = {"layers": [dict({"name": "l%d" % i, "bias": 1.0}, **l) for i, l in enumerate(layers)]}
            fn = "create"
            if weights_section is not None:
                doc["weights"] = weights_section
                fn = "create_with_weights"
                self._f(fn).restype = C.c_void_p
            js = json.dumps(doc)
            with _quiet_stdout():
                self.h = C.c_void_p(self._f(fn)(js.encode(), P, maxT))
            if not self.h:
                self.lib.ref_last_error.restype = C.c_char_p
                raise RuntimeError(self.lib.ref_last_error().decode())
        else:
            n = len(layers)
            types = (C.c_int * n)(*[TYPE_CODES[l["type"]] for l in layers])
            sizes = (C.c_int * n)(*[l["size"] for l in layers])
            biases = (C.c_float * n)(*[float(l.get("bias", 1.0)) for l in layers])
            self.h = C.c_void_p(self._f("create")(n, types, sizes, biases, P, maxT))
        self.T = 0

    def _f(self, name):
        return getattr(self.lib, self.pre + name)

    def close(self):
        if self.h:
            self._f("destroy")(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def num_weights(self, i):
        return int(self._f("num_weights")(self.h, i))

    def export_json(self):
        """the network document as the reference writes it: its layers' exportLayer / exportWeights and its own JSON writer"""
        fn = self._f("export_json")
        fn.restype = C.c_long
        need = -int(fn(self.h, None, 0))
        buf = C.create_string_buffer(need)
        n = int(fn(self.h, buf, need))
        if n <= 0:
            raise RuntimeError("export_json failed")
        return buf.value.decode()

    def set_weights(self, i, w):
        w = np.ascontiguousarray(w, np.float32)
        assert w.size == self.num_weights(i)
        self._f("set_weights")(self.h, i, _ptr(w))

    def get_weights(self, i):
        w = np.empty(self.num_weights(i), np.float32)
        self._f("get_weights")(self.h, i, _ptr(w))
        return w

    def weight_updates(self, i):
        g = np.empty(self.num_weights(i), np.float32)
        self._f("get_weight_updates")(self.h, i, _ptr(g))
        return g

    def load(self, lens, inputs, targets):
        """inputs [T,P,in], targets [T,P,out] float32 (padded frames zero); lens: real lengths, len<=P."""
        lens = np.ascontiguousarray(lens, np.int32)
        inputs = np.ascontiguousarray(inputs, np.float32)
        targets = np.ascontiguousarray(targets, np.float32)
        T = inputs.shape[0]
        assert inputs.shape[1] == self.P and targets.shape[:2] == inputs.shape[:2]
        rc = self._f("load")(self.h, T, len(lens), _ptr(lens, _ip), _ptr(inputs), _ptr(targets))
        if rc != 0:
            raise RuntimeError("oracle load failed")
        self.T = int(lens.max())

    def forward(self):
        return float(self._f("forward")(self.h))

    def backward(self):
        self._f("backward")(self.h)

    def _get(self, name, i):
        size = self.layers[i]["size"]
        out = np.empty((self.T, self.P, size), np.float32)
        n = self._f(name)(self.h, i, _ptr(out))
        assert n == out.size, (n, out.size)
        return out

    def outputs(self, i):
        return self._get("get_outputs", i)

    def output_errors(self, i):
        return self._get("get_output_errors", i)

    def output_errors_in(self, i):
        return self._get("get_output_errors_in", i)

    def sgd_update(self, lr, momentum):
        self._f("sgd_update")(self.h, C.c_float(lr), C.c_float(momentum))
