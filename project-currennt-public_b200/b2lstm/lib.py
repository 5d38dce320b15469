"""ctypes bindings of include/b2lstm.h.

Net mirrors the call order of the reference toolkit's training loop (Optimizer::_processDataSet,
optimizers/Optimizer.cu:68-231 of the reference): load_fraction -> forward (returns the SSE) ->
backward -> update_weights, or train_step for all of it.  LstmLayer mirrors layers::LstmLayer on
caller-owned device buffers (any object with a data_ptr(), e.g. torch CUDA tensors).
"""
import ctypes as C
import json
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))


def library_path():
    return os.path.join(os.path.dirname(_HERE), "libb2lstm.so")


class B2Error(RuntimeError):
    pass


_fp = C.POINTER(C.c_float)
_ip = C.POINTER(C.c_int)

# name -> (restype, argtypes); mirrors include/b2lstm.h one to one
SIGNATURES = {
    "b2_last_error_string": (C.c_char_p, []),
    "b2_version": (C.c_char_p, []),
    "b2_matrix_multiply": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int,
                                     C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "b2_matrix_multiply_noalloc": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                             C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "b2_lstm_num_weights": (C.c_size_t, [C.c_void_p]),
    "b2_lstm_create": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "b2_lstm_destroy": (None, [C.c_void_p]),
    "b2_lstm_load_sequences": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "b2_lstm_forward": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b2_lstm_backward": (C.c_int, [C.c_void_p] * 8),
    "b2_lstm_set_recurrence_mode": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_lstm_set_check_padding": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_lstm_state_bytes": (C.c_size_t, [C.c_void_p]),
    "b2_lstm_recurrence_path": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_net_recurrence_path": (C.c_int, [C.c_void_p, C.c_int, C.c_int]),
    "b2_lstm_synchronize": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b2_net_create": (C.c_int, [C.c_char_p, C.c_int, C.c_int, C.c_uint, C.POINTER(C.c_void_p)]),
    "b2_config_set_lstm_forget_gate_bias": (None, [C.c_float]),
    "b2_config_set_weights_uniform": (None, [C.c_float, C.c_float]),
    "b2_net_save_weights_binary": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int]),
    "b2_config_set_ptc_plan": (None, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "b2_net_destroy": (None, [C.c_void_p]),
    "b2_net_parallel_sequences": (C.c_int, [C.c_void_p]),
    "b2_net_max_seq_length": (C.c_int, [C.c_void_p]),
    "b2_net_num_layers": (C.c_int, [C.c_void_p]),
    "b2_net_layer_size": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_net_num_weights": (C.c_size_t, [C.c_void_p, C.c_int]),
    "b2_net_set_weights": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "b2_net_get_weights": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "b2_net_get_weight_updates": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "b2_net_weights_dev": (C.c_void_p, [C.c_void_p, C.c_int]),
    "b2_net_weight_updates_dev": (C.c_void_p, [C.c_void_p, C.c_int]),
    "b2_net_outputs_dev": (C.c_void_p, [C.c_void_p, C.c_int]),
    "b2_net_output_errors_dev": (C.c_void_p, [C.c_void_p, C.c_int]),
    "b2_net_load_fraction": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b2_net_load_fraction_dev": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b2_net_forward": (C.c_int, [C.c_void_p, C.POINTER(C.c_double)]),
    "b2_net_backward": (C.c_int, [C.c_void_p]),
    "b2_net_update_weights": (C.c_int, [C.c_void_p, C.c_float, C.c_float]),
    "b2_net_set_optimizer": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_net_get_optimizer_stats": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t, C.POINTER(C.c_size_t)]),
    "b2_net_accumulate_weight_updates": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_net_update_weights_batch": (C.c_int, [C.c_void_p, C.c_float, C.c_float]),
    "b2_net_train_epoch_batch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.POINTER(C.c_double),
                                           C.POINTER(C.c_longlong)]),
    "b2_net_train_step": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float,
                                    C.c_float, C.POINTER(C.c_double)]),
    "b2_net_prefetch_fraction": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b2_net_train_step_prefetched": (C.c_int, [C.c_void_p, C.c_float, C.c_float, C.POINTER(C.c_double)]),
    "b2_net_read_error": (C.c_int, [C.c_void_p, C.POINTER(C.c_double)]),
    "b2_net_train_step_dev": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float,
                                        C.c_float]),
    "b2_net_get_outputs": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "b2_net_get_output_errors": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "b2_net_synchronize": (C.c_int, [C.c_void_p]),
    "b2_net_stream": (C.c_void_p, [C.c_void_p]),
    "b2_net_set_recurrence_mode": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_net_set_force_ffma": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_net_launch_count": (C.c_ulonglong, [C.c_void_p]),
    "b2_net_set_profiling": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_net_get_profile": (C.c_int, [C.c_void_p, C.c_int, C.POINTER(C.c_char_p), _fp, _ip]),
    "b2_selftest_bounded_wait": (C.c_int, [_ip, _ip]),
    "b2_selftest_inject_status": (C.c_int, [C.c_void_p, C.c_int]),
    "b2_dp_get_unique_id": (C.c_int, [C.c_void_p]),
    "b2_dp_attach": (C.c_int, [C.c_void_p, C.c_int, C.c_int, C.c_void_p]),
    "b2_dp_detach": (C.c_int, [C.c_void_p]),
    "b2_dp_allreduce_scalar": (C.c_int, [C.c_void_p, C.POINTER(C.c_double)]),
    "b2_dp_world_size": (C.c_int, [C.c_void_p]),
    "b2_net_train_step_empty": (C.c_int, [C.c_void_p, C.c_float, C.c_float]),
    "b2_net_backward_empty": (C.c_int, [C.c_void_p]),
    "b2_data_open": (C.c_int, [C.POINTER(C.c_void_p), C.POINTER(C.c_char_p), C.c_int, C.c_void_p]),
    "b2_data_close": (None, [C.c_void_p]),
    "b2_data_info": (C.c_int, [C.c_void_p, _ip, C.POINTER(C.c_longlong), _ip, _ip, _ip, _ip]),
    "b2_data_output_mean_stdev": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, _ip]),
    "b2_data_next_fraction": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b2_data_fraction_seq_info": (C.c_int, [C.c_void_p, C.c_int, C.c_char_p, C.c_int, _ip]),
    "b2_data_reseed": (None, [C.c_uint]),
    "b2_net_train_epoch": (C.c_int, [C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.POINTER(C.c_double),
                                     C.POINTER(C.c_longlong)]),
    "b2_net_export_json": (C.c_int, [C.c_void_p, C.c_char_p, C.c_size_t, C.POINTER(C.c_size_t), C.c_int]),
    "b2_net_save_network": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int]),
    "b2_net_get_weight_deltas": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "b2_net_set_weight_deltas": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p]),
    "b2_optimizer_create": (C.c_int, [C.POINTER(C.c_void_p), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "b2_optimizer_destroy": (None, [C.c_void_p]),
    "b2_optimizer_train": (C.c_int, [C.c_void_p, _ip]),
    "b2_optimizer_get_state": (C.c_int, [C.c_void_p, C.c_void_p]),
    "b2_optimizer_save_state": (C.c_int, [C.c_void_p, C.c_char_p, C.c_char_p, C.c_char_p, C.c_int]),
    "b2_optimizer_restore_state": (C.c_int, [C.c_void_p, C.c_char_p, C.c_char_p, C.c_size_t]),
}

_lib = None


def lib():
    """The loaded shared library.  Raises if it has not been built: there is no other code path."""
    global _lib
    if _lib is None:
        path = library_path()
        if not os.path.exists(path):
            raise B2Error("%s is missing: build it with `make -C %s/csrc` (or __graft_entry__.build())"
                          % (path, os.path.dirname(_HERE)))
        _lib = C.CDLL(path, mode=C.RTLD_GLOBAL)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.restype = res
            fn.argtypes = args
    return _lib


def _check(rc):
    if rc != 0:
        raise B2Error("b2lstm error %d: %s" % (rc, lib().b2_last_error_string().decode()))


def _dev(x):
    """device address of a tensor-like object (or a raw int / None)"""
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return x.data_ptr()


class _LstmDesc(C.Structure):
    _fields_ = [("parallel_sequences", C.c_int), ("max_seq_length", C.c_int), ("prev_size", C.c_int),
                ("size", C.c_int), ("bidirectional", C.c_int), ("bias", C.c_float)]


def lstm_num_weights(prev_size, size, bidirectional):
    d = _LstmDesc(1, 1, prev_size, size, int(bidirectional), 1.0)
    return int(lib().b2_lstm_num_weights(C.byref(d)))


def matrix_multiply(Cm, ldc, A, lda, transA, B, ldb, transB, m, n, k, accumulate=False, force_ffma=False, stream=None):
    _check(lib().b2_matrix_multiply(_dev(Cm), ldc, _dev(A), lda, int(transA), _dev(B), ldb, int(transB), m, n, k,
                                    int(accumulate), int(force_ffma), stream))


def matrix_multiply_noalloc(Cm, ldc, A, lda, transA, B, ldb, transB, m, n, k, accumulate=False, stream=None):
    """b2_matrix_multiply_noalloc: the FFMA product with its scratch in a fixed array of the library
    image, for hosts that cannot have device memory allocated for them (see include/b2lstm.h)."""
    _check(lib().b2_matrix_multiply_noalloc(_dev(Cm), ldc, _dev(A), lda, int(transA), _dev(B), ldb, int(transB), m, n, k,
                                            int(accumulate), stream))


class LstmLayer:
    """layers::LstmLayer on caller-owned device buffers (see include/b2lstm.h)."""

    def __init__(self, parallel_sequences, max_seq_length, prev_size, size, bidirectional, bias=1.0):
        self.desc = _LstmDesc(parallel_sequences, max_seq_length, prev_size, size, int(bidirectional), bias)
        self.h = C.c_void_p()
        _check(lib().b2_lstm_create(C.byref(self.desc), C.byref(self.h)))
        self.num_weights = int(lib().b2_lstm_num_weights(C.byref(self.desc)))

    def close(self):
        if self.h:
            lib().b2_lstm_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load_sequences(self, cur_max_len, cur_min_len, pat_types_dev):
        _check(lib().b2_lstm_load_sequences(self.h, cur_max_len, cur_min_len, _dev(pat_types_dev)))

    def forward(self, weights, x, y, stream=None):
        _check(lib().b2_lstm_forward(self.h, _dev(weights), _dev(x), _dev(y), stream))

    def backward(self, weights, x, y, dy, dx, dw, stream=None):
        _check(lib().b2_lstm_backward(self.h, _dev(weights), _dev(x), _dev(y), _dev(dy), _dev(dx), _dev(dw), stream))

    def set_recurrence_mode(self, mode):
        _check(lib().b2_lstm_set_recurrence_mode(self.h, mode))

    def synchronize(self, stream=None):
        _check(lib().b2_lstm_synchronize(self.h, stream))

    def recurrence_path(self, backward=False):
        return int(lib().b2_lstm_recurrence_path(self.h, int(backward)))

    def set_check_padding(self, on):
        _check(lib().b2_lstm_set_check_padding(self.h, int(on)))

    @property
    def state_bytes(self):
        return int(lib().b2_lstm_state_bytes(self.h))


def selftest_bounded_wait():
    """(recorded status, left through the timeout path): see b2_selftest_bounded_wait"""
    st, gu = C.c_int(), C.c_int()
    _check(lib().b2_selftest_bounded_wait(C.byref(st), C.byref(gu)))
    return st.value, bool(gu.value)


def dp_unique_id():
    buf = C.create_string_buffer(128)
    _check(lib().b2_dp_get_unique_id(buf))
    return buf.raw


class Net:
    """NeuralNetwork + steepest-descent step.  layers: list of dicts as in the reference's network.jsn."""

    def __init__(self, layers, parallel_sequences, max_seq_length, seed=1234, weights=None):
        doc = {"layers": [dict({"name": "l%d" % i}, **l) for i, l in enumerate(layers)]}
        if weights is not None:
            doc["weights"] = weights
        self.layers = doc["layers"]
        self.P, self.maxT = parallel_sequences, max_seq_length
        self.h = C.c_void_p()
        _check(lib().b2_net_create(json.dumps(doc).encode(), parallel_sequences, max_seq_length, seed, C.byref(self.h)))
        self.T = 0

    def close(self):
        if self.h:
            lib().b2_net_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def num_weights(self, i):
        return int(lib().b2_net_num_weights(self.h, i))

    def set_weights(self, i, w):
        w = np.ascontiguousarray(w, np.float32)
        if w.size != self.num_weights(i):
            raise B2Error("layer %d takes %d weights, got %d" % (i, self.num_weights(i), w.size))
        _check(lib().b2_net_set_weights(self.h, i, w.ctypes.data))

    def get_weights(self, i):
        w = np.empty(self.num_weights(i), np.float32)
        _check(lib().b2_net_get_weights(self.h, i, w.ctypes.data))
        return w

    def weight_updates(self, i):
        g = np.empty(self.num_weights(i), np.float32)
        _check(lib().b2_net_get_weight_updates(self.h, i, g.ctypes.data))
        return g

    def _lens(self, lens):
        lens = np.ascontiguousarray(lens, np.int32)
        self.T = int(lens.max())
        return lens

    def load_fraction(self, lens, inputs, targets):
        """Host arrays: inputs [T,P,in], targets [T,P,out] float32 (padding zero); lens of the real sequences."""
        lens = self._lens(lens)
        inputs = np.ascontiguousarray(inputs, np.float32)
        targets = np.ascontiguousarray(targets, np.float32)
        _check(lib().b2_net_load_fraction(self.h, inputs.shape[0], len(lens), lens.ctypes.data, inputs.ctypes.data,
                                          targets.ctypes.data))
        _check(lib().b2_net_synchronize(self.h))   # the host arrays may go away after this call

    def load_fraction_dev(self, lens, T, inputs_dev, targets_dev):
        lens = self._lens(lens)
        _check(lib().b2_net_load_fraction_dev(self.h, T, len(lens), lens.ctypes.data, _dev(inputs_dev), _dev(targets_dev)))

    def forward(self):
        e = C.c_double()
        _check(lib().b2_net_forward(self.h, C.byref(e)))
        return e.value

    def backward(self):
        _check(lib().b2_net_backward(self.h))

    def accumulate_weight_updates(self, first):
        _check(lib().b2_net_accumulate_weight_updates(self.h, int(first)))

    def update_weights_batch(self, lr, momentum):
        _check(lib().b2_net_update_weights_batch(self.h, lr, momentum))

    def update_weights(self, lr, momentum):
        _check(lib().b2_net_update_weights(self.h, lr, momentum))

    def train_step(self, lens, inputs, targets, lr, momentum, want_error=True):
        """inputs/targets: host arrays (numpy, or pinned torch CPU tensors via .numpy())."""
        lens = self._lens(lens)
        e = C.c_double()
        _check(lib().b2_net_train_step(self.h, inputs.shape[0], len(lens), lens.ctypes.data, inputs.ctypes.data,
                                       targets.ctypes.data, lr, momentum, C.byref(e) if want_error else None))
        return e.value if want_error else None

    def prefetch_fraction(self, lens, inputs, targets):
        """Start the host->device copy of the NEXT fraction (pinned host arrays that stay alive)."""
        lens = np.ascontiguousarray(lens, np.int32)
        self._next_T = int(lens.max())
        _check(lib().b2_net_prefetch_fraction(self.h, inputs.shape[0], len(lens), lens.ctypes.data, inputs.ctypes.data,
                                              targets.ctypes.data))

    def train_step_prefetched(self, lr, momentum, want_error=True):
        e = C.c_double()
        _check(lib().b2_net_train_step_prefetched(self.h, lr, momentum, C.byref(e) if want_error else None))
        self.T = self._next_T
        return e.value if want_error else None

    def read_error(self):
        e = C.c_double()
        _check(lib().b2_net_read_error(self.h, C.byref(e)))
        return e.value

    def train_step_dev(self, lens, T, inputs_dev, targets_dev, lr, momentum):
        lens = self._lens(lens)
        _check(lib().b2_net_train_step_dev(self.h, T, len(lens), lens.ctypes.data, _dev(inputs_dev), _dev(targets_dev),
                                           lr, momentum))

    def _vec(self, fn, i):
        out = np.empty((self.T, self.P, self.layers[i]["size"]), np.float32)
        _check(fn(self.h, i, out.ctypes.data))
        return out

    def outputs(self, i):
        return self._vec(lib().b2_net_get_outputs, i)

    def output_errors(self, i):
        return self._vec(lib().b2_net_get_output_errors, i)

    def synchronize(self):
        _check(lib().b2_net_synchronize(self.h))

    @property
    def stream(self):
        return lib().b2_net_stream(self.h)

    def set_recurrence_mode(self, mode):
        _check(lib().b2_net_set_recurrence_mode(self.h, mode))

    def set_force_ffma(self, on):
        _check(lib().b2_net_set_force_ffma(self.h, int(on)))

    RECURRENCE_PATHS = {0: "stepwise", 1: "persistent_ffma", 3: "tensor_core_per_step", 5: "persistent_tensor_core"}

    def recurrence_path(self, layer, backward=False):
        """which recurrence kernels layer `layer` really ran in its last sweep (-1: not a (b)lstm layer / none yet)"""
        return int(lib().b2_net_recurrence_path(self.h, layer, int(backward)))

    def recurrence_paths(self):
        """{layer index: (forward path name, backward path name)} of the (b)lstm layers"""
        out = {}
        for i in range(int(lib().b2_net_num_layers(self.h))):
            f = self.recurrence_path(i, False)
            if f >= 0:
                b = self.recurrence_path(i, True)
                out[i] = (self.RECURRENCE_PATHS.get(f, str(f)), self.RECURRENCE_PATHS.get(b, str(b)))
        return out

    @property
    def launch_count(self):
        return int(lib().b2_net_launch_count(self.h))

    def set_profiling(self, on):
        _check(lib().b2_net_set_profiling(self.h, int(on)))

    def get_profile(self):
        """{phase name: (milliseconds, launches)} accumulated since profiling was switched on; clears."""
        cap = 64
        names = (C.c_char_p * cap)()
        ms = (C.c_float * cap)()
        ln = (C.c_int * cap)()
        n = lib().b2_net_get_profile(self.h, cap, names, ms, ln)
        return {names[i].decode(): (float(ms[i]), int(ln[i])) for i in range(n)}

    def set_optimizer(self, option):
        """0 plain, 1 AdaGrad, 2 average gradient, 3 SGD accumulating AdaGrad statistics (AdaGrad after a validation
        stall), 4 SGD with learning-rate decay after a validation stall, 5 Adam"""
        _check(lib().b2_net_set_optimizer(self.h, option))

    def optimizer_stats(self, i):
        n = C.c_size_t()
        _check(lib().b2_net_get_optimizer_stats(self.h, i, None, 0, C.byref(n)))
        out = np.empty(n.value, np.float32)
        if n.value:
            _check(lib().b2_net_get_optimizer_stats(self.h, i, out.ctypes.data, n.value, None))
        return out

    def export_json(self, digits=0):
        """The network as the reference's network.jsn text (layers + weights)."""
        need = C.c_size_t()
        _check(lib().b2_net_export_json(self.h, None, 0, C.byref(need), digits))
        buf = C.create_string_buffer(need.value)
        _check(lib().b2_net_export_json(self.h, buf, need.value, None, digits))
        return buf.value.decode()

    def save_weights_binary(self, filename, with_type_codes=False):
        """NeuralNetwork::printWeightMatrix: header + raw float weights (pyTools/ioTools/nnio.py reads it)"""
        _check(lib().b2_net_save_weights_binary(self.h, os.fsencode(filename), int(with_type_codes)))

    def save_network(self, filename, digits=0):
        _check(lib().b2_net_save_network(self.h, os.fsencode(filename), digits))

    def weight_deltas(self, i):
        out = np.empty(self.num_weights(i), np.float32)
        _check(lib().b2_net_get_weight_deltas(self.h, i, out.ctypes.data))
        return out

    def set_weight_deltas(self, i, d):
        d = np.ascontiguousarray(d, np.float32)
        _check(lib().b2_net_set_weight_deltas(self.h, i, d.ctypes.data))

    def dp_attach(self, rank, world, unique_id):
        _check(lib().b2_dp_attach(self.h, rank, world, unique_id))

    def dp_detach(self):
        _check(lib().b2_dp_detach(self.h))

    def dp_allreduce_scalar(self, v):
        d = C.c_double(v)
        _check(lib().b2_dp_allreduce_scalar(self.h, C.byref(d)))
        return d.value


class _DataOptions(C.Structure):
    _fields_ = [("parallel_sequences", C.c_int), ("fraction", C.c_float), ("trunc_seq_length", C.c_int),
                ("fraction_shuffling", C.c_int), ("sequence_shuffling", C.c_int), ("random_seed", C.c_uint),
                ("training_mode", C.c_int), ("loader_threads", C.c_int), ("shard_rank", C.c_int), ("shard_count", C.c_int)]


class _Fraction(C.Structure):
    _fields_ = [("max_seq_length", C.c_int), ("min_seq_length", C.c_int), ("num_sequences", C.c_int),
                ("total_frames", C.c_longlong), ("seq_lengths", _ip), ("inputs", _fp), ("targets", _fp),
                ("pat_types", C.POINTER(C.c_char))]


class DataSet:
    """data_sets::DataSet of the reference over .nc files (b2_data_*): iterate epochs with
    `for frac in ds.epoch():`; a fraction is a dict of numpy views that stay valid for two more
    fractions."""

    def __init__(self, paths, parallel_sequences, fraction=1.0, trunc_seq_length=0, fraction_shuffling=False,
                 sequence_shuffling=False, random_seed=0, training_mode=True, loader_threads=0, shard_rank=0,
                 shard_count=1):
        if isinstance(paths, str):
            paths = [paths]
        arr = (C.c_char_p * len(paths))(*[os.fsencode(p) for p in paths])
        opt = _DataOptions(parallel_sequences, fraction, trunc_seq_length, int(fraction_shuffling),
                           int(sequence_shuffling), random_seed, int(training_mode), loader_threads, shard_rank, shard_count)
        self.h = C.c_void_p()
        _check(lib().b2_data_open(C.byref(self.h), arr, len(paths), C.byref(opt)))
        self.P = parallel_sequences
        n, ts, mn, mx, i, o = C.c_int(), C.c_longlong(), C.c_int(), C.c_int(), C.c_int(), C.c_int()
        _check(lib().b2_data_info(self.h, C.byref(n), C.byref(ts), C.byref(mn), C.byref(mx), C.byref(i), C.byref(o)))
        self.total_sequences, self.total_timesteps = n.value, ts.value
        self.min_seq_length, self.max_seq_length = mn.value, mx.value
        self.input_size, self.output_size = i.value, o.value

    def close(self):
        if self.h:
            lib().b2_data_close(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def output_mean_stdev(self):
        m = np.zeros(self.output_size, np.float32)
        s = np.zeros(self.output_size, np.float32)
        present = C.c_int()
        _check(lib().b2_data_output_mean_stdev(self.h, m.ctypes.data, s.ctypes.data, C.byref(present)))
        return m, s, bool(present.value)

    def next_fraction(self):
        """dict for the next fraction, or None once at the end of an epoch"""
        f = _Fraction()
        rc = lib().b2_data_next_fraction(self.h, C.byref(f))
        if rc == 1:
            return None
        _check(rc)
        T, P, n = f.max_seq_length, self.P, f.num_sequences
        if n == 0:      # a shard without sequences in this fraction
            return {"T": 0, "min_seq_length": 0, "num_sequences": 0, "total_frames": 0, "seq_lengths": np.zeros(0, np.int32),
                    "inputs": np.zeros((0, P, self.input_size), np.float32),
                    "targets": np.zeros((0, P, self.output_size), np.float32), "pat_types": np.zeros((0, P), np.int8),
                    "tags": [], "original_seq_idx": []}
        tags, orig = [], []
        buf = C.create_string_buffer(1024)
        k = C.c_int()
        for i in range(n):
            _check(lib().b2_data_fraction_seq_info(self.h, i, buf, 1024, C.byref(k)))
            tags.append(buf.value.decode())
            orig.append(k.value)
        return {"T": T, "min_seq_length": f.min_seq_length, "num_sequences": n, "total_frames": f.total_frames,
                "seq_lengths": np.ctypeslib.as_array(f.seq_lengths, (n,)).copy(),
                "inputs": np.ctypeslib.as_array(f.inputs, (T, P, self.input_size)),
                "targets": np.ctypeslib.as_array(f.targets, (T, P, self.output_size)),
                "pat_types": np.frombuffer(C.string_at(f.pat_types, T * P), np.int8).reshape(T, P),
                "tags": tags, "original_seq_idx": orig}

    def epoch(self):
        while True:
            f = self.next_fraction()
            if f is None:
                return
            yield f


def data_reseed(seed):
    lib().b2_data_reseed(seed)


def train_epoch(net, data, lr, momentum):
    """b2_net_train_epoch: (error, frames); lr < 0 = validation pass (forward and error only)"""
    e, n = C.c_double(), C.c_longlong()
    _check(lib().b2_net_train_epoch(net.h, data.h, lr, momentum, C.byref(e), C.byref(n)))
    return e.value, n.value


def train_epoch_batch(net, data, lr, momentum):
    """b2_net_train_epoch_batch (batch learning: one update per epoch): (error, frames)"""
    e, n = C.c_double(), C.c_longlong()
    _check(lib().b2_net_train_epoch_batch(net.h, data.h, lr, momentum, C.byref(e), C.byref(n)))
    return e.value, n.value


def write_nc(path, seq_tags, seq_lengths, inputs, targets, output_means=None, output_stdevs=None, version=2):
    """Writes a data set in the toolkit's .nc layout (netCDF classic via scipy, as the reference's
    pyTools/dataTools/ncDataHandle.py does): inputs [numTimesteps, inputPattSize], targets
    [numTimesteps, targetPattSize], sequences back to back."""
    from scipy.io import netcdf_file
    inputs = np.asarray(inputs, np.float32)
    targets = np.asarray(targets, np.float32)
    n = len(seq_lengths)
    taglen = max(len(t) for t in seq_tags) + 1
    with netcdf_file(path, "w", version=version) as f:
        f.createDimension("numSeqs", n)
        f.createDimension("numTimesteps", inputs.shape[0])
        f.createDimension("inputPattSize", inputs.shape[1])
        f.createDimension("targetPattSize", targets.shape[1])
        f.createDimension("maxSeqTagLength", taglen)
        tv = f.createVariable("seqTags", "S1", ("numSeqs", "maxSeqTagLength"))
        lv = f.createVariable("seqLengths", "i", ("numSeqs",))
        iv = f.createVariable("inputs", "f", ("numTimesteps", "inputPattSize"))
        ov = f.createVariable("targetPatterns", "f", ("numTimesteps", "targetPattSize"))
        tags = np.zeros((n, taglen), "S1")
        for i, t in enumerate(seq_tags):
            tags[i, :len(t)] = list(t)
        tv[:] = tags
        lv[:] = np.asarray(seq_lengths, np.int32)
        iv[:] = inputs
        ov[:] = targets
        if output_means is not None:
            mv = f.createVariable("outputMeans", "f", ("targetPattSize",))
            sv = f.createVariable("outputStdevs", "f", ("targetPattSize",))
            mv[:] = np.asarray(output_means, np.float32)
            sv[:] = np.asarray(output_stdevs, np.float32)


class _OptimizerOptions(C.Structure):
    _fields_ = [("learning_rate", C.c_float), ("momentum", C.c_float), ("max_epochs", C.c_int),
                ("max_epochs_no_best", C.c_int), ("validate_every", C.c_int), ("test_every", C.c_int),
                ("batch_learning", C.c_int), ("second_learning_rate", C.c_float), ("lr_decay_rate", C.c_float)]


class _OptimizerState(C.Structure):
    _fields_ = [("finished", C.c_int), ("cur_epoch", C.c_int), ("epochs_since_lowest_error", C.c_int),
                ("lowest_validation_error", C.c_float), ("cur_training_error", C.c_float),
                ("cur_validation_error", C.c_float), ("cur_test_error", C.c_float),
                ("cur_training_error_per_frame", C.c_float), ("cur_validation_error_per_frame", C.c_float),
                ("cur_test_error_per_frame", C.c_float), ("learning_rate", C.c_float), ("optimizer_option", C.c_int)]


class Optimizer:
    """optimizers::SteepestDescentOptimizer of the reference around a Net and its data sets:
    train() runs one epoch (plus validation / test passes when due) and returns True when finished."""

    def __init__(self, net, training_set, validation_set=None, test_set=None, learning_rate=1e-5, momentum=0.9,
                 max_epochs=-1, max_epochs_no_best=20, validate_every=1, test_every=1, batch_learning=False,
                 second_learning_rate=0.01, lr_decay_rate=0.1):
        opt = _OptimizerOptions(learning_rate, momentum, max_epochs, max_epochs_no_best, validate_every, test_every,
                                int(batch_learning), second_learning_rate, lr_decay_rate)
        self.h = C.c_void_p()
        self._keep = (net, training_set, validation_set, test_set)
        _check(lib().b2_optimizer_create(C.byref(self.h), net.h, training_set.h,
                                         validation_set.h if validation_set else None,
                                         test_set.h if test_set else None, C.byref(opt)))

    def close(self):
        if self.h:
            lib().b2_optimizer_destroy(self.h)
            self.h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def train(self):
        fin = C.c_int()
        _check(lib().b2_optimizer_train(self.h, C.byref(fin)))
        return bool(fin.value)

    @property
    def state(self):
        s = _OptimizerState()
        _check(lib().b2_optimizer_get_state(self.h, C.byref(s)))
        return {k: getattr(s, k) for k, _ in _OptimizerState._fields_}

    def save_state(self, filename, configuration="", info_rows="", digits=0):
        _check(lib().b2_optimizer_save_state(self.h, os.fsencode(filename), configuration.encode(), info_rows.encode(), digits))

    def restore_state(self, filename):
        buf = C.create_string_buffer(1 << 16)
        _check(lib().b2_optimizer_restore_state(self.h, os.fsencode(filename), buf, len(buf)))
        return buf.value.decode()
