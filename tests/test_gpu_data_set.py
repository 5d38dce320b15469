"""GPU tests of the epoch loop over a .nc data set (b2_net_train_epoch): the loop that prefetches
fraction k+1 while fraction k trains must give exactly what separate train steps on the same
fractions give, and a validation pass must leave the weights alone."""
import numpy as np
import pytest

import parity
from make_golden import run as run_kind
from oracle import ref_available

pytestmark = pytest.mark.gpu


def L(*spec):
    return [dict(type=t, size=s, **({} if t in ("input", "sse") else {"bias": 1.0})) for t, s in spec]


def corpus(tmp_path, lens, n_in, n_out, seed):
    import b2lstm
    rng = np.random.default_rng(seed)
    n = int(sum(lens))
    x = rng.standard_normal((n, n_in)).astype(np.float32)
    y = rng.standard_normal((n, n_out)).astype(np.float32)
    path = str(tmp_path / ("c%d.nc" % seed))
    b2lstm.write_nc(path, ["s%03d" % i for i in range(len(lens))], lens, x, y)
    return path


def test_epoch_loop_equals_separate_train_steps(tmp_path):
    import b2lstm
    from b2lstm import workloads
    layers = L(("input", 9), ("feedforward_tanh", 16), ("blstm", 64), ("feedforward_identity", 4), ("sse", 4))
    P = 4
    lens = [12, 30, 7, 22, 18, 25, 9, 14, 27, 5, 20]          # 11 sequences: the last fraction is short
    path = corpus(tmp_path, lens, 9, 4, 5)
    w = workloads.make_weights(layers, 77, 0.1)
    lr, mom = 1e-3, 0.9

    def fresh():
        net = b2lstm.Net(layers, P, max(lens))
        for i, wi in w.items():
            net.set_weights(i, wi)
        return net

    # (a) the library's epoch loop, two epochs
    net = fresh()
    ds = b2lstm.DataSet(path, P)
    got = [b2lstm.train_epoch(net, ds, lr, mom) for _ in range(2)]
    net.synchronize()
    wa = {i: net.get_weights(i) for i in w}
    net.close()
    ds.close()

    # (b) the same fractions, one plain train step each
    net = fresh()
    ds = b2lstm.DataSet(path, P)
    want = []
    for _ in range(2):
        err, frames = 0.0, 0
        for f in ds.epoch():
            e = net.train_step(f["seq_lengths"], np.array(f["inputs"]), np.array(f["targets"]), lr, mom)
            err += e / ds.total_sequences
            frames += f["total_frames"]
        want.append((err, frames))
    net.synchronize()
    wb = {i: net.get_weights(i) for i in w}

    assert got == want
    assert got[0][1] == sum(lens)
    for i in w:
        assert np.array_equal(wa[i], wb[i])
        assert not np.array_equal(wa[i], w[i])

    # (c) validation pass: forward and error only
    e1, n1 = b2lstm.train_epoch(net, ds, -1.0, 0.0)
    e2, n2 = b2lstm.train_epoch(net, ds, -1.0, 0.0)
    assert e1 == e2 and n1 == n2 == sum(lens) and e1 > 0
    for i in w:
        assert np.array_equal(net.get_weights(i), wb[i])
    net.close()
    ds.close()


def test_first_fraction_of_a_data_set_matches_the_checker(tmp_path):
    """A fraction assembled from the .nc file goes through the same forward / backward as the checker's
    run on the arrays the file was written from."""
    import b2lstm
    from b2lstm import workloads
    layers = L(("input", 6), ("blstm", 32), ("feedforward_identity", 3), ("sse", 3))
    P = 3
    lens = np.array([9, 14, 11], np.int32)
    x, tg = workloads.make_fraction(6, 3, P, lens, 501, 502)
    wl = dict(P=P, lens=lens, x=x, tg=tg)
    path = str(tmp_path / "one.nc")
    workloads.write_nc(wl, path)
    w = workloads.make_weights(layers, 503, 0.2)
    kind = "ref" if ref_available() else "port"
    want = run_kind(kind, layers, P, lens, x, tg, w)
    ds = b2lstm.DataSet(path, P, training_mode=False)
    f = ds.next_fraction()
    net = b2lstm.Net(layers, P, int(lens.max()))
    for i, wi in w.items():
        net.set_weights(i, wi)
    net.load_fraction(f["seq_lengths"], np.array(f["inputs"]), np.array(f["targets"]))
    got = {"loss": net.forward()}
    net.backward()
    for i in (1, 2):
        got["out%d" % i] = net.outputs(i)
        got["dw%d" % i] = net.weight_updates(i)
    parity.compare_run(layers, got, want, "nc fraction", lstm_pad_zero_lens=lens)
    net.close()
