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


def test_epoch_loop_rejects_a_data_set_opened_for_another_batch_shape(tmp_path):
    """The reference reads parallel_sequences and the sequence length limit of data set and network from one
    Configuration; here they are two handles, and a mismatch must be refused, not trained on mis-strided frames."""
    import b2lstm
    layers = L(("input", 5), ("lstm", 8), ("feedforward_identity", 2), ("sse", 2))
    path = corpus(tmp_path, [6, 9, 4, 7], 5, 2, 9)
    for net_P, net_T, data_P in [(4, 9, 2), (2, 9, 4), (2, 8, 2)]:
        net = b2lstm.Net(layers, net_P, net_T)
        ds = b2lstm.DataSet(path, data_P)
        for fn in (b2lstm.train_epoch, b2lstm.train_epoch_batch):
            with pytest.raises(b2lstm.B2Error, match="error -1"):       # B2_ERR_BAD_SHAPE
                fn(net, ds, 1e-3, 0.9)
        ds.close()
        net.close()


def test_a_recorded_timeout_reaches_the_caller_of_the_epoch_loop(tmp_path):
    """A kernel that gives up a bounded wait records B2_ERR_STEP_TIMEOUT in a device status word.  Written there
    from the host (no kernel is made to fail), the code must come back from the epoch loop and from the training
    run, which must not go on to store the weights; afterwards the net trains normally."""
    import b2lstm
    from b2lstm.lib import lib
    layers = L(("input", 5), ("blstm", 16), ("feedforward_identity", 2), ("sse", 2))
    path = corpus(tmp_path, [6, 9, 4, 7, 8], 5, 2, 10)
    net = b2lstm.Net(layers, 2, 9)
    ds = b2lstm.DataSet(path, 2)
    assert lib().b2_selftest_inject_status(net.h, -3) == 0
    with pytest.raises(b2lstm.B2Error, match="error -3"):
        b2lstm.train_epoch(net, ds, 1e-3, 0.9)
    ds.close()
    ds = b2lstm.DataSet(path, 2)
    opt = b2lstm.Optimizer(net, ds, max_epochs=3)
    assert lib().b2_selftest_inject_status(net.h, -3) == 0
    with pytest.raises(b2lstm.B2Error, match="error -3"):
        opt.train()
    assert opt.state["cur_epoch"] == 1
    opt.close()
    ds.close()
    ds = b2lstm.DataSet(path, 2)
    err, frames = b2lstm.train_epoch(net, ds, 1e-3, 0.9)                 # the status word was cleared by the report
    assert frames == 34 and err > 0
    ds.close()
    net.close()
