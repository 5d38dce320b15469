"""GPU tests of network export and of the training run around the epoch loop (b2_net_export_json,
b2_optimizer_*): JSON round trips with the reference's member names, early stopping on the
validation error, autosave / continue."""
import json

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def L(*spec):
    return [dict(type=t, size=s, **({} if t in ("input", "sse") else {"bias": 1.0})) for t, s in spec]


LAYERS = L(("input", 7), ("feedforward_tanh", 12), ("blstm", 16), ("lstm", 9), ("feedforward_identity", 3), ("sse", 3))


def corpus(tmp_path, name, lens, seed, w_true):
    """targets are a fixed linear map of the inputs plus noise: something a few epochs can learn"""
    import b2lstm
    rng = np.random.default_rng(seed)
    n = int(sum(lens))
    x = rng.standard_normal((n, 7)).astype(np.float32)
    y = (np.tanh(x @ w_true) + 0.05 * rng.standard_normal((n, 3))).astype(np.float32)
    path = str(tmp_path / name)
    b2lstm.write_nc(path, ["%s%03d" % (name[:2], i) for i in range(len(lens))], lens, x, y)
    return path


def test_export_json_round_trips_exactly_and_keeps_the_reference_layout():
    import b2lstm
    from b2lstm import workloads
    w = workloads.make_weights(LAYERS, 5, 0.3)
    net = b2lstm.Net(LAYERS, 2, 8)
    for i, wi in w.items():
        net.set_weights(i, wi)
    doc = json.loads(net.export_json())
    assert [l["type"] for l in doc["layers"]] == [l["type"] for l in LAYERS]
    assert [l["size"] for l in doc["layers"]] == [l["size"] for l in LAYERS]
    assert all(("bias" in l) == (l["type"] not in ("input", "sse")) for l in doc["layers"])
    for i, wi in w.items():
        sec = doc["weights"][doc["layers"][i]["name"]]
        ls, pls = LAYERS[i]["size"], LAYERS[i - 1]["size"]
        per = 4 if "lstm" in LAYERS[i]["type"] else 1
        assert len(sec["input"]) == ls * per * pls and len(sec["bias"]) == ls * per
        flat = np.array(sec["input"] + sec["bias"] + sec["internal"], np.float32)
        assert np.array_equal(flat, wi)                     # 9 significant digits: exact for fp32
    # a net created from the exported document holds the same weights
    net2 = b2lstm.Net([{k: v for k, v in l.items()} for l in doc["layers"]], 2, 8, weights=doc["weights"])
    for i, wi in w.items():
        assert np.array_equal(net2.get_weights(i), wi)
    # the reference's writer prints "%g": six digits
    short = json.loads(net.export_json(digits=6))
    a = np.array(short["weights"][doc["layers"][2]["name"]]["input"], np.float32)
    assert np.allclose(a, w[2][:a.size], rtol=1e-5) and not np.array_equal(a, w[2][:a.size])
    net.close()
    net2.close()


def test_binary_weight_dump_has_the_layout_of_the_reference(tmp_path):
    """b2_net_save_weights_binary = NeuralNetwork::printWeightMatrix; the expected bytes come from the restatement that
    tests/test_weights_binary.py pins to the reference's own reader."""
    import b2lstm
    import parity
    from b2lstm import workloads
    w = workloads.make_weights(LAYERS, 5, 0.3)
    net = b2lstm.Net(LAYERS, 2, 8)
    for i, wi in w.items():
        net.set_weights(i, wi)
    for codes in (False, True):
        path = str(tmp_path / ("w%d.bin" % codes))
        net.save_weights_binary(path, with_type_codes=codes)
        assert open(path, "rb").read() == parity.weight_dump_bytes(LAYERS, w, with_type_codes=codes)
    net.close()


def test_training_run_stops_on_validation_error_and_restores_best_weights(tmp_path):
    import b2lstm
    from b2lstm import workloads
    w_true = np.random.default_rng(0).standard_normal((7, 3)).astype(np.float32)
    train = corpus(tmp_path, "train.nc", [20, 35, 28, 31, 25, 22, 38, 27], 1, w_true)
    valid = corpus(tmp_path, "valid.nc", [30, 24, 33], 2, w_true)
    P = 4
    w = workloads.make_weights(LAYERS, 9, 0.1)

    def fresh():
        net = b2lstm.Net(LAYERS, P, 40)
        for i, wi in w.items():
            net.set_weights(i, wi)
        return net

    net = fresh()
    tr, va = b2lstm.DataSet(train, P), b2lstm.DataSet(valid, P)
    opt = b2lstm.Optimizer(net, tr, va, learning_rate=3e-4, momentum=0.9, max_epochs=6, max_epochs_no_best=3)
    hist = []
    while not opt.train():
        hist.append(opt.state)
    hist.append(opt.state)
    assert hist[-1]["finished"] == 1 and hist[-1]["cur_epoch"] == len(hist) <= 6
    assert hist[-1]["cur_training_error"] < hist[0]["cur_training_error"]          # it learns
    best = min(h["cur_validation_error"] for h in hist)
    assert hist[-1]["lowest_validation_error"] == best
    # finished: the weights of the best validation epoch are back in the net
    e, _ = b2lstm.train_epoch(net, va, -1.0, 0.0)
    assert abs(e - best) <= 1e-6 * abs(best)
    per_frame = hist[-1]["cur_training_error"] * tr.total_sequences / tr.total_timesteps
    assert abs(hist[-1]["cur_training_error_per_frame"] - per_frame) <= 1e-6 * per_frame

    # autosave after two epochs, continue in a fresh process state: same trajectory as an uninterrupted run
    net_a = fresh()
    tr_a, va_a = b2lstm.DataSet(train, P), b2lstm.DataSet(valid, P)
    opt_a = b2lstm.Optimizer(net_a, tr_a, va_a, learning_rate=3e-4, momentum=0.9, max_epochs=6, max_epochs_no_best=3)
    opt_a.train()
    opt_a.train()
    save = str(tmp_path / "epoch002.autosave")
    opt_a.save_state(save, configuration="max_epochs = 6", info_rows="row one\nrow two")
    doc = json.load(open(save))
    for key in ("configuration", "info_rows", "layers", "weights", "optimizer_finished", "optimizer_cur_epoch",
                "optimizer_epochs_since_lowest_error", "optimizer_lowest_validation_error", "optimizer_cur_training_error",
                "optimizer_cur_validation_error", "optimizer_cur_test_error", "optimizer_status", "optimizer_best_weights",
                "steepest_descent_optimizer_weight_deltas"):
        assert key in doc, key
    assert doc["optimizer_cur_epoch"] == 2 and doc["info_rows"] == "row one;;;row two"
    assert len(doc["optimizer_best_weights"]) == len(LAYERS) and doc["optimizer_best_weights"][0] == []

    net_b = b2lstm.Net(LAYERS, P, 40, seed=999)                    # different initial weights on purpose
    tr_b, va_b = b2lstm.DataSet(train, P), b2lstm.DataSet(valid, P)
    opt_b = b2lstm.Optimizer(net_b, tr_b, va_b, learning_rate=3e-4, momentum=0.9, max_epochs=6, max_epochs_no_best=3)
    assert opt_b.restore_state(save) == "row one\nrow two"
    saved = lambda st: {k: v for k, v in st.items() if not k.endswith("_per_frame")}   # per-frame errors are not part of the file
    assert saved(opt_b.state) == saved(opt_a.state)
    for i in w:
        assert np.array_equal(net_b.get_weights(i), net_a.get_weights(i))
        assert np.array_equal(net_b.weight_deltas(i), net_a.weight_deltas(i))
    fa, fb = opt_a.train(), opt_b.train()
    assert fa == fb and opt_a.state == opt_b.state == hist[2]
    for i in w:
        assert np.array_equal(net_b.get_weights(i), net_a.get_weights(i))
    for o in (opt, opt_a, opt_b):
        o.close()
    for n in (net, net_a, net_b):
        n.close()


@pytest.mark.parametrize("option", [1, 2, 3, 5])
def test_optimizer_options_follow_the_reference_formulas(option):
    """AdaGrad (1), averaged gradient (2), SGD accumulating AdaGrad statistics (3) and Adam (5): three
    updates on different fractions against a float32 numpy restatement of the reference's functors
    (optimizers/SteepestDescentOptimizer.cu:127-194 with the constants of MacroDefine.hpp:39-42), fed
    with the gradients the GPU produced."""
    import b2lstm
    from b2lstm import workloads
    layers = L(("input", 5), ("blstm", 12), ("feedforward_identity", 3), ("sse", 3))
    P = 3
    w0 = workloads.make_weights(layers, 21, 0.2)
    net = b2lstm.Net(layers, P, 12)
    for i, wi in w0.items():
        net.set_weights(i, wi)
    net.set_optimizer(option)
    f32 = np.float32
    lr, mom = f32(1e-2), f32(0.9)
    w = {i: wi.copy() for i, wi in w0.items()}
    delta = {i: np.zeros_like(wi) for i, wi in w0.items()}
    stats = {i: (np.zeros(2 * wi.size, f32) if option == 5 else np.full(wi.size, 1e-6, f32)) for i, wi in w0.items()}
    b1 = b2 = f32(1.0)
    for k, lens in enumerate([[12, 9, 4], [7, 7, 7], [10, 2]]):
        lens = np.array(lens, np.int32)
        x, tg = workloads.make_fraction(5, 3, P, lens, 30 + k, 40 + k)
        net.load_fraction(lens, x, tg)
        net.forward()
        net.backward()
        g = {i: net.weight_updates(i) for i in w0}
        net.update_weights(float(lr), float(mom))
        n = f32(lens.sum())
        if option == 5:
            b1, b2 = f32(b1 * f32(0.9)), f32(b2 * f32(0.999))
        for i in w0:
            ave = (g[i] / n).astype(f32)
            if option == 2:
                gi = ave
            elif option in (1, 3):
                stats[i] = (stats[i] + ave * ave).astype(f32)
                gi = (ave / np.sqrt(stats[i])).astype(f32) if option == 1 else g[i]
            else:
                m = (stats[i][0::2] * f32(0.9) + ave * (f32(1.0) - f32(0.9))).astype(f32)
                v = (stats[i][1::2] * f32(0.999) + ave * ave * (f32(1.0) - f32(0.999))).astype(f32)
                stats[i][0::2], stats[i][1::2] = m, v
                gi = ((m / (f32(1.0) - b1)) / (np.sqrt(v / (f32(1.0) - b2)) + f32(1e-8))).astype(f32)
            delta[i] = (mom * delta[i] - lr * gi).astype(f32)
            w[i] = (w[i] + delta[i]).astype(f32)
            got = net.get_weights(i)
            assert np.allclose(got, w[i], rtol=2e-5, atol=1e-7), (option, k, i, np.abs(got - w[i]).max())
            if option != 2:
                assert np.allclose(net.optimizer_stats(i), stats[i], rtol=2e-5, atol=1e-6 * np.abs(stats[i]).max())
            else:
                assert net.optimizer_stats(i).size == 0
            w[i] = got                       # follow the device weights: the next gradients come from them
            net.set_weight_deltas(i, delta[i])
    net.set_optimizer(0)
    assert net.optimizer_stats(1).size == 0
    net.close()


@pytest.mark.parametrize("option", [3, 4])
def test_a_validation_stall_changes_the_schedule_of_options_3_and_4_instead_of_ending_the_run(tmp_path, option):
    """Optimizer::train, branch `m_epochsSinceLowestError >= m_maxEpochsNoBest` (Optimizer.cu:653-668).  Option 3
    (SGD while gathering AdaGrad statistics) turns into AdaGrad with the second learning rate and forgets the lowest
    validation error; option 4 multiplies the learning rate by the decay rate; both restore the best weights, go on
    with epochs_since_lowest_error = 1 and do not finish.  A learning rate too small to change an fp32 weight makes
    the validation error stall exactly."""
    import b2lstm
    from b2lstm import workloads
    w_true = np.random.default_rng(0).standard_normal((7, 3)).astype(np.float32)
    train = corpus(tmp_path, "train.nc", [20, 35, 28, 31, 25, 22, 38, 27], 1, w_true)
    valid = corpus(tmp_path, "valid.nc", [30, 24, 33], 2, w_true)
    P = 4
    w = workloads.make_weights(LAYERS, 9, 0.1)
    net = b2lstm.Net(LAYERS, P, 40)
    for i, wi in w.items():
        net.set_weights(i, wi)
    net.set_optimizer(option)
    tr, va = b2lstm.DataSet(train, P), b2lstm.DataSet(valid, P)
    opt = b2lstm.Optimizer(net, tr, va, learning_rate=1e-20, momentum=0.0, max_epochs=8, max_epochs_no_best=2,
                           second_learning_rate=0.02, lr_decay_rate=0.25)
    states = []
    for _ in range(3):
        assert not opt.train()
        states.append(opt.state)
    assert [s["epochs_since_lowest_error"] for s in states] == [0, 1, 1]      # third epoch: 2 >= 2, the branch sets 1
    assert states[0]["cur_validation_error"] == states[1]["cur_validation_error"] == states[2]["cur_validation_error"]
    assert states[1]["optimizer_option"] == option and states[1]["learning_rate"] == np.float32(1e-20)
    for i, wi in w.items():
        assert np.array_equal(net.get_weights(i), wi)                          # best weights restored (they never moved)
    if option == 3:
        assert states[2]["optimizer_option"] == 1 and states[2]["learning_rate"] == np.float32(0.02)
        assert states[2]["lowest_validation_error"] == np.finfo(np.float32).max
        assert not opt.train()                                                  # AdaGrad epoch on the gathered statistics
        s = opt.state
        assert s["lowest_validation_error"] == s["cur_validation_error"] and s["epochs_since_lowest_error"] == 0
        assert any(not np.array_equal(net.get_weights(i), wi) for i, wi in w.items())
    else:
        assert states[2]["optimizer_option"] == 4
        assert states[2]["learning_rate"] == np.float32(np.float32(1e-20) * np.float32(0.25))
        assert states[2]["lowest_validation_error"] == states[0]["cur_validation_error"]
    opt.close()
    net.close()


def test_batch_learning_sums_the_epoch_and_updates_once(tmp_path):
    """The reference without --hybrid_online_batch: the gradients of all fractions of an epoch are summed
    and ONE update follows.  Checked against the sum of the per-fraction gradients taken separately."""
    import b2lstm
    from b2lstm import workloads
    w_true = np.random.default_rng(0).standard_normal((7, 3)).astype(np.float32)
    path = corpus(tmp_path, "batch.nc", [20, 35, 28, 31, 25, 22, 38], 4, w_true)
    P = 3
    w = workloads.make_weights(LAYERS, 9, 0.1)
    lr, mom = 1e-4, 0.9

    net = b2lstm.Net(LAYERS, P, 40)
    for i, wi in w.items():
        net.set_weights(i, wi)
    ds = b2lstm.DataSet(path, P)
    gsum = {i: np.zeros_like(wi) for i, wi in w.items()}
    err = 0.0
    for f in ds.epoch():
        net.load_fraction(f["seq_lengths"], np.array(f["inputs"]), np.array(f["targets"]))
        err += net.forward() / ds.total_sequences
        net.backward()
        for i in w:
            gsum[i] = gsum[i] + net.weight_updates(i)
    got_err, frames = b2lstm.train_epoch_batch(net, ds, lr, mom)
    assert frames == ds.total_timesteps and abs(got_err - err) <= 1e-6 * abs(err)      # weights were still the initial ones
    for i, wi in w.items():
        want = wi + (-np.float32(lr) * gsum[i]).astype(np.float32)
        assert np.allclose(net.get_weights(i), want, rtol=1e-5, atol=1e-7)
        assert np.allclose(net.weight_deltas(i), -np.float32(lr) * gsum[i], rtol=1e-4, atol=1e-9)
    net.close()


def test_random_weights_follow_the_reference_stream():
    """Layers without a weights section are initialised as layers/TrainableLayer.cu:219-233 does with the default
    uniform distribution: one mt19937 (seed = --random_seed) for all layers in order, each weight
    boost::random::uniform_real_distribution<float>(0, max - min)(gen) + min.  Checked against a numpy restatement on
    the generator's raw 32-bit outputs (numpy's legacy RandomState seeds the same init_genrand; its first output for seed
    5489, 3499211612, is the generator's published known answer)."""
    import b2lstm
    from b2lstm.lib import lib
    assert int(np.random.RandomState(5489)._bit_generator.random_raw(1)[0]) == 3499211612
    for seed, (lo, hi) in [(0, (-0.1, 0.1)), (77, (-0.05, 0.3))]:
        lib().b2_config_set_weights_uniform(lo, hi)
        try:
            net = b2lstm.Net(LAYERS, 2, 8, seed=seed)
        finally:
            lib().b2_config_set_weights_uniform(-0.1, 0.1)
        raw = np.random.RandomState(seed)._bit_generator.random_raw(20000).astype(np.uint32)
        rng_f = np.float32(np.float32(hi) - np.float32(lo))
        cand = (raw.astype(np.float32) / np.float32(4294967296.0)) * rng_f          # float arithmetic throughout
        cand = cand[cand < rng_f]                                                    # a draw that rounds up to the range is repeated
        want = cand + np.float32(lo)
        k = 0
        for i, l in enumerate(LAYERS):
            if l["type"] in ("input", "sse"):
                continue
            got = net.get_weights(i)
            assert np.array_equal(got, want[k:k + got.size]), (seed, i)
            k += got.size
        net.close()


def test_forget_gate_bias_option_shifts_only_the_forget_biases_of_fresh_lstm_layers():
    """--lstm_forget_gate_bias of the reference (layers/LstmLayer.cu:1147-1161): the value is added to the forget-gate
    biases of randomly initialised (b)lstm layers and to nothing else; layers read from a weights section keep theirs."""
    import b2lstm
    from b2lstm.lib import lib
    layers = [dict(type="input", size=5), dict(type="feedforward_tanh", size=6, bias=1.0), dict(type="blstm", size=8, bias=1.0),
              dict(type="lstm", size=3, bias=1.0), dict(type="feedforward_identity", size=2, bias=1.0), dict(type="sse", size=2)]
    plain = b2lstm.Net(layers, 2, 4, seed=77)
    w0 = {i: plain.get_weights(i) for i in (1, 2, 3, 4)}
    plain.close()
    lib().b2_config_set_lstm_forget_gate_bias(1.5)
    try:
        shifted = b2lstm.Net(layers, 2, 4, seed=77)
        w1 = {i: shifted.get_weights(i) for i in (1, 2, 3, 4)}
        shifted.close()
        sizes = {1: (6, 5, 1), 2: (8, 6, 4), 3: (3, 8, 4), 4: (2, 3, 1)}      # layer: (size, preceding size, input weights per unit)
        section = {}
        for i, (ls, pls, per) in sizes.items():
            n_in, n_b = per * ls * pls, per * ls
            section["l%d" % i] = {"input": w0[i][:n_in].tolist(), "bias": w0[i][n_in:n_in + n_b].tolist(),
                                  "internal": w0[i][n_in + n_b:].tolist()}
        given = b2lstm.Net(layers, 2, 4, seed=77, weights=section)     # weights from the JSON section: untouched
        w2 = {i: given.get_weights(i) for i in (1, 2, 3, 4)}
        given.close()
    finally:
        lib().b2_config_set_lstm_forget_gate_bias(0.0)
    for i, (ls, pls) in {2: (8, 6), 3: (3, 8)}.items():
        d = w1[i] - w0[i]
        lo = 4 * ls * pls + 2 * ls
        assert np.allclose(d[lo:lo + ls], 1.5) and not d[:lo].any() and not d[lo + ls:].any()
    for i in (1, 4):
        assert np.array_equal(w1[i], w0[i])
    for i in (1, 2, 3, 4):
        assert np.array_equal(w2[i], w0[i])


def _mixed_net():
    from b2lstm import workloads
    layers = [dict(type="input", size=5), dict(type="feedforward_tanh", size=6, bias=1.0), dict(type="blstm", size=8, bias=0.5),
              dict(type="lstm", size=3, bias=1.0), dict(type="feedforward_identity", size=2, bias=1.0), dict(type="sse", size=2)]
    return layers, workloads.make_weights(layers, 5, 0.3)


def test_export_equals_what_the_reference_writes():
    """The network document against the reference's own writer: Layer::exportLayer, TrainableLayer::exportWeights
    (layers/TrainableLayer.cu:441-480) and its rapidjson PrettyWriter, run on the same weights.  Same layer entries,
    same section split (input | bias | internal) and, at the reference's 6 significant digits, the same numbers."""
    import b2lstm
    from oracle import OracleNet, ref_available
    if not ref_available():
        pytest.skip("the reference library (oracle/_ref) did not travel with the repository")
    layers, w = _mixed_net()
    ref = OracleNet(layers, 2, 4, "ref")
    net = b2lstm.Net(layers, 2, 4)
    for i, wi in w.items():
        ref.set_weights(i, wi)
        net.set_weights(i, wi)
    want = json.loads(ref.export_json())
    got = json.loads(net.export_json(digits=6))
    ref.close()
    net.close()
    assert [l["name"] for l in got["layers"]] == [l["name"] for l in want["layers"]]
    for a, b in zip(got["layers"], want["layers"]):
        for key in ("type", "size", "bias"):
            assert a.get(key) == b.get(key), (a, b)
    assert sorted(got["weights"]) == sorted(want["weights"])
    for name, sec in want["weights"].items():
        for part in ("input", "bias", "internal"):
            assert got["weights"][name][part] == sec[part], (name, part)


def test_network_files_travel_between_the_two_implementations():
    """A document the reference wrote is read by b2_net_create, and a document this library wrote (9 digits: exact for
    fp32) is read by the reference's TrainableLayer constructor (layers/TrainableLayer.cu:135-205)."""
    import b2lstm
    from oracle import OracleNet, ref_available
    if not ref_available():
        pytest.skip("the reference library (oracle/_ref) did not travel with the repository")
    layers, w = _mixed_net()
    ref = OracleNet(layers, 2, 4, "ref")
    for i, wi in w.items():
        ref.set_weights(i, wi)
    doc = json.loads(ref.export_json())
    ref.close()
    net = b2lstm.Net(layers, 2, 4, weights=doc["weights"])
    for i in w:
        sec = doc["weights"]["l%d" % i]
        written = np.array(sec["input"] + sec["bias"] + sec["internal"], np.float32)
        assert np.array_equal(net.get_weights(i), written)
        assert np.allclose(written, w[i], rtol=1e-5, atol=0)
    net.close()
    net = b2lstm.Net(layers, 2, 4)
    for i, wi in w.items():
        net.set_weights(i, wi)
    doc = json.loads(net.export_json())
    net.close()
    back = OracleNet(layers, 2, 4, "ref", weights_section=doc["weights"])
    for i in w:
        assert np.array_equal(back.get_weights(i), w[i])
    back.close()
