"""GPU parity tests: the CUDA path, called through the C ABI (ctypes), against
(1) the golden tensors produced by the reference's own Cpu code,
(2) the checker on fresh seeded inputs: the compiled reference where it travelled with the
    repository, otherwise the C restatement that the CPU tests pin to it,
for every recurrence / GEMM variant the library offers."""
import numpy as np
import pytest

import parity
from make_golden import run as run_kind
from oracle import ref_available

pytestmark = pytest.mark.gpu

VARIANTS = [dict(recurrence=0, ffma=1), dict(recurrence=1, ffma=1), dict(recurrence=1, ffma=0), dict(recurrence=2, ffma=0),
            dict(recurrence=3, ffma=0), dict(recurrence=0, ffma=0), dict(recurrence=4, ffma=0)]
VARIANT_IDS = ["stepwise-ffma", "persistent-ffma", "persistent-tensor", "persistent_cluster-tensor", "tensor_recurrence-tensor",
               "stepwise-tensor", "persistent_l2-tensor"]


def run_gpu(layers, P, lens, x, tg, weights, variant, lr=1e-4, mom=0.9, maxT=None, paths=None):
    """paths: optional dict that receives {layer: (forward path, backward path)} of the (b)lstm layers"""
    import b2lstm
    net = b2lstm.Net(layers, P, maxT or x.shape[0])
    net.set_recurrence_mode(variant["recurrence"])
    net.set_force_ffma(variant["ffma"])
    for i, w in weights.items():
        net.set_weights(i, w)
    net.load_fraction(lens, x, tg)
    out = {"loss": net.forward()}
    for i in range(1, len(layers)):
        if layers[i]["type"] != "sse":
            out["out%d" % i] = net.outputs(i)
    net.backward()
    for i in range(1, len(layers)):
        # what a layer received as output errors: a feed-forward layer turns them into deltas in
        # place (as the reference does), an lstm layer leaves them untouched -> compare lstm inputs
        if layers[i]["type"] in ("lstm", "blstm"):
            out["dyin%d" % i] = net.output_errors(i)
        if i in weights:
            out["dw%d" % i] = net.weight_updates(i)
    net.update_weights(lr, mom)
    net.synchronize()
    if paths is not None:
        paths.update(net.recurrence_paths())
    for i in weights:
        out["wnew%d" % i] = net.get_weights(i)
    out["launches"] = net.launch_count
    net.close()
    return out


@pytest.mark.parametrize("variant", VARIANTS, ids=VARIANT_IDS)
@pytest.mark.parametrize("name", parity.golden_cases())
def test_golden(name, variant):
    g = parity.load_golden(name)
    got = run_gpu(g["layers"], g["P"], g["lens"], g["x"], g["tg"], g["weights"], variant)
    assert got["launches"] > 0
    parity.compare_run(g["layers"], got, g, name, lstm_pad_zero_lens=g["lens"])
    for i in g["weights"]:
        parity.assert_rel_close(got["wnew%d" % i] - g["w%d" % i], g["wnew%d" % i] - g["w%d" % i],
                                "%s weight step of layer %d" % (name, i))


def checker():
    return "ref" if ref_available() else "port"


def L(*spec):
    return [dict(type=t, size=s, **({} if t in ("input", "sse") else {"bias": 1.0})) for t, s in spec]


SHAPES = []
for els in (1, 3, 32, 33):
    for P in (1, 3):
        for T in (1, 2, 5):
            for bi in (0, 1):
                SHAPES.append((els, P, T, bi))


@pytest.mark.parametrize("variant", VARIANTS[:4], ids=VARIANT_IDS[:4])
def test_small_shapes_exhaustive(variant):
    """els in {1,3,32,33} x P in {1,3} x T in {1,2,5} x uni/bi, ragged lengths, run twice (determinism)."""
    from b2lstm import workloads
    for k, (els, P, T, bi) in enumerate(SHAPES):
        ls = els * (2 if bi else 1)
        layers = L(("input", 5), ("blstm" if bi else "lstm", ls), ("feedforward_identity", 3), ("sse", 3))
        lens = np.array([T] + [max(1, T - 1 - p) for p in range(P - 1)], np.int32)
        x, tg = workloads.make_fraction(5, 3, P, lens, 500 + k, 600 + k)
        w = workloads.make_weights(layers, 700 + k, 0.3)
        want = run_kind(checker(), layers, P, lens, x, tg, w)
        got = run_gpu(layers, P, lens, x, tg, w, variant)
        parity.compare_run(layers, got, want, "els%d P%d T%d bi%d" % (els, P, T, bi), lstm_pad_zero_lens=lens)
        again = run_gpu(layers, P, lens, x, tg, w, variant)
        for key in got:
            if key != "launches":
                assert np.array_equal(np.asarray(got[key]), np.asarray(again[key])), "not deterministic: " + key


@pytest.mark.parametrize("variant", VARIANTS[:5], ids=VARIANT_IDS[:5])
def test_cfg0_full(variant):
    """Configuration 0 at full size: 64 -> lstm 128 -> ff 32 -> sse, 4 x 200 frames."""
    from b2lstm import workloads
    wl = workloads.build(0)
    want = run_kind(checker(), wl["layers"], wl["P"], wl["lens"], wl["x"], wl["tg"], wl["weights"])
    got = run_gpu(wl["layers"], wl["P"], wl["lens"], wl["x"], wl["tg"], wl["weights"], variant)
    parity.compare_run(wl["layers"], got, want, "cfg0")


@pytest.mark.parametrize("variant", VARIANTS[1:5], ids=VARIANT_IDS[1:5])
@pytest.mark.parametrize("cfg,P,scale", [(1, 6, 0.04), (3, 1, 0.01), (4, 5, 0.03)])
def test_config_layer_sizes_reduced_frames(cfg, P, scale, variant):
    """Configurations 1, 3, 4 with their real layer sizes on a reduced frame budget (the checker is
    a serial CPU program): ragged lengths, padding, both directions, 256/512-unit recurrences."""
    from b2lstm import workloads
    wl = workloads.build(cfg, scale_frames=scale, P=P)
    want = run_kind(checker(), wl["layers"], wl["P"], wl["lens"], wl["x"], wl["tg"], wl["weights"])
    got = run_gpu(wl["layers"], wl["P"], wl["lens"], wl["x"], wl["tg"], wl["weights"], variant)
    parity.compare_run(wl["layers"], got, want, "cfg%d reduced" % cfg, lstm_pad_zero_lens=wl["lens"])


def test_cfg2_stack_takes_the_large_batch_recurrence():
    """Configuration 2's own stack (512 -> 4x blstm 1024/direction -> 256) with 16 parallel sequences on a few
    frames, recurrence mode 1 (the library chooses): the choice must be a tensor-core recurrence, as for the
    full-size workload, and the result must match the checker."""
    from b2lstm import workloads
    wl = workloads.build(2, scale_frames=0.004, P=16)
    want = run_kind(checker(), wl["layers"], wl["P"], wl["lens"], wl["x"], wl["tg"], wl["weights"])
    paths = {}
    got = run_gpu(wl["layers"], wl["P"], wl["lens"], wl["x"], wl["tg"], wl["weights"], dict(recurrence=1, ffma=0), paths=paths)
    assert sorted(paths) == [1, 2, 3, 4]
    for i, (f, b) in paths.items():
        assert f in ("tensor_core_per_step", "persistent_tensor_core") and b == f, (i, f, b)
    parity.compare_run(wl["layers"], got, want, "cfg2 stack", lstm_pad_zero_lens=wl["lens"])


def test_cfg1_fraction_at_full_size_against_the_reference():
    """One fraction of configuration 1 at FULL size (32 sequences of 300..1200 frames, about 24k frames): error,
    every layer's outputs, the output errors into the blstm layers and every gradient block against the
    reference's own code (its OpenMP host build: same sources and the same per-weight summation order as the
    serial build, about a minute on the host cores)."""
    from b2lstm import workloads
    from oracle import ref_available
    if not ref_available(omp=True):
        pytest.skip("the OpenMP build of the reference did not travel with the repository")
    import os
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    wl = workloads.build(1)
    want = run_kind("ref_omp", wl["layers"], wl["P"], wl["lens"], wl["x"], wl["tg"], wl["weights"])
    paths = {}
    got = run_gpu(wl["layers"], wl["P"], wl["lens"], wl["x"], wl["tg"], wl["weights"], dict(recurrence=1, ffma=0), paths=paths)
    print("cfg1 full size: recurrence paths", paths, "error", got["loss"], "reference", want["loss"])
    # The reference adds the 4.5 million squared differences of this fraction in fp32 (SsePostOutputLayer.cu:197-209);
    # the library accumulates in double.  The error bound is widened to what fp32 accumulation of that many terms
    # can lose; every other quantity keeps its bound.
    parity.compare_run(wl["layers"], got, want, "cfg1 full size", lstm_pad_zero_lens=wl["lens"], loss_rtol=5e-4)


@pytest.mark.parametrize("variant", VARIANTS[1:5] + VARIANTS[6:], ids=VARIANT_IDS[1:5] + VARIANT_IDS[6:])
@pytest.mark.parametrize("ls,bi,P,lens", [(2048, 1, 5, [12, 12, 7, 3, 12]), (1024, 0, 1, [9]), (256, 1, 9, [14] * 9),
                                          (256, 0, 1, [11]), (128, 0, 1, [12]), (512, 1, 1, [8]),
                                          (512, 1, 32, [9] * 30 + [5, 2]), (512, 1, 38, [6] * 37 + [3]), (256, 1, 34, [7] * 34),
                                          (512, 1, 2, [6, 11]), (256, 0, 7, [10, 9, 8, 7, 6, 5, 4]),
                                          (512, 1, 40, [7] * 20 + [5] * 19 + [2]), (512, 1, 83, [5] * 80 + [3, 2, 1]),
                                          (1024, 1, 9, [6] * 8 + [4]), (1024, 1, 21, [5] * 21), (256, 1, 150, [3] * 150)])
def test_persistent_geometries(ls, bi, P, lens, variant):
    """Every register-resident geometry of the persistent kernels (128/256/512/1024 units per
    direction, 1 or 4 sequences per group, sequence counts that do not fill the last group)."""
    from b2lstm import workloads
    layers = L(("input", 16), ("blstm" if bi else "lstm", ls), ("feedforward_identity", 8), ("sse", 8))
    lens = np.array(lens, np.int32)
    x, tg = workloads.make_fraction(16, 8, P, lens, 31, 32)
    w = workloads.make_weights(layers, 33, 0.05)
    want = run_kind(checker(), layers, P, lens, x, tg, w)
    got = run_gpu(layers, P, lens, x, tg, w, variant)
    parity.compare_run(layers, got, want, "ls%d bi%d P%d" % (ls, bi, P), lstm_pad_zero_lens=lens)


@pytest.mark.parametrize("mode", [6, 5], ids=["forward_only", "forward_and_backward"])
@pytest.mark.parametrize("ls,bi,P,lens", [(1024, 1, 16, [14] * 10 + [12, 9, 9, 5, 2, 1]),
                                          (1024, 1, 32, [9] * 30 + [5, 2]),
                                          (1024, 1, 5, [12, 12, 7, 3, 12]),
                                          (512, 0, 20, [11] * 12 + [10, 9, 8, 7, 6, 5, 4, 3]),
                                          (1024, 1, 40, [7] * 20 + [5] * 19 + [2]),
                                          (1024, 1, 83, [6] * 80 + [3, 2, 1]),
                                          (1024, 1, 150, [4] * 100 + [3] * 50)])
def test_persistent_tensor_core_recurrence(ls, bi, P, lens, mode):
    """The persistent tensor-core kernels (512 units per direction; recurrent weights resident in shared memory
    as fp16 hi/lo operands): one chunk and several chunks per group of blocks, chunks of 16 and of 32 sequences,
    sequence counts that do not fill the last chunk, ragged lengths, one and two directions.  Mode 6 runs only
    the forward sweep on them (the backward sweep on the FFMA kernels), mode 5 both."""
    from b2lstm import workloads
    layers = L(("input", 16), ("blstm" if bi else "lstm", ls), ("feedforward_identity", 8), ("sse", 8))
    lens = np.array(lens, np.int32)
    x, tg = workloads.make_fraction(16, 8, P, lens, 51, 52)
    w = workloads.make_weights(layers, 53, 0.08)
    want = run_kind(checker(), layers, P, lens, x, tg, w)
    paths = {}
    got = run_gpu(layers, P, lens, x, tg, w, dict(recurrence=mode, ffma=0), paths=paths)
    assert paths[1][0] == "persistent_tensor_core", paths
    assert paths[1][1] == ("persistent_tensor_core" if mode == 5 else "persistent_ffma"), paths
    parity.compare_run(layers, got, want, "ls%d bi%d P%d" % (ls, bi, P), lstm_pad_zero_lens=lens)
    again = run_gpu(layers, P, lens, x, tg, w, dict(recurrence=mode, ffma=0))
    for key in got:
        if key != "launches":
            assert np.array_equal(np.asarray(got[key]), np.asarray(again[key])), "not deterministic: " + key


@pytest.mark.parametrize("P,lens", [(40, [9] * 20 + [8] * 10 + [5] * 10), (64, [7] * 40 + [6] * 20 + [2] * 4),
                                    (100, [6] * 70 + [4] * 30), (130, [5] * 128 + [3, 2]), (180, [4] * 170 + [3] * 10)])
def test_chunk_plans_of_the_tensor_core_recurrence_agree(P, lens):
    """b2_config_set_ptc_plan changes how the sequences of a fraction are grouped into chunks and which exchange
    carries h and the partial errors between the blocks (step counters + bulk copies, or self-validating words collected
    by the cell warps or by gather warps; one, two or more chunks in flight).  The arithmetic per cell does not depend on it: every plan must give the same bits,
    and the default plan must agree with the reference."""
    from b2lstm import workloads
    from b2lstm.lib import lib
    layers = L(("input", 16), ("blstm", 1024), ("feedforward_identity", 8), ("sse", 8))
    lens = np.array(lens, np.int32)
    x, tg = workloads.make_fraction(16, 8, P, lens, 71, 72)
    w = workloads.make_weights(layers, 73, 0.08)
    want = run_kind(checker(), layers, P, lens, x, tg, w)
    runs = {}
    try:
        for plan in [None, (1, 1), (2, 1), (2, 2), (1, 4), (3, 3), (1, 1, 8)]:
            if plan is None:
                lib().b2_config_set_ptc_plan(0, 1, 1, 0)
                lib().b2_config_set_ptc_plan(1, 2, 5, 6)
            else:
                for backward in (0, 1):
                    lib().b2_config_set_ptc_plan(backward, plan[0], plan[1], plan[2] if len(plan) > 2 else 0)
            paths = {}
            runs[plan] = run_gpu(layers, P, lens, x, tg, w, dict(recurrence=5, ffma=0), paths=paths)
            assert paths[1] == ("persistent_tensor_core", "persistent_tensor_core"), paths
    finally:
        lib().b2_config_set_ptc_plan(0, 1, 1, 0)
        lib().b2_config_set_ptc_plan(1, 2, 5, 6)
    parity.compare_run(layers, runs[None], want, "default plan, P%d" % P, lstm_pad_zero_lens=lens)
    for plan, got in runs.items():
        for key in got:
            if key != "launches":
                assert np.array_equal(np.asarray(got[key]), np.asarray(runs[None][key])), (plan, key)


def test_persistent_tensor_core_recurrence_with_large_weights_and_activations():
    """Recurrent weights far from the usual range (one direction scaled by 40, the other by 1/300) and targets
    that drive the deltas into the clip: the per-direction power-of-two scale of the fp16 operands must keep
    the result within the same bounds.  Two frames only: with weights this large the recurrence amplifies any
    rounding difference tenfold per step, so longer sequences compare chaos, not arithmetic."""
    from b2lstm import workloads
    layers = L(("input", 16), ("blstm", 1024), ("feedforward_identity", 8), ("sse", 8))
    P, lens = 16, np.array([2] * 14 + [1, 1], np.int32)
    x, tg = workloads.make_fraction(16, 8, P, lens, 61, 62, target_scale=300.0)
    w = workloads.make_weights(layers, 63, 0.02)
    ls, els, pls = 1024, 512, 16
    rec = w[1][4 * ls * (pls + 1):4 * ls * (pls + 1) + 4 * ls * els].reshape(4, 2, els, els)
    rec[:, 0] *= 40.0
    rec[:, 1] /= 300.0
    want = run_kind(checker(), layers, P, lens, x, tg, w)
    got = run_gpu(layers, P, lens, x, tg, w, dict(recurrence=5, ffma=0))
    parity.compare_run(layers, got, want, "scaled recurrent weights", lstm_pad_zero_lens=lens)


@pytest.mark.parametrize("variant", [VARIANTS[2], VARIANTS[5]], ids=[VARIANT_IDS[2], VARIANT_IDS[5]])
@pytest.mark.parametrize("ls,bi,P,lens", [(320, 1, 8, [40] * 6 + [33, 21]), (200, 0, 6, [50, 50, 47, 30, 22, 9]),
                                          (150, 0, 5, [60, 55, 50, 45, 40]), (384, 1, 4, [70, 64, 31, 70])])
def test_unit_counts_that_do_not_fill_tiles(ls, bi, P, lens, variant):
    """Units per direction that are no multiple of the 128-wide GEMM tile (160, 200, 150, 192) with
    products large enough for the tensor-core kernels: the batched recurrent-weight-gradient launch reads
    tiles that hang over into the other direction's columns and must not let them leak into the result."""
    from b2lstm import workloads
    layers = L(("input", 24), ("blstm" if bi else "lstm", ls), ("feedforward_identity", 8), ("sse", 8))
    lens = np.array(lens, np.int32)
    x, tg = workloads.make_fraction(24, 8, P, lens, 41, 42)
    w = workloads.make_weights(layers, 43, 0.05)
    want = run_kind(checker(), layers, P, lens, x, tg, w)
    got = run_gpu(layers, P, lens, x, tg, w, variant)
    parity.compare_run(layers, got, want, "ls%d bi%d P%d" % (ls, bi, P), lstm_pad_zero_lens=lens)


def test_reuse_across_fractions_of_different_length():
    """A net sized for the longest fraction processes shorter and longer fractions back to back
    (stale state in the buffers must not leak into the next fraction)."""
    import b2lstm
    from b2lstm import workloads
    layers = L(("input", 6), ("blstm", 20), ("lstm", 7), ("feedforward_identity", 3), ("sse", 3))
    P = 4
    w = workloads.make_weights(layers, 42, 0.2)
    net = b2lstm.Net(layers, P, 30)
    for i, wi in w.items():
        net.set_weights(i, wi)
    for k, lens in enumerate([[30, 22, 30, 4], [7, 7, 3], [19], [30, 30, 30, 30]]):
        lens = np.array(lens, np.int32)
        x, tg = workloads.make_fraction(6, 3, P, lens, 900 + k, 950 + k)
        want = run_kind(checker(), layers, P, lens, x, tg, w)
        net.load_fraction(lens, x, tg)
        got = {"loss": net.forward()}
        net.backward()
        for i in (1, 2, 3):
            got["out%d" % i] = net.outputs(i)
            got["dw%d" % i] = net.weight_updates(i)
        parity.compare_run(layers, got, want, "fraction %d" % k, lstm_pad_zero_lens=lens)
    net.close()


def test_prefetched_steps_equal_plain_steps():
    """Three train steps on three different fractions: once with b2_net_train_step (copy, then
    compute), once with the copy of the next fraction prefetched under the current step.  Same
    errors and bit-identical weights."""
    import torch
    import b2lstm
    from b2lstm import workloads
    layers = L(("input", 12), ("blstm", 256), ("feedforward_identity", 5), ("sse", 5))
    P = 6
    w = workloads.make_weights(layers, 61, 0.1)
    fracs = []
    for k, lens in enumerate([[20, 20, 11, 9, 4, 2], [13] * 6, [25, 3, 3]]):
        lens = np.array(lens, np.int32)
        x, tg = workloads.make_fraction(12, 5, P, lens, 70 + k, 80 + k)
        fracs.append((lens, torch.from_numpy(x).pin_memory(), torch.from_numpy(tg).pin_memory()))
    results = []
    for mode in ("plain", "prefetched"):
        net = b2lstm.Net(layers, P, 25)
        for i, wi in w.items():
            net.set_weights(i, wi)
        errs = []
        if mode == "plain":
            for lens, x, tg in fracs:
                errs.append(net.train_step(lens, x.numpy(), tg.numpy(), 1e-3, 0.9))
        else:
            net.prefetch_fraction(fracs[0][0], fracs[0][1].numpy(), fracs[0][2].numpy())
            for k in range(len(fracs)):
                net.train_step_prefetched(1e-3, 0.9, want_error=False)
                if k + 1 < len(fracs):
                    net.prefetch_fraction(fracs[k + 1][0], fracs[k + 1][1].numpy(), fracs[k + 1][2].numpy())
                errs.append(net.read_error())
        net.synchronize()
        results.append((errs, {i: net.get_weights(i) for i in w}))
        net.close()
    assert results[0][0] == results[1][0]
    for i in w:
        assert np.array_equal(results[0][1][i], results[1][1][i])
        assert not np.array_equal(results[0][1][i], w[i])


def test_layer_level_entry_points_on_caller_buffers():
    """b2_lstm_* on torch-owned device buffers, the drop-in for layers::LstmLayer<Gpu>."""
    import torch
    import b2lstm
    from b2lstm import workloads
    P, T, pls, ls = 3, 9, 6, 10
    layers = L(("input", pls), ("blstm", ls), ("feedforward_identity", 4), ("sse", 4))
    lens = np.array([9, 5, 9], np.int32)
    x, tg = workloads.make_fraction(pls, 4, P, lens, 11, 12)
    w = workloads.make_weights(layers, 13, 0.3)
    want = run_kind(checker(), layers, P, lens, x, tg, w)
    dev = torch.device("cuda:0")
    pat = np.zeros((T, P), np.int8)
    for p, n in enumerate(lens):
        pat[:n, p] = 2
        pat[0, p] = 1
        pat[n - 1, p] = 3
    layer = b2lstm.LstmLayer(P, T, pls, ls, True, 1.0)
    assert layer.num_weights == w[1].size
    tw, tx = torch.from_numpy(w[1]).to(dev), torch.from_numpy(x).to(dev)
    tpat = torch.from_numpy(pat).to(dev)
    ty = torch.full((T, P, ls), float("nan"), device=dev)
    layer.load_sequences(T, int(lens.min()), tpat)
    layer.forward(tw, tx, ty)
    torch.cuda.synchronize()
    parity.assert_outputs_close(ty.cpu().numpy(), want["out1"], "layer-level outputs")
    tdy = torch.from_numpy(want["dyin1"]).to(dev)
    tdx = torch.full((T, P, pls), float("nan"), device=dev)
    tdw = torch.full((layer.num_weights,), float("nan"), device=dev)
    layer.backward(tw, tx, ty, tdy, tdx, tdw)
    torch.cuda.synchronize()
    parity.assert_grads_close(layers, 1, tdw.cpu().numpy(), want["dw1"], "layer-level")
    assert np.isfinite(tdx.cpu().numpy()).all()
    layer.close()


def test_matrix_multiply_wrapper():
    """b2_matrix_multiply = helpers::Matrix::assignProduct/addProduct, every transpose the reference
    supports, ragged sizes, against float64 numpy."""
    import torch
    import b2lstm
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(5)
    for (m, n, k) in [(1, 1, 1), (7, 5, 3), (128, 128, 64), (130, 70, 257), (64, 512, 800), (384, 96, 4100)]:
        for ta, tb in [(0, 0), (1, 0), (0, 1)]:
            for ffma in (1, 0):
                A = rng.standard_normal((k, m) if not ta else (m, k)).astype(np.float32)   # stored column-major
                B = rng.standard_normal((n, k) if not tb else (k, n)).astype(np.float32)
                C0 = rng.standard_normal((n, m)).astype(np.float32)
                opA = A.T.astype(np.float64) if not ta else A.astype(np.float64)          # m x k
                opB = B.T.astype(np.float64) if not tb else B.astype(np.float64)          # k x n
                want = opA @ opB
                tA, tB, tC = torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev), torch.from_numpy(C0).to(dev)
                lda = m if not ta else k
                ldb = k if not tb else n
                b2lstm.matrix_multiply(tC, m, tA, lda, ta, tB, ldb, tb, m, n, k, accumulate=False, force_ffma=ffma)
                torch.cuda.synchronize()
                got = tC.cpu().numpy().T
                scale = np.sqrt(k)
                assert np.abs(got - want).max() <= 2e-6 * scale * 8, (m, n, k, ta, tb, ffma, np.abs(got - want).max())
                b2lstm.matrix_multiply(tC, m, tA, lda, ta, tB, ldb, tb, m, n, k, accumulate=True, force_ffma=ffma)
                torch.cuda.synchronize()
                assert np.abs(tC.cpu().numpy().T - 2 * want).max() <= 4e-6 * scale * 8


def test_tensor_core_gemm_keeps_fp32_accuracy_on_long_contractions():
    """The weight-gradient products contract over all frames of a fraction (tens of thousands of
    terms).  The tensor-core kernel (fp16 high/low operand parts) must stay as close to the float64 result as a plain fp32
    FFMA kernel does: relative L2 error below 2e-6 and within a small factor of the FFMA error."""
    import torch
    import b2lstm
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(11)
    for (m, n, k) in [(256, 384, 40000), (512, 2048, 9000)]:
        A = (rng.standard_normal((k, m)) * 0.5).astype(np.float32)        # m x k column-major
        B = (rng.standard_normal((k, n)) * 0.1).astype(np.float32)        # B^T stored n x k col-major -> transB
        want = A.T.astype(np.float64) @ B.astype(np.float64)
        tA, tB = torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)
        errs = {}
        for ffma in (1, 0):
            tC = torch.zeros((n, m), device=dev)
            b2lstm.matrix_multiply(tC, m, tA, m, 0, tB, n, 1, m, n, k, accumulate=False, force_ffma=ffma)
            torch.cuda.synchronize()
            got = tC.cpu().numpy().T.astype(np.float64)
            errs[ffma] = np.linalg.norm(got - want) / np.linalg.norm(want)
        print("gemm %dx%dx%d rel L2 error: ffma %.3g tensor %.3g" % (m, n, k, errs[1], errs[0]))
        assert errs[0] < 2e-6 and errs[0] < 8 * errs[1] + 2e-7, errs


def test_tensor_core_gemm_over_operand_magnitudes_and_dynamic_range():
    """The fp16 operand parts carry a power-of-two scale per operand, taken from its largest finite entry.  Products of
    very small, very large and all-zero operands, and of operands whose entries span many orders of magnitude (the
    deltas of a long sequence do), must stay at fp32 accuracy against float64: per row of the result, the error is
    measured against the row's own scale sum_k |a_ik||b_kj|."""
    import torch
    import b2lstm
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(17)
    m, n, k = 256, 320, 4096
    base_a = rng.standard_normal((k, m))
    base_b = rng.standard_normal((k, n))
    # rows of A whose entries are 1e-6 .. 1 of the largest; the same over the contraction index for B
    spread_a = base_a * (10.0 ** rng.uniform(-6, 0, size=(1, m)))
    spread_b = base_b * (10.0 ** rng.uniform(-6, 0, size=(k, 1)))
    cases = [("small", base_a * 1e-22, base_b * 1e-12), ("large", base_a * 1e15, base_b * 1e12),
             ("mixed", base_a * 1e-20, base_b * 1e18), ("spread", spread_a, spread_b),
             ("zero", base_a * 0.0, base_b)]
    for name, a64, b64 in cases:
        A, B = a64.astype(np.float32), b64.astype(np.float32)
        want = A.T.astype(np.float64) @ B.astype(np.float64)
        mag = np.abs(A.T.astype(np.float64)) @ np.abs(B.astype(np.float64))
        tA, tB = torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)
        tC = torch.full((n, m), 7.0, device=dev)
        b2lstm.matrix_multiply(tC, m, tA, m, 0, tB, n, 1, m, n, k, accumulate=False, force_ffma=0)
        torch.cuda.synchronize()
        got = tC.cpu().numpy().T.astype(np.float64)
        assert np.isfinite(got).all(), name
        if name == "zero":
            assert (got == 0.0).all()
            continue
        rel = np.abs(got - want) / mag
        print("gemm operands %-6s: largest error / sum|a||b| = %.3g" % (name, rel.max()))
        assert rel.max() < 3e-7, (name, rel.max())


def test_padding_that_does_not_trail_its_sequence_is_refused_when_the_check_is_on():
    import torch
    import b2lstm
    P, T = 3, 6
    layer = b2lstm.LstmLayer(P, T, 4, 6, True, 1.0)
    pat = np.full((T, P), 2, np.int8)
    pat[4:, 1] = 0                               # sequence 1: padding from frame 4 on (fine)
    good = torch.from_numpy(pat.copy()).cuda()
    pat[2, 2] = 0                                # sequence 2: a padding frame in the middle
    bad = torch.from_numpy(pat).cuda()
    layer.load_sequences(T, 4, bad)              # unchecked by default, as before
    layer.set_check_padding(True)
    layer.load_sequences(T, 4, good)
    with pytest.raises(b2lstm.B2Error, match="padding must trail"):
        layer.load_sequences(T, 4, bad)
    layer.close()


def test_errors_are_status_codes():
    import b2lstm
    layers = L(("input", 4), ("lstm", 4), ("sse", 4))
    net = b2lstm.Net(layers, 2, 5)
    with pytest.raises(b2lstm.B2Error):
        net.forward()                       # nothing loaded
    with pytest.raises(b2lstm.B2Error):
        net.load_fraction(np.array([9], np.int32), np.zeros((9, 2, 4), np.float32), np.zeros((9, 2, 4), np.float32))
    net.close()


def test_a_wait_that_nothing_satisfies_runs_out_and_leaves_the_context_usable():
    """The failure path of the persistent kernels without any fault: a block waits, with the sweeps' own
    bounded wait, for a step tag that nothing writes.  The wait runs out, the kernel records
    B2_ERR_STEP_TIMEOUT and returns; afterwards the same context trains a step with correct results."""
    import time
    import b2lstm
    from b2lstm import workloads
    from b2lstm.lib import selftest_bounded_wait
    t0 = time.time()
    status, gave_up = selftest_bounded_wait()
    assert status == -3 and gave_up                 # B2_ERR_STEP_TIMEOUT
    assert time.time() - t0 < 30.0
    layers = L(("input", 6), ("blstm", 256), ("feedforward_identity", 3), ("sse", 3))
    lens = np.array([9, 7, 9, 4], np.int32)
    x, tg = workloads.make_fraction(6, 3, 4, lens, 11, 12)
    w = workloads.make_weights(layers, 13, 0.1)
    want = run_kind(checker(), layers, 4, lens, x, tg, w)
    got = run_gpu(layers, 4, lens, x, tg, w, VARIANTS[2])
    parity.compare_run(layers, got, want, "after the timed-out wait", lstm_pad_zero_lens=lens)
