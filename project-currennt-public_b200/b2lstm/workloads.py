"""The five benchmark configurations and their seeded synthetic data.

They stand in for the reference toolkit's speech-synthesis example data (382-dim linguistic
inputs, acoustic targets), whose files are not distributed.  Seeds: inputs 1000+cfg, targets
2000+cfg, weights 3000+cfg, lengths 4000+cfg (numpy Generator(PCG64)).  Weights are always
injected from these arrays into every implementation under comparison, never drawn twice.
"""
import numpy as np


def _L(*spec):
    out = []
    for ty, size in spec:
        d = {"type": ty, "size": size}
        if ty not in ("input", "sse"):
            d["bias"] = 1.0
        out.append(d)
    return out


CONFIGS = {
    0: dict(name="cfg0_plumbing_lstm128", P=4, len_lo=200, len_hi=200, wrange=0.08, binary_dims=0,
            layers=_L(("input", 64), ("lstm", 128), ("feedforward_identity", 32), ("sse", 32))),
    1: dict(name="cfg1_acoustic_2xff512_2xblstm256", P=32, len_lo=300, len_hi=1200, wrange=0.08, binary_dims=350,
            layers=_L(("input", 382), ("feedforward_tanh", 512), ("feedforward_tanh", 512), ("blstm", 512),
                      ("blstm", 512), ("feedforward_identity", 187), ("sse", 187))),
    2: dict(name="cfg2_deep_4xblstm1024", P=64, len_lo=2000, len_hi=2000, wrange=0.05, binary_dims=0,
            layers=_L(("input", 512), ("blstm", 2048), ("blstm", 2048), ("blstm", 2048), ("blstm", 2048),
                      ("feedforward_identity", 256), ("sse", 256))),
    3: dict(name="cfg3_latency_1x8000_2xblstm512", P=1, len_lo=8000, len_hi=8000, wrange=0.08, binary_dims=0,
            layers=_L(("input", 128), ("blstm", 1024), ("blstm", 1024), ("feedforward_identity", 80), ("sse", 80))),
    4: dict(name="cfg4_dp_256seq_3xblstm512", P=256, len_lo=600, len_hi=1000, wrange=0.08, binary_dims=350,
            layers=_L(("input", 382), ("blstm", 1024), ("blstm", 1024), ("blstm", 1024),
                      ("feedforward_identity", 187), ("sse", 187))),
}


def lstm_num_weights(prev, size, bidirectional):
    els = size // 2 if bidirectional else size
    return size * (4 * (prev + 1) + 4 * els + 3)


def layer_num_weights(layers, i):
    ty = layers[i]["type"]
    if ty.startswith("feedforward"):
        return layers[i]["size"] * (layers[i - 1]["size"] + 1)
    if ty in ("lstm", "blstm"):
        return lstm_num_weights(layers[i - 1]["size"], layers[i]["size"], ty == "blstm")
    return 0


def make_weights(layers, seed, wrange=0.08):
    """{layer index: float32 vector} drawn U(-wrange, wrange)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    out = {}
    for i in range(len(layers)):
        n = layer_num_weights(layers, i)
        if n:
            out[i] = rng.uniform(-wrange, wrange, n).astype(np.float32)
    return out


def make_lengths(P, lo, hi, seed, n_seqs=None):
    rng = np.random.Generator(np.random.PCG64(seed))
    n = P if n_seqs is None else n_seqs
    if lo == hi:
        return np.full(n, lo, np.int32)
    lens = rng.integers(lo, hi + 1, n).astype(np.int32)
    # the reference sorts sequences by length before building fractions (data_sets/DataSet.cpp:1898-1900)
    return np.sort(lens)[::-1].copy()


def make_fraction(in_dim, out_dim, P, lens, seed_in, seed_tg, binary_dims=0, target_scale=1.0, T=None):
    """inputs [T,P,in], targets [T,P,out], zero on padding frames (fraction layout of the reference)."""
    T = int(max(lens)) if T is None else T
    ri = np.random.Generator(np.random.PCG64(seed_in))
    rt = np.random.Generator(np.random.PCG64(seed_tg))
    x = ri.standard_normal((T, P, in_dim), dtype=np.float32)
    if binary_dims:
        x[:, :, :binary_dims] = (ri.random((T, P, binary_dims), dtype=np.float32) < 0.1).astype(np.float32)
    tg = rt.standard_normal((T, P, out_dim), dtype=np.float32) * np.float32(target_scale)
    for p in range(P):
        L = int(lens[p]) if p < len(lens) else 0
        x[L:, p] = 0
        tg[L:, p] = 0
    return x, tg


def build(cfg, scale_frames=1.0, P=None, rank=0):
    """Materialise configuration `cfg`: dict(layers, P, lens, x, tg, weights).  scale_frames < 1
    shortens every sequence (same layer sizes) for bounded CPU runs; P overrides the number of
    parallel sequences (data-parallel shards); rank offsets the data seeds."""
    c = CONFIGS[cfg]
    P = c["P"] if P is None else P
    lo, hi = max(1, int(c["len_lo"] * scale_frames)), max(1, int(c["len_hi"] * scale_frames))
    lens = make_lengths(P, lo, hi, 4000 + cfg + 100 * rank)
    layers = c["layers"]
    x, tg = make_fraction(layers[0]["size"], layers[-1]["size"], P, lens, 1000 + cfg + 100 * rank,
                          2000 + cfg + 100 * rank, c["binary_dims"])
    return dict(name=c["name"], layers=layers, P=P, lens=lens, x=x, tg=tg,
                weights=make_weights(layers, 3000 + cfg, c["wrange"]))


def gemm_flops_per_frame(layers):
    """Forward GEMM flops per frame (2*m*k per dense product); training is 3x this."""
    f = 0
    for i in range(1, len(layers)):
        ty, ls, pls = layers[i]["type"], layers[i]["size"], layers[i - 1]["size"]
        if ty.startswith("feedforward"):
            f += 2 * ls * pls
        elif ty in ("lstm", "blstm"):
            els = ls // 2 if ty == "blstm" else ls
            f += 8 * ls * pls + 8 * ls * els
    return f


def write_nc(wl, path):
    """Writes a built workload as a data set in the toolkit's .nc layout (sequences back to back,
    padding frames dropped); reading it with parallel_sequences = wl["P"] and training_mode off
    gives back the same fraction."""
    from .lib import write_nc as _write
    P, lens = wl["P"], wl["lens"]
    T = int(lens.max())
    x = np.asarray(wl["x"]).reshape(T, P, -1)
    tg = np.asarray(wl["tg"]).reshape(T, P, -1)
    xs = np.concatenate([x[:int(n), p] for p, n in enumerate(lens)], axis=0)
    ts = np.concatenate([tg[:int(n), p] for p, n in enumerate(lens)], axis=0)
    _write(path, ["seq%05d" % p for p in range(P)], [int(n) for n in lens], xs, ts)
