"""Host-side logic of data-parallel training: which sequences of a fraction a rank processes.

The reference sorts sequences by length before it builds fractions (data_sets/DataSet.cpp:1898-1900
of the reference), so dealing them in snake order (0..w-1, w-1..0, ...) gives every rank nearly the
same number of frames and nearly the same longest sequence.  Each rank pads only to its own longest sequence; gradients are sums over
frames, so the all-reduced sum equals the single-GPU gradient up to fp32 summation order.
"""
import numpy as np


def shard_indices(n_seqs, rank, world):
    """indices (into the length-sorted fraction) of the sequences rank `rank` of `world` processes"""
    i = np.arange(n_seqs)
    pos, rnd = i % world, i // world
    owner = np.where(rnd % 2 == 0, pos, world - 1 - pos)
    return i[owner == rank]


def shard_fraction(lens, x, tg, rank, world):
    """(lens, x, tg) of this rank's sequences: x [T,P,in] -> [T_r, P_r, in] with T_r the rank's own max length"""
    idx = shard_indices(len(lens), rank, world)
    if len(idx) == 0:
        raise ValueError("rank %d of %d has no sequence in a fraction of %d" % (rank, world, len(lens)))
    lens_r = np.ascontiguousarray(np.asarray(lens)[idx], np.int32)
    T = int(lens_r.max())
    return lens_r, np.ascontiguousarray(x[:T, idx]), np.ascontiguousarray(tg[:T, idx])


def frames_per_rank(lens, world):
    lens = np.asarray(lens)
    return [int(lens[shard_indices(len(lens), r, world)].sum()) for r in range(world)]
