"""CPU tests of the .nc reader and the fraction assembler (b2_data_*): host code, no GPU needed.

The checker is a numpy restatement of the reference's DataSet constructor and _makeFractionTask
(data_sets/DataSet.cpp:1443-1500 segment table, :1898-1900 sort, :491-519 shuffles, :640-1020
fraction layout).  The reference's own DataSet.cpp needs libnetcdf and Boost and cannot be built
here; files are written with scipy's netcdf_file exactly as the reference's
pyTools/dataTools/ncDataHandle.py writes them.
"""
import os

import numpy as np
import pytest

import b2lstm
from b2lstm.lib import B2Error


def make_corpus(seed, lens, n_in=5, n_out=3):
    rng = np.random.default_rng(seed)
    n = int(sum(lens))
    x = rng.standard_normal((n, n_in)).astype(np.float32)
    y = rng.standard_normal((n, n_out)).astype(np.float32)
    tags = ["utt_%03d_%d" % (i, seed) for i in range(len(lens))]
    return tags, list(lens), x, y


def segments(lens, tags, trunc):
    """segment table of one file: (tag, index in utterance, first frame in the file, length)"""
    out, frame = [], 0
    for tag, n in zip(tags, lens):
        k = 0
        while n > 0:
            ln = min(trunc, n) if (trunc > 0 and n > 1.5 * trunc) else n
            out.append((tag, k, frame, ln))
            n -= ln
            frame += ln
            k += 1
    return out


def check_fraction(f, P, source):
    """every slot of the fraction holds the frames of the sequence it names, padding is zero / NONE"""
    T, n = f["T"], f["num_sequences"]
    assert T == max(f["seq_lengths"]) and f["min_seq_length"] == min(f["seq_lengths"])
    assert f["total_frames"] == int(sum(f["seq_lengths"]))
    assert f["inputs"].shape[:2] == (T, P) and f["pat_types"].shape == (T, P)
    for i in range(P):
        if i < n:
            x, y, begin = source[(f["tags"][i], f["original_seq_idx"][i])]
            ln = int(f["seq_lengths"][i])
            assert np.array_equal(f["inputs"][:ln, i], x[begin:begin + ln])
            assert np.array_equal(f["targets"][:ln, i], y[begin:begin + ln])
            want = np.full(ln, 2, np.int8)
            want[-1] = 3
            want[0] = 1
            assert np.array_equal(f["pat_types"][:ln, i], want)
        else:
            ln = 0
        assert not f["inputs"][ln:, i].any() and not f["targets"][ln:, i].any()
        assert not f["pat_types"][ln:, i].any()


@pytest.mark.parametrize("version", [1, 2])
@pytest.mark.parametrize("P", [1, 3, 4])
def test_fractions_hold_the_file_contents_sorted_by_length(tmp_path, version, P):
    tags, lens, x, y = make_corpus(7, [5, 3, 9, 4, 7, 2, 6, 11, 1, 8])
    path = str(tmp_path / "train.nc")
    b2lstm.write_nc(path, tags, lens, x, y, version=version)
    ds = b2lstm.DataSet(path, P)
    assert (ds.total_sequences, ds.total_timesteps) == (10, sum(lens))
    assert (ds.min_seq_length, ds.max_seq_length, ds.input_size, ds.output_size) == (1, 11, 5, 3)
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]])
    source = {(t, 0): (x, y, int(s)) for t, s in zip(tags, starts)}
    for epoch in range(2):
        got = []
        for f in ds.epoch():
            check_fraction(f, P, source)
            got += list(f["seq_lengths"])
        assert got == sorted(lens)             # distinct lengths: the order is fully determined
    m, s, present = ds.output_mean_stdev()
    assert not present and not m.any() and (s == 1).all()


def test_inference_mode_keeps_file_order_and_reads_mean_stdev(tmp_path):
    tags, lens, x, y = make_corpus(8, [4, 9, 2, 6, 6, 3])
    path = str(tmp_path / "test.nc")
    b2lstm.write_nc(path, tags, lens, x, y, output_means=[0.5, -1, 2], output_stdevs=[1, 2, 3])
    ds = b2lstm.DataSet(path, 4, training_mode=False)
    fr = list(ds.epoch())
    assert [f["tags"] for f in fr] == [tags[:4], tags[4:]]
    assert fr[1]["num_sequences"] == 2 and fr[1]["inputs"].shape[1] == 4
    m, s, present = ds.output_mean_stdev()
    assert present and m.tolist() == [0.5, -1, 2] and s.tolist() == [1, 2, 3]


def test_truncation_into_segments_follows_the_one_and_a_half_rule(tmp_path):
    tags, lens, x, y = make_corpus(9, [10, 25, 7, 16, 15])
    path = str(tmp_path / "t.nc")
    b2lstm.write_nc(path, tags, lens, x, y)
    trunc = 10
    segs = segments(lens, tags, trunc)
    # 25 -> 10 + 15 (15 is not more than 1.5 x 10), 16 -> 10 + 6, 15 stays whole
    assert [s[3] for s in segs] == [10, 10, 15, 7, 10, 6, 15]
    ds = b2lstm.DataSet(path, 2, trunc_seq_length=trunc, training_mode=False)
    assert ds.total_sequences == len(segs) and ds.total_timesteps == sum(lens) and ds.max_seq_length == 15
    source = {(t, k): (x, y, b) for t, k, b, _ in segs}
    got = []
    for f in ds.epoch():
        check_fraction(f, 2, source)
        got += list(zip(f["tags"], f["original_seq_idx"], [int(v) for v in f["seq_lengths"]]))
    assert got == [(t, k, ln) for t, k, _, ln in segs]


def test_several_files_and_a_fraction_of_each(tmp_path):
    a = make_corpus(1, [3, 8, 5, 9])
    b = make_corpus(2, [7, 2, 6, 4, 10, 12])
    pa, pb = str(tmp_path / "a.nc"), str(tmp_path / "b.nc")
    b2lstm.write_nc(pa, *a)
    b2lstm.write_nc(pb, *b)
    ds = b2lstm.DataSet([pa, pb], 3, fraction=0.5)      # int(4*0.5)=2 and int(6*0.5)=3 sequences
    assert ds.total_sequences == 5 and ds.total_timesteps == 3 + 8 + 7 + 2 + 6
    source = {}
    for tags, lens, x, y in (a, b):
        starts = np.concatenate([[0], np.cumsum(lens)[:-1]])
        for t, s in zip(tags, starts):
            source[(t, 0)] = (x, y, int(s))
    got = []
    for f in ds.epoch():
        check_fraction(f, 3, source)
        got += list(f["seq_lengths"])
    assert got == [2, 3, 6, 7, 8]


def test_record_dimension_and_double_variables_are_read(tmp_path):
    from scipy.io import netcdf_file
    tags, lens, x, y = make_corpus(3, [4, 6, 5])
    path = str(tmp_path / "rec.nc")
    with netcdf_file(path, "w", version=1) as f:
        f.createDimension("numTimesteps", None)          # unlimited: inputs and targets are interleaved per record
        f.createDimension("numSeqs", 3)
        f.createDimension("inputPattSize", 5)
        f.createDimension("targetPattSize", 3)
        f.createDimension("maxSeqTagLength", 16)
        tv = f.createVariable("seqTags", "S1", ("numSeqs", "maxSeqTagLength"))
        lv = f.createVariable("seqLengths", "i", ("numSeqs",))
        iv = f.createVariable("inputs", "d", ("numTimesteps", "inputPattSize"))
        ov = f.createVariable("targetPatterns", "f", ("numTimesteps", "targetPattSize"))
        arr = np.zeros((3, 16), "S1")
        for i, t in enumerate(tags):
            arr[i, :len(t)] = list(t)
        tv[:] = arr
        lv[:] = np.asarray(lens, np.int32)
        iv[:] = x.astype(np.float64)
        ov[:] = y
    ds = b2lstm.DataSet(path, 2, training_mode=False)
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]])
    source = {(t, 0): (x, y, int(s)) for t, s in zip(tags, starts)}
    for f in ds.epoch():
        check_fraction(f, 2, source)


# ---- shuffling: std::random_shuffle driven by boost::uniform_int over one mt19937 ------------------
class MT19937:
    """the published Mersenne Twister, seeded as std::mt19937(seed) / boost::mt19937::seed(seed)"""

    def __init__(self, seed):
        self.mt = [0] * 624
        self.mt[0] = seed & 0xFFFFFFFF
        for i in range(1, 624):
            self.mt[i] = (1812433253 * (self.mt[i - 1] ^ (self.mt[i - 1] >> 30)) + i) & 0xFFFFFFFF
        self.idx = 624

    def __call__(self):
        if self.idx >= 624:
            mt = self.mt
            for i in range(624):
                yv = (mt[i] & 0x80000000) | (mt[(i + 1) % 624] & 0x7FFFFFFF)
                mt[i] = mt[(i + 397) % 624] ^ (yv >> 1) ^ (0x9908B0DF if yv & 1 else 0)
            self.idx = 0
        yv = self.mt[self.idx]
        self.idx += 1
        yv ^= yv >> 11
        yv ^= (yv << 7) & 0x9D2C5680
        yv ^= (yv << 15) & 0xEFC60000
        yv ^= yv >> 18
        return yv & 0xFFFFFFFF


def test_generator_restatement_matches_the_standard_known_answer():
    g = MT19937(5489)
    for _ in range(9999):
        g()
    assert g() == 4123659995        # 10000th output of a default-seeded mt19937 (C++ standard, [rand.predef])


def shuffle_ref(items, gen):
    def below(n):
        rng = n - 1
        bucket = 0xFFFFFFFF // (rng + 1)
        if 0xFFFFFFFF % (rng + 1) == rng:
            bucket += 1
        while True:
            r = gen() // bucket
            if r <= rng:
                return r
    for i in range(1, len(items)):
        j = below(i + 1)
        if i != j:
            items[i], items[j] = items[j], items[i]


def test_sequence_and_fraction_shuffling_draw_from_one_generator(tmp_path):
    lens = [5, 3, 9, 4, 7, 2, 6, 11, 1, 8, 10]
    tags, lens, x, y = make_corpus(11, lens)
    path = str(tmp_path / "s.nc")
    b2lstm.write_nc(path, tags, lens, x, y)
    P, seed = 3, 1234
    b2lstm.data_reseed(seed)
    ds = b2lstm.DataSet(path, P, sequence_shuffling=True, fraction_shuffling=True, random_seed=seed)
    gen = MT19937(seed)
    order = sorted(range(len(lens)), key=lambda i: lens[i])
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]])
    source = {(t, 0): (x, y, int(s)) for t, s in zip(tags, starts)}
    for epoch in range(3):                     # reshuffled before every epoch, from the running generator
        shuffle_ref(order, gen)
        fr = [order[i:i + P] for i in range(0, len(order), P)]
        shuffle_ref(fr, gen)
        order = [i for f in fr for i in f]
        got = []
        for f in ds.epoch():
            check_fraction(f, P, source)
            got += f["tags"]
        assert got == [tags[i] for i in order]


def test_errors_carry_the_reference_messages(tmp_path):
    with pytest.raises(B2Error, match="Could not open"):
        b2lstm.DataSet(str(tmp_path / "missing.nc"), 2)
    tags, lens, x, y = make_corpus(4, [3, 4])
    path = str(tmp_path / "ok.nc")
    b2lstm.write_nc(path, tags, lens, x, y)
    with pytest.raises(B2Error, match="Invalid fraction"):
        b2lstm.DataSet(path, 2, fraction=0.0)
    other = str(tmp_path / "other.nc")
    b2lstm.write_nc(other, *make_corpus(5, [3, 4], n_in=6))
    with pytest.raises(B2Error, match="Number of inputs mismatch"):
        b2lstm.DataSet([path, other], 2)
    junk = str(tmp_path / "junk.nc")
    with open(junk, "wb") as f:
        f.write(b"\x89HDF\r\n\x1a\n" + bytes(64))
    with pytest.raises(B2Error, match="netCDF-4"):
        b2lstm.DataSet(junk, 2)
    cut = str(tmp_path / "cut.nc")
    with open(path, "rb") as f:
        data = f.read()
    with open(cut, "wb") as f:
        f.write(data[:-16])
    with pytest.raises(B2Error, match="beyond the end"):
        b2lstm.DataSet(cut, 2)


def test_workload_written_as_nc_reads_back_as_the_same_fraction(tmp_path):
    from b2lstm import workloads
    wl = workloads.build(0)
    path = str(tmp_path / "cfg0.nc")
    workloads.write_nc(wl, path)
    P = wl["P"]
    ds = b2lstm.DataSet(path, P, training_mode=False)
    f = ds.next_fraction()
    T = int(wl["lens"].max())
    assert f["T"] == T and list(f["seq_lengths"]) == list(wl["lens"])
    assert np.array_equal(f["inputs"].reshape(-1), np.asarray(wl["x"]).reshape(-1)[:f["inputs"].size])
    assert np.array_equal(f["targets"].reshape(-1), np.asarray(wl["tg"]).reshape(-1)[:f["targets"].size])
    assert ds.next_fraction() is None


@pytest.mark.parametrize("world", [2, 3, 8])
def test_shards_deal_every_fraction_in_snake_order(tmp_path, world):
    """Data-parallel sharding: with S shards a fraction spans P*S sequences; position k goes to shard
    k % S in even rounds and S-1 - k % S in odd rounds (the rule of b2lstm.dp.shard_indices); every shard
    pads to its own longest sequence; shards without a sequence get an empty fraction."""
    from b2lstm.dp import shard_indices
    lens = [5, 3, 9, 4, 7, 2, 6, 11, 1, 8, 10, 13, 12]
    tags, lens, x, y = make_corpus(21, lens)
    path = str(tmp_path / "d.nc")
    b2lstm.write_nc(path, tags, lens, x, y)
    P = 2
    starts = np.concatenate([[0], np.cumsum(lens)[:-1]])
    source = {(t, 0): (x, y, int(s)) for t, s in zip(tags, starts)}
    order = [tags[i] for i in sorted(range(len(lens)), key=lambda i: lens[i])]
    sets = [b2lstm.DataSet(path, P, shard_rank=r, shard_count=world) for r in range(world)]
    n_frac = -(-len(lens) // (P * world))
    total = 0
    for k in range(n_frac):
        glob = order[k * P * world:(k + 1) * P * world]
        for r in range(world):
            f = sets[r].next_fraction()            # the views stay valid for two more fractions only: check now
            want = [glob[i] for i in shard_indices(len(glob), r, world)]
            assert f["tags"] == want
            if want:
                check_fraction(f, P, source)
            else:
                assert f["num_sequences"] == 0 and f["T"] == 0
            total += f["total_frames"]
    assert all(ds.next_fraction() is None for ds in sets)
    assert total == sum(lens)
