"""b2_matrix_multiply_noalloc, the entry point for hosts that cannot let the library allocate device
memory (everything on the card already belongs to the host program's own pool, or a cudaMalloc
would stall its other streams): same product as b2_matrix_multiply's FFMA path, but the split-K
partial sums sit in a fixed array inside the library instead of an allocation.

Checked through the C ABI against the existing entry point, twice in a row on different shapes, so
that what the first call leaves in the shared array cannot leak into the second.  Collected last on
purpose: a run that stops at the first failure has then already run every other test."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _product(fn, m, n, k, ta, tb, seed, **kw):
    import torch
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(seed)
    A = rng.standard_normal((k, m) if not ta else (m, k)).astype(np.float32)   # column-major storage
    B = rng.standard_normal((n, k) if not tb else (k, n)).astype(np.float32)
    tA, tB = torch.from_numpy(A).to(dev), torch.from_numpy(B).to(dev)
    tC = torch.full((n, m), float("nan"), device=dev)
    fn(tC, m, tA, m if not ta else k, ta, tB, k if not tb else n, tb, m, n, k, accumulate=False, **kw)
    torch.cuda.synchronize()
    opA = A.T.astype(np.float64) if not ta else A.astype(np.float64)
    opB = B.T.astype(np.float64) if not tb else B.astype(np.float64)
    return tC.cpu().numpy().T, opA @ opB


def test_noalloc_matches_existing_entry_point_on_two_calls_in_a_row():
    import b2lstm
    # first a long contraction that needs split-K scratch, then a different shape that reuses the
    # array with other contents, then the first again
    for call, (m, n, k, ta, tb) in enumerate([(96, 80, 6000, 0, 1), (200, 33, 2500, 1, 0), (96, 80, 6000, 0, 1)]):
        got, exact = _product(b2lstm.matrix_multiply_noalloc, m, n, k, ta, tb, seed=40 + call)
        ref, _ = _product(b2lstm.matrix_multiply, m, n, k, ta, tb, seed=40 + call, force_ffma=True)
        tol = 2e-6 * np.sqrt(k) * 8            # the tolerance of the other GEMM tests
        assert np.isfinite(got).all()
        assert np.abs(got - ref).max() <= tol, (call, np.abs(got - ref).max())
        assert np.abs(got - exact).max() <= tol, (call, np.abs(got - exact).max())


def test_noalloc_rejects_sizes_beyond_its_fixed_scratch():
    import torch
    import b2lstm
    t = torch.zeros(8, device="cuda:0")
    with pytest.raises(b2lstm.B2Error, match="fixed scratch limit"):
        b2lstm.matrix_multiply_noalloc(t, 4096, t, 4096, 0, t, 8, 0, 4096, 4096, 8)


def test_noalloc_rejects_negative_sizes_and_short_leading_dimensions():
    import torch
    import b2lstm
    t = torch.zeros(64, device="cuda:0")
    for args in [(t, 4, t, 4, 0, t, 4, 0, -1, 4, 4), (t, 3, t, 4, 0, t, 4, 0, 4, 4, 4), (t, 4, t, 3, 0, t, 4, 0, 4, 4, 4),
                 (t, 4, t, 4, 0, t, 3, 0, 4, 4, 4), (t, 4, t, 3, 1, t, 4, 0, 4, 4, 4)]:
        with pytest.raises(b2lstm.B2Error, match="error -5"):            # B2_ERR_BAD_ARG
            b2lstm.matrix_multiply_noalloc(*args)


def test_noalloc_leaves_the_free_device_memory_unchanged():
    """What the name promises, observed from outside: once the first call on the device has been made, further
    calls (split-K shapes included) leave cudaMemGetInfo's free byte count exactly where it was."""
    import torch
    import b2lstm
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(3)
    shapes = [(96, 80, 6000), (64, 64, 4096), (200, 33, 2500)]
    ops = []
    for m, n, k in shapes:                                   # all operands exist before the measurement starts
        ops.append((torch.from_numpy(rng.standard_normal((k, m)).astype(np.float32)).to(dev),
                    torch.from_numpy(rng.standard_normal((n, k)).astype(np.float32)).to(dev),
                    torch.empty((n, m), device=dev), m, n, k))
    A, B, Cm, m, n, k = ops[0]
    b2lstm.matrix_multiply_noalloc(Cm, m, A, m, 0, B, k, 0, m, n, k)          # first call: address look-up
    torch.cuda.synchronize()
    free0 = torch.cuda.mem_get_info()[0]
    for A, B, Cm, m, n, k in ops[1:] + ops:
        b2lstm.matrix_multiply_noalloc(Cm, m, A, m, 0, B, k, 0, m, n, k)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free0
