"""Integration tests of the host-buffer allreduce through the tester binary,
one case per case of the reference's tests/allreduce_test.py (exit status is
the assertion channel).  Differences: the ranks are started by `ibcomm_run`
instead of mpiexec, and Rabenseifner accepts world sizes that are not a power
of two (the reference exits with NOT_SUPPORTED there)."""
import pytest

INVALID_ARGUMENT, TRANSPORT_ERROR, CUDA_ERROR, NOT_SUPPORTED = 1, 2, 3, 4
RING, RABEN = "ring", "rabenseifner"
INT = 4


def check(ranks, bins, np, algo, buffsize, init="i*np+p", expect="i*np*np+np*(np-1)/2", chunksize=None, extra=()):
    env = {} if chunksize is None else {"IBCOMM_CHUNKSIZE": chunksize}
    code, out, err = ranks(np, [bins["allreduce_tester"], "--device", "cpu", *extra, algo, str(buffsize), init, expect], env)
    return code


def test_1proc(ranks, bins):
    assert check(ranks, bins, 1, RING, 1024) == 0
    assert check(ranks, bins, 1, RABEN, 1024) == 0


def test_small_buffer(ranks, bins):
    for np in (1, 2, 3, 5):
        assert check(ranks, bins, np, RING, np * 2 * INT) == 0
    assert check(ranks, bins, 2, RING, 2521 * INT) == 0
    for np in (1, 2, 3, 5, 6, 7):  # 3, 5, 6, 7: the non-power-of-two extension
        assert check(ranks, bins, np, RABEN, np * 2 * INT) == 0
    assert check(ranks, bins, 2, RABEN, 2521 * INT) == 0


def test_basic(ranks, bins):
    for np in (2, 3, 4):
        assert check(ranks, bins, np, RING, "128M") == 0
    for np in (2, 3, 4):
        assert check(ranks, bins, np, RABEN, "128M") == 0


def test_chunk_size(ranks, bins):
    for chunk in (4, 8, 16, 32, 64, 128):
        assert check(ranks, bins, 4, RING, "1k", chunksize=chunk) == 0


def test_invalid_error(ranks, bins):
    for chunk in (0, 1, 2, 3):
        assert check(ranks, bins, 4, RING, "1k", chunksize=chunk) == INVALID_ARGUMENT
    assert check(ranks, bins, 4, RING, "1k", chunksize="-128") == INVALID_ARGUMENT
    assert check(ranks, bins, 4, RING, "1k", chunksize="1k") == INVALID_ARGUMENT
    assert check(ranks, bins, 2, RING, INT, init="1", expect="np") == NOT_SUPPORTED
    assert check(ranks, bins, 2, RABEN, INT, init="1", expect="np") == NOT_SUPPORTED


def test_wrong_result_is_counted(ranks, bins):
    # exit status = number of ranks whose check failed
    assert check(ranks, bins, 3, RING, 64, init="i", expect="i*2") == 3
    assert check(ranks, bins, 2, RING, 64, init="p", expect="1+p*0") == 0


def test_float_and_double(ranks, bins):
    assert check(ranks, bins, 4, RING, "64k", init="1/np*p+i", expect="(np-1)/2+i*np", extra=("--dtype", "double")) == 0
    assert check(ranks, bins, 5, RABEN, "64k", init="p+1", expect="np*(np+1)/2", extra=("--dtype", "float")) == 0


def test_bad_usage(ranks, bins):
    code, _, _ = ranks(1, [bins["allreduce_tester"], "ring", "97MiB", "1", "1"])
    assert code == 1
    code, _, _ = ranks(1, [bins["allreduce_tester"], "ring", "64"])
    assert code == 1
    code, _, _ = ranks(1, [bins["allreduce_tester"], "--device", "cpu", "ring", "64", "q+", "1"])
    assert code == 1


@pytest.mark.slow
def test_aging(ranks, bins):
    for algo in (RING, RABEN):
        assert check(ranks, bins, 4, algo, "128M", extra=("--iters", "100")) == 0


def test_reduce_scatter_and_all_gather(ranks, bins):
    # The halves through the tester: the buffer size is the full buffer, `i` the
    # index in it; the closed-form oracle of the allreduce cases applies as is.
    for np in (1, 2, 3, 5):
        assert check(ranks, bins, np, RING, np * 1000 * INT, extra=("--op", "reduce_scatter")) == 0
        assert check(ranks, bins, np, RING, np * 1000 * INT, init="i*3+1", expect="i*3+1", extra=("--op", "all_gather")) == 0
    assert check(ranks, bins, 4, RING, "8M", extra=("--op", "reduce_scatter")) == 0   # larger than a transport ring
    assert check(ranks, bins, 4, RING, "8M", init="i", expect="i", extra=("--op", "all_gather")) == 0
    assert check(ranks, bins, 3, RING, 3 * 16 * INT, init="i", expect="i+1", extra=("--op", "all_gather")) == 3
    assert check(ranks, bins, 3, RING, 40, extra=("--op", "reduce_scatter")) == INVALID_ARGUMENT  # 10 ints, 3 ranks
    assert check(ranks, bins, 2, RABEN, 64, extra=("--op", "reduce_scatter")) == INVALID_ARGUMENT


def test_subset_of_the_ranks(ranks, bins):
    # A communicator over some of the job's ranks (what survivors of a failed rank build): p and np
    # refer to the subset, the other ranks do not take part.
    assert check(ranks, bins, 4, RING, 4000, extra=("--ranks", "0,2,3")) == 0
    assert check(ranks, bins, 4, RABEN, 4000, init="p+1", expect="3", extra=("--ranks", "3,1")) == 0
    assert check(ranks, bins, 5, RING, 4000, init="np", expect="np*np", extra=("--ranks", "4,0,1,3")) == 0
    assert check(ranks, bins, 2, RING, 4000, init="1", expect="1", extra=("--ranks", "0,5")) == INVALID_ARGUMENT
