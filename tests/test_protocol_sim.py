"""The expert-parallel flag protocol under random interleavings (host-side model, no GPU): no reader ever sees a row
of another epoch; a withheld flag ends in a bounded wait that reports; releasing a flag before the stores is caught."""
import pytest

from nanopysche_b200.parallel.protocol_sim import Fault, StaleRead, simulate


@pytest.mark.parametrize("n_ranks", [2, 4, 8])
def test_protocol_is_race_free_under_random_interleavings(n_ranks):
    for seed in range(60):
        assert simulate(n_ranks, epochs=4, seed=seed) == [0] * n_ranks


def test_withheld_dispatch_flag_times_out_everywhere_and_terminates():
    st = simulate(4, epochs=3, seed=1, fault=Fault(skip_dispatch_flag=(2, 2)), wait_budget=200)
    assert all(s == 2 for s in st)       # every rank's wait on rank 2 (or on a rank that stopped) ran out and reported


def test_withheld_combine_flag_is_reported_by_the_waiting_source():
    st = simulate(4, epochs=2, seed=3, fault=Fault(skip_combine_flag=(1, 1)), wait_budget=200)
    assert any(s == 2 for s in st)


def test_flag_released_before_the_stores_is_detected():
    hits = 0
    for seed in range(200):
        try:
            simulate(4, epochs=3, seed=seed, fault=Fault(early_flag=(1, 2)))
        except StaleRead:
            hits += 1
    assert hits > 0, "the checker never saw the stale row that an early flag release allows"
