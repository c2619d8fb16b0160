"""The pipeline executor's point-to-point traffic replayed under NCCL's ordering rules (one stream per communicator
and rank, rendezvous of matching operations, matching by order): every schedule must run to completion with the
executor's assignment of channels to communicators, and the simulator must find the known ways to stand still."""
import pytest

from nanopysche_b200.parallel.pipeline_sim import check_schedule, simulate, trace_rank

SCHEDULES = ["1F1B", "GPipe", "DualPipe", "ZBVZeroBubble", "InterleavedZeroBubble", "Interleaved1F1B", "LoopedBFS"]


@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("p", [2, 3, 4, 8])
def test_every_schedule_completes_under_nccl_ordering(schedule, p):
    for m in sorted({p, 2 * p, 8}):
        if schedule == "DualPipe" and m % 2:
            continue
        for prefetch in (1, 2):
            ok, stuck = check_schedule(schedule, p, m, prefetch=prefetch)
            assert ok, (schedule, p, m, prefetch, stuck[:4])


def test_simulator_finds_a_receive_posted_in_front_of_a_send_on_one_communicator():
    # everything on one communicator: rank 0's prefetched gradient receive sits in front of its activation send
    ok, stuck = check_schedule("1F1B", 2, 4, chan_key=lambda kind, s, r: ("all",))
    assert not ok and any("recv ('grad', 0, 0)" in x for x in stuck)
    # one communicator per kind is enough for a one-directional schedule on two ranks
    ok, _ = check_schedule("GPipe", 2, 2, prefetch=1, chan_key=lambda kind, s, r: (kind,))
    assert ok


def test_communicators_shared_by_sender_parity_block_bidirectional_schedules():
    parity = lambda kind, s, r: (kind, s & 1)   # noqa: E731
    assert check_schedule("DualPipe", 2, 8, chan_key=parity)[0]            # two ranks: each stream has one direction
    ok, stuck = check_schedule("DualPipe", 4, 8, chan_key=parity)
    assert not ok and stuck
    assert not check_schedule("ZBVZeroBubble", 4, 8, chan_key=parity)[0]
    assert not check_schedule("Interleaved1F1B", 3, 6, chan_key=parity)[0]


def test_order_mismatch_is_reported():
    progs = [trace_rank("1F1B", 2, 4, r) for r in range(2)]
    # swap the labels of rank 0's first two activation sends: the receiver now meets the wrong message first
    sends = [op for op in progs[0] if op.kind == "send" and op.label[0] == "act"]
    sends[0].label, sends[1].label = sends[1].label, sends[0].label
    ok, msg = simulate(progs)
    assert not ok and "met" in msg[0]


def test_timed_replay_reproduces_closed_form_bubbles_and_ranks_schedules():
    from nanopysche_b200.parallel.pipeline_sim import timeline

    for p, m in ((4, 8), (4, 16), (8, 16)):
        closed = (p - 1) / (m + p - 1)
        for sch in ("GPipe", "1F1B"):
            t = timeline(sch, p, m, t_fwd=1.0, t_bwd=2.0)
            assert t["makespan"] == pytest.approx((m + p - 1) * 3.0)
            assert t["bubble"] == pytest.approx(closed, abs=1e-9)
        # two half-size stages per rank: compare at equal work per rank (half the cost per action)
        zb = timeline("ZBVZeroBubble", p, m, t_fwd=0.5, t_bwd=1.0)
        dual = timeline("DualPipe", p, m, t_fwd=1.0, t_bwd=2.0)
        assert zb["bubble"] < 0.5 * closed and dual["bubble"] < 0.5 * closed
    # a transfer cost lengthens the step of a schedule whose transfers are on the critical path
    assert timeline("GPipe", 4, 8, t_p2p=0.25)["makespan"] > timeline("GPipe", 4, 8)["makespan"]


def test_recommend_ranks_schedules_by_replayed_step_time():
    from nanopysche_b200.parallel.pipeline_sim import recommend

    ranked = recommend(4, 8, t_fwd=1.0, t_bwd=2.0, t_p2p=0.05)
    names = [n for n, _, _ in ranked]
    assert names[-1] == "1F1B" and names.index("DualPipe") < names.index("Interleaved1F1B") < names.index("1F1B")
    assert all(a[1] <= b[1] for a, b in zip(ranked, ranked[1:]))
    assert "DualPipe" not in [n for n, _, _ in recommend(3, 5)]
