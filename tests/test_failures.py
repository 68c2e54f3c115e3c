"""Failure detection without a GPU: heartbeats, stall watchdog, fleet-health state machine, rollout retries, and a
two-rank gloo job in which one rank leaves between steps and the other learns of it on the host."""

import os
import socket
import time

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rl_b200.distributed.health import DictStore, HealthPolicy, HealthTracker, Heartbeat, PeerLostError, ShardState, StallWatchdog
from rl_b200.experience.failures import DataFailure, FailureKind, InfraFailure, classify
from rl_b200.experience.rollout_manager import RetryPolicy, RolloutManager, TooManyFailures


class _Clock:
    def __init__(self):
        self.t = 0.0

    def __call__(self):
        return self.t


def test_heartbeat_detects_silent_peer_with_fake_clock():
    store, clk = DictStore(), _Clock()
    a = Heartbeat(store, 0, 3, timeout_s=5, clock=clk)
    b = Heartbeat(store, 1, 3, timeout_s=5, clock=clk)
    c = Heartbeat(store, 2, 3, timeout_s=5, clock=clk)
    for hb in (a, b, c):
        hb.beat()
    assert a.dead_peers() == []
    for step in range(1, 8):
        clk.t = float(step)
        a.beat(); b.beat()        # rank 2's message is "dropped" from now on
        dead = a.dead_peers()
    assert dead == [2]
    with pytest.raises(PeerLostError):
        a.check()
    c.beat()
    assert a.dead_peers() == []   # it came back


def test_stall_watchdog():
    clk, seen = _Clock(), []
    w = StallWatchdog(10.0, on_stall=seen.append, clock=clk)
    clk.t = 9.0
    assert not w.poll()
    clk.t = 11.0
    assert w.poll() and len(seen) == 1 and seen[0] == pytest.approx(11.0)
    w.poll()
    assert len(seen) == 1  # fires once per stall
    w.progress()
    assert not w.poll()


def test_fleet_health_state_machine():
    h = HealthTracker(4, HealthPolicy(suspect_after_failures=1, dead_after_failures=3, recover_after_successes=2, max_restarts=1))
    assert h.select() == [0, 1, 2, 3]
    assert h.report_failure(1, "timeout") == ShardState.SUSPECT
    assert h.select() == [0, 2, 3, 1] and h.select(include_suspect=False) == [0, 2, 3]
    h.report_success(1)
    assert h.state(1) == ShardState.SUSPECT
    h.report_success(1)
    assert h.state(1) == ShardState.HEALTHY
    for _ in range(3):
        h.report_failure(2, "oom")
    assert h.state(2) == ShardState.DEAD and 2 not in h.select()
    assert h.begin_restart(2) == ShardState.RESTARTING
    assert h.finish_restart(2, ok=True) == ShardState.HEALTHY
    h.report_failure(2, "killed", fatal=True)
    assert h.begin_restart(2) == ShardState.RETIRED  # restart budget of 1 is spent
    # weights: shard 3 misses two publications
    h.set_weight_version(1, updated_shards=[0, 1])
    assert h.state(3) == ShardState.HEALTHY           # one version behind is allowed
    h.set_weight_version(2, updated_shards=[0, 1])
    assert h.state(3) == ShardState.STALE and 3 not in h.select()
    h.set_weight_version(3)
    assert h.state(3) == ShardState.HEALTHY
    assert h.serviceable() and h.summary() == {"healthy": 3, "retired": 1}


def test_rollout_manager_retries_infra_and_masks_data_failures():
    assert classify(TimeoutError()) == FailureKind.INFRA and classify(ValueError()) == FailureKind.DATA
    calls = {}

    def job(x):
        calls[x] = calls.get(x, 0) + 1
        if x == "flaky" and calls[x] < 3:
            raise ConnectionError("shard went away")
        if x == "bad":
            raise DataFailure("malformed tool call")
        return x.upper()

    m = RolloutManager(RetryPolicy(max_attempts=3, max_failed_fraction=0.5))
    out = m.run(job, ["a", "flaky", "bad", "b"])
    assert [r.ok for r in out] == [True, True, False, True] and out[1].value == "FLAKY" and out[1].attempts == 3
    assert out[2].attempts == 1 and out[2].kind == FailureKind.DATA and calls["bad"] == 1
    assert m.stats["retries"] == 2 and m.stats["infra_failures"] == 2 and m.stats["data_failures"] == 1

    def always(x):
        raise InfraFailure("down")

    with pytest.raises(TooManyFailures):
        RolloutManager(RetryPolicy(max_attempts=2, max_failed_fraction=0.25)).run(always, [1, 2, 3, 4])


def test_rollout_manager_moves_to_another_shard_and_honours_deadline():
    h = HealthTracker(2, HealthPolicy(dead_after_failures=2))
    seen = []

    def job(x, shard):
        seen.append(shard)
        if shard == 0:
            raise TimeoutError("no answer")
        return x

    m = RolloutManager(RetryPolicy(max_attempts=3), health=h)
    out = m.run(job, [10, 11])
    assert all(r.ok for r in out) and seen[:2] == [0, 1] and h.state(0) in (ShardState.SUSPECT, ShardState.DEAD)
    clk = _Clock()

    def slow(x):
        clk.t += 10
        raise ConnectionError("x")

    r = RolloutManager(RetryPolicy(max_attempts=10, deadline_s=15, max_failed_fraction=1.0), clock=clk).run(slow, [0])[0]
    assert not r.ok and r.attempts == 2 and r.failures[-1].error == "deadline exceeded"


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _leaver(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=__import__("datetime").timedelta(seconds=30))
    dist.init_process_group("gloo", store=dist.PrefixStore("pg", store), rank=rank, world_size=world)
    hb = Heartbeat(dist.PrefixStore("hb", store), rank, world, interval_s=0.1, timeout_s=1.0).start()
    steps = 0
    try:
        for step in range(50):
            hb.check()                      # between steps, before the next collective
            t = torch.ones(1)
            dist.all_reduce(t)
            steps += 1
            if rank == 1 and step == 2:     # leaves between steps: nothing of its own in flight
                hb.leave()
                break
            time.sleep(0.2)
    except PeerLostError as e:
        with open(out, "w") as f:
            f.write(f"{steps} {e}")
    finally:
        hb.stop()
    if rank == 1:
        time.sleep(3.0)  # keep the process (and its sockets) alive while rank 0 notices the silence


def test_rank_that_leaves_is_detected_on_the_host(tmp_path):
    out = str(tmp_path / "r0.txt")
    ctx = mp.get_context("spawn")
    port = _free_port()
    ps = [ctx.Process(target=_leaver, args=(r, 2, port, out)) for r in range(2)]
    for p in ps:
        p.start()
    for p in ps:
        p.join(60)
    msg = open(out).read()
    assert msg.startswith("3 ") and "ranks [1]" in msg


def test_ft_launcher_restarts_on_crash_and_on_hang(tmp_path):
    """Job-level supervision: a crash (non-zero exit) and a hang (stale heartbeat) both lead to a restart; the job, which
    keeps its progress in a file as a checkpoint would, completes on a later attempt."""
    import sys
    import textwrap

    from rl_b200.distributed.ft_launcher import run_with_restarts

    script = tmp_path / "job.py"
    state = tmp_path / "state.txt"
    script.write_text(textwrap.dedent(f"""
        import os, sys, time
        sys.path.insert(0, {str(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))!r})
        from rl_b200.distributed.ft_launcher import beat
        state = {str(state)!r}
        step = int(open(state).read()) if os.path.exists(state) else 0
        attempt = int(os.environ["RLB_FT_ATTEMPT"])
        while step < 6:
            step += 1
            open(state, "w").write(str(step))
            beat(step)
            if attempt == 0 and step == 2:
                sys.exit(3)                      # crash
            if attempt == 1 and step == 4:
                time.sleep(600)                  # hang: no more heartbeats
            time.sleep(0.05)
    """))
    logs = []
    res = run_with_restarts([sys.executable, str(script)], max_restarts=3, initial_timeout_s=30, step_timeout_s=1.5, poll_s=0.1, grace_s=2,
                            log=logs.append)
    assert res.returncode == 0 and res.restarts == 2
    assert "exit code 3" in res.reasons[0] and "no heartbeat" in res.reasons[1]
    assert int(state.read_text()) == 6
    # restart budget: a job that always fails gives up with its exit code
    bad = tmp_path / "bad.py"
    bad.write_text("import sys; sys.exit(5)")
    res = run_with_restarts([sys.executable, str(bad)], max_restarts=1, poll_s=0.05, log=logs.append)
    assert res.returncode == 5 and res.restarts == 1 and len(res.reasons) == 2
