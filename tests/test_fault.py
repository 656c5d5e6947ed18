"""Failure handling on the host: watchdog, non-finite guard, heartbeats, a rank that leaves between steps, a collective
that times out, atomic checkpoints and resume from the newest complete one.  No GPU is involved and nothing is made to
fault: failures are a callback that fires, a process that exits, a file that is missing."""

import subprocess
import sys
import time
from pathlib import Path

import pytest
import torch
import torch.distributed as dist

from sample_efficient_gpt_b200.utils.fault import NonFiniteGuard, RankHeartbeat, StepWatchdog

ROOT = Path(__file__).resolve().parent.parent


def test_watchdog_fires_only_without_beats():
    fired = []
    wd = StepWatchdog(0.3, on_timeout=lambda: fired.append(time.monotonic()), poll_s=0.05)
    for _ in range(8):
        time.sleep(0.1)
        wd.beat()
    assert not fired and not wd.fired
    time.sleep(0.6)
    assert len(fired) == 1 and wd.fired
    wd.stop()
    idle = StepWatchdog(0.0, on_timeout=lambda: fired.append(0))  # 0 disables
    time.sleep(0.1)
    assert len(fired) == 1 and not idle.fired


def test_non_finite_guard():
    g = NonFiniteGuard(3)
    assert g.check(1.0) and not g.check(float("nan")) and not g.check(float("inf")) and g.check(2.0)
    assert g.streak == 0 and g.total == 2
    g.check(float("nan"))
    g.check(float("-inf"))
    with pytest.raises(FloatingPointError):
        g.check(float("nan"))
    off = NonFiniteGuard(0)
    assert not any(off.check(float("nan")) for _ in range(10)) and off.total == 10


def test_heartbeat_detects_a_silent_rank():
    store = dist.HashStore()
    a = RankHeartbeat(store, 0, 2, interval_s=0.05, timeout_s=0.4)
    b = RankHeartbeat(store, 1, 2, interval_s=0.05, timeout_s=0.4)
    time.sleep(0.3)
    assert a.dead_ranks() == [] and b.dead_ranks() == []
    b.stop()
    deadline = time.monotonic() + 5
    dead = []
    while not dead and time.monotonic() < deadline:
        time.sleep(0.1)
        dead = a.dead_ranks()
    assert dead == [1]
    a.stop()


def _two_ranks(scenario: str, port: int):
    procs = [subprocess.Popen([sys.executable, str(ROOT / "tests" / "fault_worker.py"), scenario, str(r), str(port)],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, cwd=ROOT) for r in range(2)]
    outs = []
    for p in procs:
        try:
            outs.append(p.communicate(timeout=90)[0])
        except subprocess.TimeoutExpired:
            p.kill()
            outs.append(p.communicate()[0] + "\nKILLED")
    return procs, outs


def test_rank_leaves_between_steps_and_peer_stops_cleanly():
    procs, outs = _two_ranks("leave", 29641)
    assert "RANK1-LEFT" in outs[1], outs[1][-2000:]
    assert "DETECTED dead=[1]" in outs[0], outs[0][-2000:]
    assert procs[0].returncode == 0 and procs[1].returncode == 0


def test_collective_after_peer_left_ends_with_an_error():
    procs, outs = _two_ranks("timeout", 29643)
    assert "COLLECTIVE-ERROR" in outs[0] and "COLLECTIVE-RETURNED" not in outs[0], outs[0][-2000:]


def test_checkpoint_is_atomic_and_resume_picks_newest_complete(tmp_path):
    from sample_efficient_gpt_b200.training import checkpoint as ck

    model = torch.nn.Linear(4, 4)
    opt = torch.optim.SGD(model.parameters(), lr=0.1)
    names = []
    for it in (10, 20):
        path = tmp_path / f"{it}.pt"
        ck.save_checkpoint(path, None, model, [opt], it, "run")
        names.append(path)
    (tmp_path / "30.pt.tmp4242").write_bytes(b"partial write of a crashed save")
    assert not any(p.name.endswith(".tmp") for p in names)
    newest = ck.find_latest(tmp_path)
    assert newest is not None and Path(newest).name == "20.pt"
    assert torch.load(newest, weights_only=False)["iteration"] == 20
    (tmp_path / "latest").unlink()  # a lost pointer file falls back to the directory scan
    assert Path(ck.find_latest(tmp_path)).name == "20.pt"
