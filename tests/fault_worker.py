"""Two CPU ranks for the failure-handling tests (started as plain child processes by test_fault.py).

Scenario ``leave``: rank 1 takes part in two all-reduces, then leaves between steps (stops its heartbeat and exits).
Rank 0 consults the heartbeat table before its next collective, sees rank 1 dead and stops cleanly without launching it.
Scenario ``timeout``: rank 0 does not look at the heartbeats; its next all-reduce ends with an error after the short
process-group timeout instead of blocking forever.
"""

import datetime
import sys
import time
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

from sample_efficient_gpt_b200.utils.fault import RankHeartbeat  # noqa: E402


def main():
    scenario, rank, port = sys.argv[1], int(sys.argv[2]), int(sys.argv[3])
    store = dist.TCPStore("127.0.0.1", port, 2, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    dist.init_process_group("gloo", store=dist.PrefixStore("pg", store), rank=rank, world_size=2, timeout=datetime.timedelta(seconds=3))
    hb = RankHeartbeat(dist.PrefixStore("hb", store), rank, 2, interval_s=0.1, timeout_s=1.0)
    x = torch.ones(4)
    for _ in range(2):
        dist.all_reduce(x)
    assert x[0].item() == 4.0
    assert hb.dead_ranks() == []
    if rank == 1:
        hb.stop()
        store.set("left/1", "1")  # the store outlives this rank (rank 0 hosts it)
        print("RANK1-LEFT", flush=True)
        return
    store.wait(["left/1"])
    if scenario == "leave":
        deadline = time.monotonic() + 10
        dead = []
        while not dead and time.monotonic() < deadline:
            time.sleep(0.2)
            dead = hb.dead_ranks()
        print(f"DETECTED dead={dead}", flush=True)
    else:
        time.sleep(0.5)
        try:
            dist.all_reduce(x)
            print("COLLECTIVE-RETURNED", flush=True)
        except Exception as e:  # gloo reports the lost peer / the timeout as RuntimeError
            print(f"COLLECTIVE-ERROR {type(e).__name__}", flush=True)
    hb.stop()


if __name__ == "__main__":
    main()
