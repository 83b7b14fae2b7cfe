"""Worker of tests/test_rank_failure.py: two gloo ranks on CPU run data-parallel "steps" (a dW-sized all-reduce each).
Rank 1 fails on the host between steps (it raises before step 1). Rank 0 must learn of it without hanging, in both ways
a trainer around this library can use:

  mode heartbeat : every rank posts a key in the rendezvous store before each step and waits (bounded) for its peers'
                   keys; a missing key means a failed peer, and no collective is launched for that step;
  mode timeout   : rank 0 launches the collective anyway; the process group's short timeout (or the closed connection)
                   ends it with an error instead of a hang.

No GPU is involved and nothing faults: the failure is an exception on the host."""
import argparse
import datetime
import os
import sys
import time

import torch
import torch.distributed as dist


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--mode", required=True, choices=["heartbeat", "timeout"])
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    store = dist.TCPStore(os.environ["MASTER_ADDR"], int(os.environ["MASTER_PORT"]), world, rank == 0,
                          timeout=datetime.timedelta(seconds=30))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    dw = torch.full((1000, 16), float(rank + 1))

    def heartbeat(step):
        store.set(f"hb/{rank}/{step}", "1")
        peers = [f"hb/{r}/{step}" for r in range(world) if r != rank]
        store.wait(peers, datetime.timedelta(seconds=3))       # raises when a peer's key never arrives

    # step 0: everybody is alive
    heartbeat(0)
    dist.all_reduce(dw)
    assert float(dw[0, 0]) == sum(range(1, world + 1))
    print(f"rank {rank}: step 0 reduced", flush=True)

    if rank == 1:
        raise RuntimeError("injected host-side failure of rank 1 before step 1")

    t0 = time.time()
    if a.mode == "heartbeat":
        try:
            heartbeat(1)
        except Exception as e:                                   # noqa: BLE001 (any store error means: peer missing)
            print(f"rank 0: peer missed its heartbeat before step 1 ({type(e).__name__}); no collective launched, "
                  f"{time.time() - t0:.1f} s", flush=True)
            os._exit(0)                                          # leave without a collective teardown with a dead peer
        print("rank 0: the failure was not detected", flush=True)
        os._exit(4)
    try:
        dist.all_reduce(dw)
    except Exception as e:                                       # noqa: BLE001
        print(f"rank 0: the collective of step 1 ended with an error ({type(e).__name__}) after "
              f"{time.time() - t0:.1f} s instead of hanging", flush=True)
        os._exit(0)
    print("rank 0: the collective returned although rank 1 is gone", flush=True)
    os._exit(5)


if __name__ == "__main__":
    main()
