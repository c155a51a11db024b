"""One rank of the host-side failure tests: a tensor-parallel server group on the CPU (gloo, emulated kernels, library
collectives) whose follower misbehaves on purpose - on the host, between steps, never inside a kernel:

  leave     the follower announces that it leaves and exits before answering step 3
  die       the follower exits without a word before answering step 3 (its heartbeat stops)
  stall     the follower sleeps past the readiness deadline before answering step 3
  instep    the follower answers ready for step 3 and then stalls before its collectives (rank 0 is already inside
            the step: the process group's short timeout ends its collective with an error)

Rank 0 runs the scheduler with two live requests.  It has to notice within the deadline, go dead with a cause that
names the rank, fail the live requests, refuse new ones, and leave cleanly; it prints one JSON line.
Launched as plain child processes (not under a launcher that would kill the group when one rank exits)."""
import json
import os
import sys
import time
from datetime import timedelta

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from poot_b200 import LLM, SamplingParams                                   # noqa: E402
from poot_b200.parallel.tp import NcclComm                                  # noqa: E402
from poot_b200.serve.follower import LeaderStepEngine, follow, init_control_group   # noqa: E402
from poot_b200.serve.metrics import Metrics                                 # noqa: E402
from poot_b200.serve.scheduler import EngineDead, Job, ServeEngine          # noqa: E402
from poot_b200.utils.kernel_emulation import emulated_kernels               # noqa: E402

FAIL_AT = 3


def main() -> int:
    mode = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    dist.init_process_group("gloo", timeout=timedelta(seconds=4 if mode == "instep" else 60))
    cp = init_control_group(ready_deadline=1.5, step_deadline=10.0, heartbeat=0.1, heartbeat_timeout=1.0)
    with emulated_kernels():
        llm = LLM.random("tiny-llama", device="cpu", rows=2, max_seq=64, prefill_chunk=16, num_blocks=16, std=0.05,
                         vocab=2048, n_layers=2, tp_rank=rank, tp_world=world,
                         comm=NcclComm(rank, world, torch.device("cpu")))
        if rank != 0:
            def misbehave(n):
                if n != FAIL_AT or rank != 1:
                    return
                if mode == "leave":
                    cp.leave("test: this rank was told to leave between two steps")
                    cp.close()
                    os._exit(0)
                if mode == "die":
                    os._exit(7)
                if mode == "stall":
                    time.sleep(4.0)

            inner = llm.driver.engine
            if mode == "instep" and rank == 1:
                real = inner.run_step

                def slow(inp, _n=[0]):
                    _n[0] += 1
                    if _n[0] == FAIL_AT + 1:
                        time.sleep(8.0)
                    return real(inp)
                inner.run_step = slow
            cause = follow(inner, before_step=misbehave)
            print(json.dumps({"rank": rank, "cause": cause}), flush=True)
            cp.close()
            os._exit(0)

        llm.driver.engine = LeaderStepEngine(llm.driver.engine)
        engine = ServeEngine(llm.driver, llm.tokenizer, Metrics(), 16, 30.0, step_deadline=20.0)
        engine.start()
        sp = SamplingParams(max_tokens=40, temperature=0.0, ignore_eos=True)
        jobs = [engine.submit(Job(prompt_tokens=[5 + i, 9, 11, 200 + i], params=sp)) for i in range(2)]
        t0 = time.monotonic()
        finals = [j.wait(timeout=40) for j in jobs]
        took = time.monotonic() - t0
        refused = False
        try:
            engine.submit(Job(prompt_tokens=[1, 2, 3], params=sp))
        except EngineDead:
            refused = True
        health = engine.health()
        print(json.dumps({"rank": 0, "mode": mode, "health": health, "took_s": took, "refused_new": refused,
                          "finals": [f.get("type") if f else None for f in finals],
                          "errors": [j.error for j in jobs], "steps": cp.n,
                          "tokens_before": [len(j.tokens) for j in jobs]}), flush=True)
        llm.driver.engine.stop_followers(health.get("cause", "shutdown"))
        cp.close()
    os._exit(0)


if __name__ == "__main__":
    sys.exit(main())
