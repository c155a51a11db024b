"""Worker of the multi-process pipeline test: one process per stage over gloo on the CPU, kernels emulated on the
host.  Rank 0 owns the driver and announces every step to the other stages (the follower loop the tensor-parallel
server uses); the residual stream travels stage to stage and the sampled tokens come back to rank 0."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from poot_b200 import LLM, SamplingParams                                   # noqa: E402
from poot_b200.serve.follower import LeaderStepEngine, follow, init_control_group   # noqa: E402
from poot_b200.utils.kernel_emulation import emulated_kernels               # noqa: E402


def main() -> int:
    import contextlib
    on_gpu = os.environ.get("POOT_PP_CUDA") == "1"          # the device twin: NCCL transfers, the real kernels
    if on_gpu:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    else:
        dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    init_control_group()
    kw = dict(device="cuda" if on_gpu else "cpu", rows=2, max_seq=64, prefill_chunk=16, num_blocks=16, std=0.05, vocab=2048,
              n_layers=3)
    with (contextlib.nullcontext() if on_gpu else emulated_kernels()):
        llm = LLM.random("tiny-llama", pp_rank=rank, pp_world=world, **kw)
        st = llm.engine.stage
        assert st.index == rank and st.count == world and len(llm.engine.w.layers) == st.l1 - st.l0
        if rank != 0:
            follow(llm.driver.engine)
            dist.barrier()
            return 0
        llm.driver.engine = LeaderStepEngine(llm.driver.engine)
        g = torch.Generator().manual_seed(3)
        prompts = [torch.randint(3, 2048, (n,), generator=g).tolist() for n in (37, 9)]
        sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
        got = [llm.generate_tokens(p, sp) for p in prompts]
        sampled = llm.generate_tokens(prompts[1], SamplingParams(max_tokens=5, temperature=0.8, top_k=20, seed=7, ignore_eos=True))
        llm.driver.engine.stop_followers()
        whole = LLM.random("tiny-llama", **kw)
        want = [whole.generate_tokens(p, sp) for p in prompts]
        want_sampled = whole.generate_tokens(prompts[1], SamplingParams(max_tokens=5, temperature=0.8, top_k=20, seed=7, ignore_eos=True))
        print(json.dumps({"ok": got == want and sampled == want_sampled, "got": got, "want": want,
                          "sent_bytes": llm.engine.link.sent_bytes}), flush=True)
        dist.barrier()
    return 0


if __name__ == "__main__":
    sys.exit(main())
