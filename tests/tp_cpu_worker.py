"""Worker of the host tensor-parallel test: ranks over gloo, kernels emulated, the library-collective comm (the
baseline path of the device engine: local GEMM, all-reduce, residual add; vocabulary-parallel head with the greedy
pick merged from per-shard partial tables or, for sampling, from gathered logits)."""
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from poot_b200.models.config import DecoderConfig                           # noqa: E402
from poot_b200.parallel.tp import NcclComm                                  # noqa: E402
from poot_b200.runtime.engine import DecoderEngine                          # noqa: E402
from poot_b200.runtime.session import FixedBatchSession                     # noqa: E402
from poot_b200.runtime.weights import random_weights                        # noqa: E402
from poot_b200.utils.kernel_emulation import emulated_kernels               # noqa: E402


def run(cfg, rank, world, comm):
    w = random_weights(cfg, "cpu", seed=0, std=0.05, tp_rank=rank, tp_world=world,
                       ep_rank=rank if (cfg.is_moe and world > 1) else 0, ep_world=world if cfg.is_moe else 1)
    eng = DecoderEngine(w, num_blocks=9, max_seqs=2, max_tokens=48, max_blocks_per_seq=4, comm=comm, device="cpu", use_graphs=False)
    s = FixedBatchSession(eng, 2, 64)
    g = torch.Generator().manual_seed(5)
    prompts = torch.randint(0, cfg.vocab, (2, 19), generator=g, dtype=torch.int32)
    out = [s.prefill_fast(prompts).clone()]
    for _ in range(3):
        out.append(s.decode(out[-1][:, 0].tolist()).clone())
    out.append(s.decode(out[-1][:, 0].tolist(), sampler=1).clone())       # a sampling step gathers the whole logits
    return torch.stack(out), eng


def main() -> int:
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    results = {}
    with emulated_kernels():
        # two experts per rank: each rank groups only the rows routed to its own experts (row-grouped regime at prefill,
        # one group per (token, slot) never applies under expert parallelism)
        for name, kw in (("dense", {}), ("moe", dict(n_experts=2 * world, top_k=2, moe_ffn=128))):
            cfg = DecoderConfig(n_layers=2, hidden=128, n_heads=max(4, world), n_kv_heads=2 if world <= 2 else world, head_dim=64,
                                ffn=256, vocab=4096, max_position=256, **kw)
            got, eng = run(cfg, rank, world, NcclComm(rank, world, torch.device("cpu")))
            eng.samp_params[:2] = torch.tensor([[1.0, -1e30, 1.0, 1.0]] * 2)
            want, ref = run(cfg, 0, 1, None)
            # greedy steps must agree token for token; logits of the last greedy step within bf16 noise
            same = bool(torch.equal(got[:4], want[:4]))
            results[name] = {"tokens_equal": same, "got": got[:4, :, 0].tolist(), "want": want[:4, :, 0].tolist()}
    ok = all(r["tokens_equal"] for r in results.values())
    flags = [None] * world
    dist.all_gather_object(flags, ok)
    if rank == 0:
        print(json.dumps({"ok": all(flags), **results}), flush=True)
    dist.barrier()
    return 0


if __name__ == "__main__":
    sys.exit(main())
