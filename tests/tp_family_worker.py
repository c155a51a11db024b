"""Worker of the host tensor-parallel test over model families: ranks over gloo, kernels emulated, the
library-collective comm.  For every family named on the command line the sharded engine (Megatron shares of the
family's tensors: biases, sinks, ALiBi slopes, norms placed after the projections ...) must compute what one rank
picks, judged on the logits: the vocabulary shards of every rank, gathered, must equal one rank's logits within bf16
noise over a prefill and teacher-forced decode steps."""
import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from poot_b200.models.registry import Registry                              # noqa: E402
from poot_b200.oracle.runner import random_weights_f32                      # noqa: E402
from poot_b200.parallel.tp import NcclComm                                  # noqa: E402
from poot_b200.runtime.engine import DecoderEngine                          # noqa: E402
from poot_b200.runtime.session import FixedBatchSession                     # noqa: E402
from poot_b200.runtime.weights import from_named_tensors                    # noqa: E402
from poot_b200.utils.kernel_emulation import emulated_kernels               # noqa: E402

from test_engine_emulated import HF_BASE, HF_FAMILIES                       # noqa: E402


# routed experts make a model discontinuous: where two router scores nearly tie, the other summation order of a sharded
# projection can pick the other expert; the token seed of such a family avoids a near-tie on the compared steps
TOKEN_SEED = {"gpt_oss": 7}


def named_weights(model):
    cfg = model.cfg
    w = random_weights_f32(model, seed=2, std=0.08)
    for k in w:
        if k.endswith(("norm", "norm_w")):
            w[k] = (1.0 + 0.1 * np.random.default_rng(len(k)).standard_normal(w[k].shape)).astype(np.float32)
    named = {k: torch.from_numpy(v).to(torch.bfloat16).float() for k, v in w.items()}
    for l in [l for l in range(cfg.n_layers) if cfg.has_ffn(l) and cfg.moe_layer(l)]:
        p = f"layers.{l}."
        for e in range(cfg.n_experts):
            named[p + f"experts.{e}.gate"] = named[p + "experts_in"][e, :cfg.moe_ffn]
            named[p + f"experts.{e}.up"] = named[p + "experts_in"][e, cfg.moe_ffn:] if cfg.gated_ffn else named[p + "experts_in"][e]
            named[p + f"experts.{e}.down"] = named[p + "experts_out"][e]
    return named


ON_DEVICE = os.environ.get("POOT_TP_CUDA") == "1"       # the same comparison on GPUs over NCCL with the real kernels


def run(cfg, named, rank, world, comm):
    dev = f"cuda:{torch.cuda.current_device()}" if ON_DEVICE else "cpu"
    w = from_named_tensors(cfg, named, dev, tp_rank=rank, tp_world=world)
    eng = DecoderEngine(w, num_blocks=9, max_seqs=2, max_tokens=48, max_blocks_per_seq=4, comm=comm, device=dev, use_graphs=False)
    s = FixedBatchSession(eng, 2, 64)
    g = torch.Generator().manual_seed(TOKEN_SEED.get(cfg.family, 5))
    prompts = torch.randint(0, cfg.vocab, (2, 19), generator=g, dtype=torch.int32)
    nxt = torch.randint(0, cfg.vocab, (2, 3), generator=g, dtype=torch.int32)

    def logits():
        local = eng.last_local_logits[:2].float().contiguous()
        if comm is None:
            return local.cpu().clone()
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(parts, local)
        return torch.cat(parts, 1).cpu()
    s.prefill_fast(prompts)
    out = [logits()]
    for t in range(3):
        s.decode(nxt[:, t].tolist())
        out.append(logits())
    return torch.stack(out)


def main() -> int:
    import contextlib
    if ON_DEVICE:
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    dist.init_process_group("nccl" if ON_DEVICE else "gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    results = {}
    with (contextlib.nullcontext() if ON_DEVICE else emulated_kernels()):
        for name in sys.argv[1:]:
            header = HF_FAMILIES[name] if name in ("mpt", "bloom") else {**HF_BASE, **HF_FAMILIES[name]}
            model = Registry.builtin().resolve_hf(header)
            named = named_weights(model)
            try:
                got = run(model.cfg, named, rank, world, NcclComm(rank, world, torch.device("cuda", torch.cuda.current_device()) if ON_DEVICE else torch.device("cpu")))
                want = run(model.cfg, named, 0, 1, None)
                err = (got - want).abs().max().item()
                ref = max(1.0, want.abs().max().item())
                results[name] = {"equal": err < 0.02 * ref, "err": err, "scale": ref, "per_step": (got - want).abs().amax(dim=(1, 2)).tolist()}
            except Exception as e:                                  # reported per family, judged by the test
                results[name] = {"equal": False, "error": f"{type(e).__name__}: {e}"}
    flags = [None] * world
    dist.all_gather_object(flags, {k: (v["equal"], v.get("error")) for k, v in results.items()})
    if rank == 0:
        print(json.dumps({"ranks": flags, **results}), flush=True)
    dist.barrier()
    return 0


if __name__ == "__main__":
    sys.exit(main())
