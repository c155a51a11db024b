"""``python -m poot_b200.serve MODEL [HOST:PORT] [--rows N] [--max-seq N] [--placement tensor:0,1,..] ...``

Single placement runs in this process.  A ``tensor:`` placement is launched one process per GPU
(``python -m torch.distributed.run --nproc-per-node N -m poot_b200.serve ...``): rank 0 owns the HTTP server, the
scheduler and the driver; the other ranks follow the step inputs it broadcasts (website/docs/serve/tensor-parallelism.md).
"""
from __future__ import annotations

import os
import signal
import sys
import threading

from .config import parse_args
from .http import Server, ServerState
from .metrics import Metrics
from .scheduler import ServeEngine


def main(argv=None) -> int:
    try:
        cfg = parse_args(list(sys.argv[1:] if argv is None else argv))
    except ValueError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    from ..llm import LLM
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    comm = None
    if cfg.backend not in ("b200", "cuda", "auto", "oracle", "graph"):
        print(f"poot-serve: --backend {cfg.backend!r}: this build has the device backend (b200), the general device executor "
              "(`graph`) and `oracle`", file=sys.stderr)
        return 2
    if cfg.backend in ("oracle", "graph") and world > 1:
        print(f"poot-serve: the {cfg.backend} backend runs in one process", file=sys.stderr)
        return 2
    pp = 1
    if world > 1:
        import torch
        import torch.distributed as dist
        from ..driver.placement import Placement
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
        dist.init_process_group("nccl")
        if Placement.parse(cfg.placement).kind == "pipeline":     # one stage per process: layers split, no collectives
            pp = world
        else:
            from ..parallel.tp import make_comm
            kind = _comm_kind(cfg.model) if cfg.comm == "auto" else cfg.comm
            comm = make_comm(kind, rank, world, torch.device("cuda", torch.cuda.current_device()))
        from ..ops import cuda_ops as _K
        _K.set_step_budget(cfg.device_step_budget_secs)
        from .follower import init_control_group
        init_control_group(ready_deadline=cfg.ready_deadline_secs, step_deadline=max(cfg.step_deadline_secs, 1.0),
                           heartbeat_timeout=cfg.rank_heartbeat_timeout_secs)
    if _is_encoder_checkpoint(cfg.model):
        return _serve_encoder(cfg)
    from ..driver.features import Incompatible as _Inc, Unavailable as _Unav
    mtp_k = cfg.draft_mtp
    if mtp_k and (world > 1 or cfg.model == "fake" or cfg.lora or cfg.lora_slots):
        print("poot-serve: --draft-mtp runs on the single-device engine, without adapters", file=sys.stderr)
        return 2
    try:
        llm = _open_model(cfg, rank, world, pp, comm, mtp_k)
    except (_Unav, _Inc) as e:
        print(f"poot-serve: {e}", file=sys.stderr)
        return 2
    return _serve(cfg, llm, rank, world, pp, comm)


def _open_model(cfg, rank: int, world: int, pp: int, comm, mtp_k: int):
    from ..llm import LLM
    if cfg.model == "fake":
        return LLM.fake(rows=cfg.rows, max_seq=cfg.max_seq, prefill_chunk=cfg.prefill_chunk, prefill_budget=cfg.prefill_budget or None)
    if cfg.model.startswith("random:"):
        return LLM.random(cfg.model.split(":", 1)[1], rows=cfg.rows, max_seq=cfg.max_seq, prefill_chunk=cfg.prefill_chunk,
                          kv_fraction=cfg.kv_fraction, tp_rank=rank if pp == 1 else 0, tp_world=world if pp == 1 else 1,
                          comm=comm, prefill_budget=cfg.prefill_budget or None, pp_rank=rank if pp > 1 else 0, pp_world=pp,
                          draft_mtp=mtp_k)
    if cfg.backend == "graph":
        # every traced family, equation by equation on the device (no adapter, no draft layer)
        import torch
        return LLM.graph(cfg.model, device="cuda" if torch.cuda.is_available() else "cpu", rows=cfg.rows, max_seq=cfg.max_seq,
                         prefill_chunk=cfg.prefill_chunk, num_blocks=cfg.rows * ((cfg.max_seq + 15) // 16) + 8,
                         prefill_budget=cfg.prefill_budget or None)
    if cfg.backend == "oracle":
        return LLM.oracle(cfg.model, rows=cfg.rows, max_seq=cfg.max_seq, prefill_chunk=cfg.prefill_chunk, lora=cfg.lora,
                          num_blocks=cfg.rows * ((cfg.max_seq + 15) // 16) + 8, prefill_budget=cfg.prefill_budget or None,
                          draft_mtp=mtp_k)
    return LLM.load(cfg.model, rows=cfg.rows, max_seq=cfg.max_seq, prefill_chunk=cfg.prefill_chunk,
                    kv_fraction=cfg.kv_fraction, tp_rank=rank if pp == 1 else 0, tp_world=world if pp == 1 else 1,
                    comm=comm, lora=cfg.lora, prefill_budget=cfg.prefill_budget or None,
                    pp_rank=rank if pp > 1 else 0, pp_world=pp, draft_mtp=mtp_k)


def _serve(cfg, llm, rank: int, world: int, pp: int, comm) -> int:
    from ..llm import LLM
    if cfg.lora_slots > 0:
        if world > 1 or llm.engine is None:
            print("poot-serve: --lora-slots needs the single-device engine", file=sys.stderr)
            return 2
        llm.engine.enable_adapters(cfg.lora_slots, cfg.lora_max_rank)
    if world > 1 and pp == 1 and llm.cfg is not None and llm.engine is not None:
        # the group's plan - placement without duplication, the step's communication rows against the links'
        # capabilities, every device's own byte total - is admitted before the first step (plan/multi_device.py)
        import torch
        from ..driver.placement import Placement as _Pl
        from ..plan.multi_device import MultiDeviceError, Topology, plan_tensor_parallel
        ords = list(_Pl.parse(cfg.placement).ordinals) if cfg.placement != "single" else list(range(world))
        total = torch.cuda.get_device_properties(torch.cuda.current_device()).total_memory
        try:
            plan_tensor_parallel(llm.cfg, Topology.nvswitch(ords, total), cfg.rows, llm.engine.kv.num_blocks, cfg.rows,
                                 comm="fused" if getattr(comm, "fused", False) else "nccl").validate()
        except MultiDeviceError as e:
            print(f"poot-serve: placement {cfg.placement}: {e}", file=sys.stderr)
            return 2
    if world > 1:
        from .follower import follow, LeaderStepEngine
        if rank != 0:
            _drain_on_signal()
            cause = follow(llm.driver.engine)
            print(f"poot-serve rank {rank}: leaving ({cause})", file=sys.stderr, flush=True)
            _leave(llm, collective=cause == "shutdown")
        llm.driver.engine = LeaderStepEngine(llm.driver.engine)
    template = cfg.chat_template
    if cfg.chat_template_file:
        with open(cfg.chat_template_file) as f:
            template = f.read()
    from ..driver.features import Feature as _F, check as _check
    draft = llm.draft                    # --draft-mtp: the model's own multi-token-prediction layer, attached at load
    if cfg.host_embedding:
        if world > 1 or llm.engine is None:
            print("poot-serve: --host-embedding needs the single-device engine", file=sys.stderr)
            return 2
        try:
            freed = llm.engine.host_embedding()
        except ValueError as e:
            print(f"poot-serve: --host-embedding: {e}", file=sys.stderr)
            return 2
        print(f"poot-serve: embedding table hosted, {freed / 2**20:.0f} MiB of device memory freed", file=sys.stderr)
    if cfg.expert_pool:
        from ..driver.placement import Placement as _Pl
        from ..driver.expert_residency import ExpertResidency
        _check([_F.EXPERT_POOL, *_Pl.parse(cfg.placement).features])
        if llm.engine is None:
            print("poot-serve: --expert-pool needs the device engine", file=sys.stderr)
            return 2
        llm.engine.enable_expert_pool(cfg.expert_pool, ExpertResidency())
    if cfg.check_ranges and llm.cfg is not None:
        _prove_ranges(llm.cfg, cfg)
    if cfg.draft_model:
        from ..driver.placement import Placement
        from ..driver.speculate import ModelDraft
        _check([_F.DRAFT_MODEL, *Placement.parse(cfg.placement).features])
        path, _, k = cfg.draft_model.rpartition(":")
        small = (LLM.oracle(path, rows=1, max_seq=cfg.max_seq) if cfg.backend == "oracle" else
                 LLM.load(path, rows=1, max_seq=cfg.max_seq, prefill_chunk=cfg.prefill_chunk, kv_fraction=0.05))
        if small.cfg.vocab != llm.cfg.vocab:
            print("poot-serve: the draft model's vocabulary differs from the served model's", file=sys.stderr)
            return 2
        draft = ModelDraft(small.driver, int(k))
    if cfg.draft_lookup:
        from ..driver.features import Feature, check
        from ..driver.placement import Placement
        from ..driver.speculate import LookupDraft
        draft = LookupDraft.parse(cfg.draft_lookup)
        check([Feature.DRAFT_LOOKUP, *Placement.parse(cfg.placement).features])
    timing = None
    if cfg.device_timing:
        from ..driver.features import Feature, check
        from ..driver.placement import Placement
        from ..profile import TimingOptions, TimingSnapshot
        check([Feature.DEVICE_TIMING, *Placement.parse(cfg.placement).features])     # refused over a device group
        timing = TimingSnapshot(TimingOptions("detailed", max_steps=cfg.timing_max_steps,
                                              max_dispatch_records=cfg.timing_max_dispatch_records,
                                              sample_every=cfg.timing_sample_every))
        if hasattr(llm.driver.engine, "device_timing"):
            llm.driver.engine.device_timing = True
    engine = ServeEngine(llm.driver, llm.tokenizer, Metrics(), cfg.max_pending_requests, cfg.max_queue_wait_secs,
                         draft=draft, timing=timing, step_deadline=cfg.step_deadline_secs or None)
    state = ServerState(engine, cfg, cfg.model_id or os.path.basename(cfg.model.rstrip("/")) or "model",
                        family=llm.cfg.family if llm.cfg is not None else "llama", chat_template=template)
    handle = getattr(llm, "handle", None)
    if handle is not None and getattr(handle.model, "kind", "decoder") == "vlm" and world == 1:
        from ..vlm import VisionLLM
        state.vision = VisionLLM(handle, llm.tokenizer, template, llm)     # /v1/chat/completions takes image_url parts
    server = Server(state)
    engine.start()
    server.start()
    print(f"poot-b200 serving {state.model_id} on http://{cfg.addr} (rows={cfg.rows}, max_seq={cfg.max_seq})", flush=True)
    stop = threading.Event()
    for sig in (signal.SIGINT, signal.SIGTERM):
        signal.signal(sig, lambda *_: stop.set())
    stop.wait()
    server.shutdown()
    if world > 1:
        clean = engine.state != "dead"
        llm.driver.engine.stop_followers("shutdown" if clean else (engine.cause or "engine dead"))
        _leave(llm, collective=clean)
    llm.close()
    return 0


def _comm_kind(model: str) -> str:
    """The fused GEMM + NVLink programs are written for the pre-norm SwiGLU rope layer; a checkpoint of another
    attention stack shards the same way over the library collectives."""
    import json
    path = os.path.join(model, "config.json")
    from ..parallel.tp import DEFAULT_COMM
    if not os.path.isfile(path):
        return DEFAULT_COMM
    from ..models.registry import Registry, UnsupportedFamily
    try:
        with open(path) as f:
            cfg = Registry.builtin().resolve_hf(json.load(f)).cfg
    except (UnsupportedFamily, KeyError, ValueError):
        return DEFAULT_COMM              # the load that follows reports what is wrong with the checkpoint
    return DEFAULT_COMM if getattr(cfg, "plain_block", True) else "nccl"


def _prove_ranges(model_cfg, cfg) -> None:
    """``--check-ranges``: an unproven index of the step graphs stops startup."""
    from ..driver.handle import prove_step_ranges
    try:
        prove_step_ranges(model_cfg, cfg.prefill_chunk)
    except ValueError as e:
        raise SystemExit(f"poot-serve: --check-ranges: {e}") from None


def _is_encoder_checkpoint(path: str) -> bool:
    import json
    header = os.path.join(path, "config.json")
    if not os.path.isfile(header):
        return False
    with open(header) as f:
        return json.load(f).get("model_type") in ("bert",)


def _serve_encoder(cfg) -> int:
    """An encoder checkpoint serves ``/v1/embeddings`` and ``/v1/rerank``: on the device engine, or on the host evaluator
    with ``--backend oracle`` (and when no device is present)."""
    from ..embed import Embedder, EmbedEngine
    backend = "oracle"
    if cfg.backend != "oracle":
        import torch
        backend = "device" if torch.cuda.is_available() else "oracle"
    emb = Embedder.load(cfg.model, backend=backend)
    engine = EmbedEngine(emb, Metrics())
    state = ServerState(engine, cfg, cfg.model_id or emb.name, family="bert")
    server = Server(state)
    server.start()
    print(f"poot-b200 serving encoder {state.model_id} on http://{cfg.addr}", flush=True)
    stop = threading.Event()
    for sig in (signal.SIGINT, signal.SIGTERM):
        signal.signal(sig, lambda *_: stop.set())
    stop.wait()
    server.shutdown()
    return 0


def _drain_on_signal() -> None:
    """A follower that is told to terminate must not exit under a kernel that is waiting for a peer: the handler sets
    the abort word, waits for the device to go idle and only then leaves."""
    def handler(*_):
        import torch
        from ..ops import cuda_ops as K
        K.request_abort()
        try:
            torch.cuda.synchronize()
        finally:
            os._exit(0)
    for sig in (signal.SIGINT, signal.SIGTERM):
        signal.signal(sig, handler)


def _leave(llm, collective: bool = True) -> None:
    """Multi-rank exit.  First make sure no kernel of this rank is resident: set the abort word (any wait on another
    rank returns at once) and synchronise.  After a clean stop the ranks then meet at a barrier before they release the
    peer mappings; after a failure there is no barrier, because a rank may be gone.  The process then leaves without
    running the process group's destructors (tearing down a group that owns captured collectives can block)."""
    import torch
    import torch.distributed as dist
    from ..ops import cuda_ops as K
    K.request_abort()
    torch.cuda.synchronize()
    if collective:
        K.clear_abort()
        dist.barrier()
        torch.cuda.synchronize()
    llm.close()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


if __name__ == "__main__":
    sys.exit(main())
