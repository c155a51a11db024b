#!/usr/bin/env python
"""Headline benchmark: Llama-3-8B (bf16, random-init weights, synthetic token ids) decode and prefill
throughput on N B200s with tensor parallelism.

    python bench.py --gpus N --steps K --warmup W

A timed *step* is one decode step of a batch of 64 sequences (each at context 512+).  The JSON line's
``value`` is decode tokens/s at batch 64 over the whole job; batch-1 decode tokens/s and the 512-token
prefill tokens/s ride in ``extra``.  Device time is taken with CUDA events around the K timed steps
(max over ranks); ``e2e`` repeats the measurement through the public step API with the per-step
host->device input copy from pinned memory and the device->host read of the sampled tokens included.
Weights (16 GB) are far larger than L2 (126 MB), so every step streams them from HBM; no L2 flush is needed.

``--impl reference`` reports that the reference (a Rust workspace that needs a pinned nightly toolchain,
LLVM 22 and crates.io) cannot be installed or run in this environment.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# The reference publishes no Llama-3-8B, no batch > 1 and no B200 number, so ``vs_baseline`` is null.  For context
# only, ``extra`` carries the ratio of the batch-1 decode rate to the reference's closest published cell: single-stream
# bf16 decode of its largest dense bf16 model (qwen3-4b, ISL 128) on an RTX PRO 6000 Blackwell.  Different model,
# different GPU: not a like-for-like comparison.
PUBLISHED_BS1_DECODE_TOK_S_QWEN3_4B_RTXPRO6000 = 112.9


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons in the background while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except Exception:
            self.proc.kill()
            out = ""
        sm, mx, reasons = [], [], set()
        for line in out.splitlines():
            p = [x.strip() for x in line.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1])); mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        # the busiest half of the samples is "under load"
        sm_sorted = sorted(sm)
        return {"sm_mhz": statistics.median(sm_sorted[: max(1, len(sm_sorted) // 2)]) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args) -> None:
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference is a Rust workspace (pinned nightly, LLVM 22 llc, crates.io deps, no setup.py/"
                      "pyproject): pip install of the reference tree fails and cargo/rustc are not in the image"}))


def driver_e2e(eng, cfg, B, prompts, W, Ksteps, max_len, timed):
    """Batch decode through the public serving path: ``Driver.open`` B sequences, prefill them in chunks, then time
    ``Ksteps`` iterations of ``Driver.step`` (host planning, pinned H2D of the step inputs, graph replay, D2H of the
    picked tokens) + ``Driver.commit``."""
    from poot_b200.driver.driver import Driver
    from poot_b200.driver.engines import DeviceStepEngine
    from poot_b200.driver.sampler import SamplingParams
    from poot_b200.ops import cuda_ops as K
    d = Driver(DeviceStepEngine(eng), eng.kv.num_blocks, B, max_len, cfg.vocab, prefill_chunk=512, prefix_caching=False)
    # sequences that finish prefill early keep decoding while the others are still being prefilled (one piece per
    # step), so every sequence needs room for about B extra tokens before the timed region starts
    budget = min(max_len - prompts.shape[1] - 1, B + W + Ksteps + 16)
    sids = [d.open(prompts[b].tolist(), SamplingParams(max_tokens=budget, ignore_eos=True)) for b in range(B)]

    def step():
        for r in d.step(sids):
            if r.token is not None:
                d.commit(r.seq_id, [r.token])

    guard = 0
    while any(d.seqs[s].generated == 0 for s in sids):       # chunked prefill until every sequence has sampled once
        step()
        guard += 1
        if guard > 4 * B + 64:
            raise RuntimeError("prefill through the driver did not converge")
    for _ in range(W):
        step()
    ms = timed(step, Ksteps)
    K.check_status()
    for s in sids:
        d.release(s, "preempted")
    return {"tok_s": B * Ksteps / (ms / 1e3), "ms_per_step": ms / Ksteps}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours")
    ap.add_argument("--model", default="llama-3-8b")
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=512)
    ap.add_argument("--comm", default="auto", choices=["auto", "fused", "nccl"],
                    help="collectives of a tensor-parallel run: the in-kernel NVLink programs (fused) or the library's "
                         "(nccl); auto = the package default (poot_b200.parallel.tp.DEFAULT_COMM)")
    ap.add_argument("--nvls", type=int, default=0, help="1: let the library use in-switch (multicast) reductions")
    ap.add_argument("--skip-bs1", action="store_true")
    ap.add_argument("--pdl", type=int, default=1, help="programmatic dependent launch between kernels")
    ap.add_argument("--gemv-max-m", type=int, default=None, help="rows served by the SIMT GEMV (0 = tensor cores)")
    ap.add_argument("--dev-set", action="append", default=[], metavar="FIELD=INT",
                    help="development only: override a model field, e.g. n_layers=2 (the JSON line is marked invalid)")
    ap.add_argument("--watchdog", type=float, default=300.0,
                    help="seconds after which a rank that is still running prints an error line and leaves "
                         "(a rank stuck in a collective must not keep the GPUs of the whole job)")
    ap.add_argument("--quant", default="none", choices=["none", "q4_k"],
                    help="q4_k: Q4_K projections + Q8_0 embeddings, batch-1 decode after a 128-token prompt")
    args = ap.parse_args()
    if args.quant != "none":
        args.batch, args.prompt, args.skip_bs1 = 1, 128, True
    if args.impl == "reference":
        reference_arm(args)
        return

    # Every way out of a multi-rank run (watchdog, SIGTERM, an exception) first makes this rank's kernels stop waiting
    # for peers and the device go idle, and only then leaves the process (poot_b200/parallel/teardown.py).
    from poot_b200.parallel import teardown

    def _say(code: int) -> None:
        if code != 0 and int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"metric": "decode tok/s", "value": None, "n_gpus": args.gpus,
                              "error": f"run ended early with code {code} (watchdog {args.watchdog:.0f} s, signal or fault); "
                                       "the device was drained before exit"}), flush=True)

    dog = teardown.install(watchdog_seconds=args.watchdog, on_exit=_say)
    if not args.nvls:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")

    import torch
    import torch.distributed as dist
    from poot_b200.models.config import PRESETS
    from poot_b200.ops import cuda_ops as K
    from poot_b200.runtime.engine import DecoderEngine, StepShape
    from poot_b200.runtime.session import FixedBatchSession
    from poot_b200.runtime.weights import random_quant_weights, random_weights

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world and world == 1 and args.gpus > 1:
        # launched without torchrun: re-exec under it
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", "29511", __file__, *sys.argv[1:]]
        os.execv(sys.executable, cmd)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    comm = None
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
        from poot_b200.parallel.tp import DEFAULT_COMM, make_comm
        if args.comm == "auto":
            args.comm = DEFAULT_COMM
        comm = make_comm(args.comm, rank, world, dev)
        teardown.set_comm(comm)

    K.set_pdl(bool(args.pdl))
    if args.gemv_max_m is not None:
        K.GEMV_MAX_M = args.gemv_max_m
    cfg = PRESETS[args.model]()
    for kv in args.dev_set:
        field, _, val = kv.partition("=")
        setattr(cfg, field, int(val))
    W, Ksteps, B, P = max(args.warmup, 3), args.steps, args.batch, args.prompt
    max_len = P + (W + Ksteps) * 2 + 64
    bps = (max_len + 15) // 16
    if args.quant == "q4_k":
        weights = random_quant_weights(cfg, dev, "Q4_K", "Q8_0", seed=0, tp_rank=rank, tp_world=world)
    else:
        ep = world if cfg.is_moe else 1      # experts split over the ranks, attention tensor-parallel over the same ranks
        weights = random_weights(cfg, dev, seed=0, tp_rank=rank, tp_world=world, ep_rank=rank if ep > 1 else 0, ep_world=ep)
    prefill_chunk_seqs = max(1, min(B, 2048 // P))
    eng = DecoderEngine(weights, num_blocks=B * bps + bps, max_seqs=B, max_tokens=max(prefill_chunk_seqs * P, B),
                        max_blocks_per_seq=bps, comm=comm)
    g = torch.Generator().manual_seed(0)
    prompts = torch.randint(0, cfg.vocab, (B, P), generator=g, dtype=torch.int32)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn, n):
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1))

    extra = {}
    # ------------------------------------------------------------------ prefill (bs1: one 512-token step)
    sess1 = FixedBatchSession(eng, 1, max_len)
    sess1.prefill_fast(prompts[:1])  # warm-up + capture
    sess1.prefill_fast(prompts[:1])
    sess1.prefill_fast(prompts[:1])
    ms = timed(lambda: sess1.prefill_fast(prompts[:1]), 5)
    extra["prefill_tok_s_bs1"] = P / (ms / 5 / 1e3)
    extra["ttft_ms_bs1"] = ms / 5

    # ------------------------------------------------------------------ decode bs1
    if not args.skip_bs1:
        tok = [1]
        shape1 = StepShape(1, 1, 0, chain=True)
        sess1.decode_chain(tok, W)
        ms = timed(lambda: eng.run(shape1), Ksteps)
        sess1.len_t = sess1.len_t + Ksteps
        extra["decode_tok_s_bs1"] = Ksteps / (ms / 1e3)
        extra["decode_ms_per_step_bs1"] = ms / Ksteps
        # end to end: per step H2D of the inputs (pinned) + D2H of the sampled token
        for _ in range(3):
            tok = sess1.decode(tok)[:, 0].tolist()
        state = {"tok": tok}

        def e2e_step1():
            state["tok"] = sess1.decode(state["tok"])[:, 0].tolist()
        ms = timed(e2e_step1, Ksteps)
        extra["e2e_decode_tok_s_bs1"] = Ksteps / (ms / 1e3)

    # ------------------------------------------------------------------ batch prefill (throughput)
    sessB = FixedBatchSession(eng, B, max_len)
    sub = FixedBatchSession(eng, prefill_chunk_seqs, max_len)

    def batch_prefill():
        # sequences are prefilled prefill_chunk_seqs at a time; block tables of the chunk are bound per step
        first = []
        for c in range(0, B, prefill_chunk_seqs):
            n = min(prefill_chunk_seqs, B - c)
            sub.block_tables_host[:n].copy_(sessB.block_tables_host[c:c + n])
            eng.block_tables[:n, :sub.blocks_per_seq].copy_(sub.block_tables_host[:n], non_blocking=True)
            if n != sub.batch:
                break
            first.append(sub.prefill_fast(prompts[c:c + n]).clone())
        return torch.cat(first)

    first = batch_prefill()
    ms = timed(batch_prefill, 1)
    extra["prefill_tok_s_batched"] = B * P / (ms / 1e3)
    first = batch_prefill()
    eng.block_tables[:B, :sessB.blocks_per_seq].copy_(sessB.block_tables_host)
    sessB.lengths = [P] * B

    # ------------------------------------------------------------------ decode bs64 (headline)
    shapeB = StepShape(B, B, 0, chain=True)
    sessB.decode_chain(first[:, 0].tolist(), W)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_dev = timed(lambda: eng.run(shapeB), Ksteps)
    sessB.len_t = sessB.len_t + Ksteps
    clocks = sampler.stop() if rank == 0 else {}
    K.check_status()
    launches = eng.launches_per_step[eng._key(shapeB)] * Ksteps
    value = B * Ksteps / (ms_dev / 1e3)

    tok = eng.picked[:B, 0].tolist()
    for _ in range(3):
        tok = sessB.decode(tok)[:, 0].tolist()
    state = {"tok": tok}

    def e2e_step():
        state["tok"] = sessB.decode(state["tok"])[:, 0].tolist()
    ms_e2e = timed(e2e_step, Ksteps)
    e2e_value = B * Ksteps / (ms_e2e / 1e3)
    K.check_status()

    # ---- the same decode measured through the serving driver (open / step / commit), one GPU only ----
    api = "FixedBatchSession.decode"
    if world == 1:
        try:
            r = driver_e2e(eng, cfg, B, prompts, W, Ksteps, max_len, timed)
            extra["e2e_session_tok_s"] = e2e_value
            e2e_value, api = r["tok_s"], "Driver.step + Driver.commit"
            extra["e2e_driver_ms_per_step"] = r["ms_per_step"]
        except Exception as e:      # keep the session-level number
            extra["e2e_driver_error"] = f"{type(e).__name__}: {e}"[:200]

    if rank == 0:
        out = {
            "metric": ("decode tok/s (bs1, Q4_K weights), max over ranks" if args.quant != "none" else
                       "decode tok/s (bs64; bs1 and prefill tok/s in extra), max over ranks"),
            "value": value, "unit": "tok/s", "n_gpus": world, "steps": Ksteps, "warmup": W,
            "ms_per_step": ms_dev / Ksteps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"model": cfg.name + ("" if args.quant == "none" else "-Q4_K(proj)+Q8_0(embed)"), "global_batch": B, "seq_len": P, "parallelism": (f"ep{world}+tp{world}(attention)" if cfg.is_moe and world > 1 else f"tp{world}"),
                       **({"INVALID": "development run with " + ",".join(args.dev_set)} if args.dev_set else {}),
                       "comm": args.comm if world > 1 else "none",
                       "l2": f"inputs larger than L2: {weights.nbytes() / 2**30:.1f} GiB of weights per rank stream from HBM every step",
                       "kv": "paged, block 16, bf16", "decode": "CUDA graph replay per token, greedy"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": sessB.h2d_bytes(B, B),
                    "d2h_bytes_per_step": B * 8, "api": api},
            "gpu_launches": launches,
            "extra": extra,
        }
        if "decode_tok_s_bs1" in extra:
            extra["bs1_vs_reference_published_qwen3_4b_rtxpro6000"] = (
                extra["decode_tok_s_bs1"] / PUBLISHED_BS1_DECODE_TOK_S_QWEN3_4B_RTXPRO6000)
        if world > 1 and args.comm != "fused":
            out["config"]["note"] = ("library collectives (the baseline path); the fused GEMM + NVLink programs are "
                                     "selected with --comm fused")
        print(json.dumps(out))
    if dog is not None:
        dog.cancel()
    if world > 1:
        # Tear-down of a process group that owns captured NCCL graphs can block; results are out, so meet, go idle,
        # release the peer mappings (close() drains the device first) and leave without running the destructors.
        sys.stdout.flush()
        dist.barrier()
        torch.cuda.synchronize()
        if comm is not None and hasattr(comm, "close"):
            comm.close()
        os._exit(0)


if __name__ == "__main__":
    try:
        main()
    except SystemExit:
        raise
    except BaseException as e:      # say what failed in the one-line format, drain the device, then leave
        import traceback
        traceback.print_exc()
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"metric": "decode tok/s", "value": None, "error": f"{type(e).__name__}: {e}"[:400]}), flush=True)
        sys.stdout.flush()
        from poot_b200.parallel import teardown as _td
        _td._state["on_exit"] = None
        _td.drain_and_exit(1)
