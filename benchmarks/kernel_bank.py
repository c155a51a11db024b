#!/usr/bin/env python
"""Kernel bank: kernel-level cases timed on the device against their memory / compute roofline.

The counterpart of the reference's performance bank (benchmarks/performance-bank/cases.json: dense and
packed decode GEMV, batched decode GEMM, prefill GEMMs, attention, expert routing).  Each case launches
one kernel over rotating operand copies larger than L2 (so every launch streams from HBM), captured in
a CUDA graph so that launch overhead is not in the number, and reports microseconds per launch plus the
achieved fraction of the measured peaks (MEASURED_PEAKS.json when present).

    python benchmarks/kernel_bank.py [--case NAME ...] [--pdl 0|1] [--once]

``--once`` runs each selected case a single time without timing (for use under ncu).
"""
from __future__ import annotations

import argparse
import json
import math
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

import torch  # noqa: E402

from poot_b200.ops import cuda_ops as K  # noqa: E402


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def time_graph(fns, reps=5):
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for f in fns:
            f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for _ in range(reps):
            for f in fns:
                f()
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (2 * reps * len(fns))


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def gemm_case(M, N, Kd, kind):
    copies = max(2, int(400e6 // (N * Kd * 2)) + 1)
    x = rnd(M, Kd)
    Ws = [rnd(N, Kd, scale=0.02) for _ in range(copies)]
    outs = [torch.empty(M, N, device="cuda", dtype=torch.bfloat16) for _ in range(copies)]
    if kind == "gemv":
        fns = [(lambda W=W, o=o: K.gemv(x, W, K.EPI_STORE, out=o)) for W, o in zip(Ws, outs)]
    elif kind == "skinny":
        fns = [(lambda W=W, o=o: K.gemm_skinny(x, W, K.EPI_STORE, out=o)) for W, o in zip(Ws, outs)]
    else:
        fns = [(lambda W=W, o=o: K.gemm(x, W, K.EPI_STORE, out=o)) for W, o in zip(Ws, outs)]
    return fns, N * Kd * 2 + M * Kd * 2 + M * N * 2, 2.0 * M * N * Kd


def attn_case(B, ctx, Hq=32, Hkv=8, D=128):
    bps = (ctx + 15) // 16
    nb = B * bps
    kpool, vpool = rnd(nb, Hkv, 16, D), rnd(nb, Hkv, 16, D)
    bt = torch.randperm(nb, device="cuda").to(torch.int32).view(B, bps)
    q = rnd(B, Hq * D)
    row_ctx = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    out = torch.empty(B, Hq * D, device="cuda", dtype=torch.bfloat16)
    splits = 1 if B * Hkv >= 148 else max(1, min(16, 296 // (B * Hkv)))
    scr = (torch.empty(B * Hq * splits * D, device="cuda"), torch.empty(B * Hq * splits * 2, device="cuda"))
    fn = lambda: K.attn_paged(q, kpool, vpool, bt, None, row_ctx, Hq, Hkv, D, 1 / math.sqrt(D), out=out,
                              splits=splits, scratch=scr)
    return [fn], 2 * B * ctx * Hkv * D * 2, 4.0 * B * ctx * Hq * D


def general_attn_case(B, ctx, Hq, Hkv, Dk, Dv):
    """The general attention kernel (head widths the tuned kernels do not take: 256, or 192 / 128 latent attention)."""
    bps = (ctx + 15) // 16
    nb = B * bps
    pd = max(Dk, Dv)
    kpool, vpool = rnd(nb, Hkv, 16, pd), rnd(nb, Hkv, 16, pd)
    bt = torch.randperm(nb, device="cuda").to(torch.int32).view(B, bps)
    q = rnd(B, Hq * Dk)
    row_ctx = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
    out = torch.empty(B, Hq * Dv, device="cuda", dtype=torch.bfloat16)
    fn = lambda: K.attn_general(q, kpool, vpool, bt, None, row_ctx, Hq, Hkv, Dk, Dv, 1 / math.sqrt(Dk), out)
    return [fn], B * ctx * Hkv * (Dk + Dv) * 2, 2.0 * B * ctx * Hq * (Dk + Dv)


def segments(n_seq, rows_each):
    segs = torch.zeros(n_seq, 4, dtype=torch.int32)
    for i in range(n_seq):
        segs[i] = torch.tensor([i * rows_each, rows_each, i, 16 if rows_each == 1 else 0])
    return segs.cuda()


def gdn_case(n_seq, rows_each, nk=16, nv=48, D=128):
    """Gated delta rule over ``n_seq`` sequence pieces (decode: one row each; prefill: ``rows_each`` rows)."""
    T = n_seq * rows_each
    C = (2 * nk + nv) * D
    qkv, ba = rnd(T, C, scale=0.3), rnd(T, 2 * nv, scale=0.3)
    state = torch.zeros(n_seq, nv, D, D, device="cuda")
    out = torch.empty(T, nv * D, device="cuda", dtype=torch.bfloat16)
    dtb, alog = torch.zeros(nv, device="cuda"), torch.zeros(nv, device="cuda")
    segs = segments(n_seq, rows_each)
    fn = lambda: K.gdn_scan(qkv, ba, 0, nv, dtb, alog, state, segs, out, nk, nv, D)
    return [fn], 2 * n_seq * nv * D * D * 4 + T * C * 2, 6.0 * T * nv * D * D


def ssd_case(n_seq, rows_each, nh=128, G=8, N=128, P=64):
    """Mamba2 recurrence over ``n_seq`` sequence pieces."""
    T = n_seq * rows_each
    I = nh * P
    C = I + 2 * G * N
    xbc, dtm = rnd(T, C, scale=0.3), rnd(T, nh, scale=0.3)
    state = torch.zeros(n_seq, nh, N, P, device="cuda")
    out = torch.empty(T, I, device="cuda", dtype=torch.bfloat16)
    z = torch.zeros(nh, device="cuda")
    segs = segments(n_seq, rows_each)
    fn = lambda: K.ssd_scan(xbc, dtm, 0, z, z, z, state, segs, out, nh, G, N, P)
    return [fn], 2 * n_seq * nh * N * P * 4 + T * C * 2, 4.0 * T * nh * N * P


def conv_case(n_seq, rows_each, C=10240, Kc=4):
    T = n_seq * rows_each
    x = rnd(T, C)
    w = torch.randn(C, Kc, device="cuda")
    state = torch.zeros(n_seq, Kc - 1, C, device="cuda")
    out = torch.empty(T, C, device="cuda", dtype=torch.bfloat16)
    segs = segments(n_seq, rows_each)
    fn = lambda: K.causal_conv_silu(x, 0, C, w, state, segs, out)
    return [fn], 2 * T * C * 2 + 2 * n_seq * (Kc - 1) * C * 4, 2.0 * T * C * Kc


def flash_case(rows, Hq=32, Hkv=8, D=128):
    """Tensor-core prefill attention of one sequence of ``rows`` tokens."""
    import numpy as np
    bps = (rows + 15) // 16
    kpool, vpool = rnd(bps, Hkv, 16, D), rnd(bps, Hkv, 16, D)
    bt = torch.arange(bps, device="cuda", dtype=torch.int32).view(1, bps)
    q = rnd(rows, Hq * D)
    out = torch.empty(rows, Hq * D, device="cuda", dtype=torch.bfloat16)
    tiles, _ = K.flash_tiles(np.zeros(rows, np.int32), np.arange(rows, dtype=np.int32))
    tl = torch.from_numpy(tiles).cuda()
    fn = lambda: K.attn_flash_prefill(q, kpool, vpool, bt, tl, Hq, Hkv, 1 / math.sqrt(D), out)
    return [fn], 2 * rows * Hkv * D * 2 + 2 * rows * Hq * D * 2, 2.0 * rows * rows * Hq * D      # causal: half of 4 L^2 H D


def route_case(T, E, k, mode):
    from poot_b200.ops import moe_ops as M
    logits = torch.randn(T, E, device="cuda")
    ids, gates = torch.zeros(T * k, dtype=torch.int32, device="cuda"), torch.zeros(T * k, device="cuda")
    dense = torch.zeros(E * T, device="cuda")
    bias = torch.zeros(E, device="cuda") if mode == "sigmoid" else None
    fn = lambda: M.moe_route(logits, k, True, ids, gates, dense, mode=mode, select_bias=bias, n_group=8 if mode == "sigmoid" else 1,
                             topk_group=4 if mode == "sigmoid" else 1)
    return [fn], T * E * 8, 0.0


def replace_rows_case(T, D, share=0.5):
    """Image rows in place of token embeddings: half of the rows flagged, so half of ``rows`` is read and written."""
    h, rows = rnd(T, D), rnd(T, D)
    flags = (torch.rand(T, device="cuda") < share).to(torch.int32)
    fn = lambda: K.replace_rows_(h, rows, flags)
    return [fn], int(2 * T * D * 2 * share) + T * 4, 0.0


def encoder_case(n_seq, length, hidden=384, heads=12, ffn=1536, layers=6):
    """A MiniLM-sized BERT encoder over a ragged batch through ``runtime/encoder_engine.py`` (the whole program: it is timed
    eagerly inside one graph capture like the kernels; bytes = the weights once, flops = the projections)."""
    from poot_b200.models.encoder import EncoderConfig, EncoderModel
    from poot_b200.runtime.encoder_engine import EncoderEngine
    cfg = EncoderConfig(n_layers=layers, hidden=hidden, n_heads=heads, ffn=ffn, vocab=30522, max_position=512)
    shapes = EncoderModel(cfg).weight_shapes()
    tensors = {k: torch.randn(*v) * 0.02 for k, v in shapes.items()}
    eng = EncoderEngine(cfg, tensors, "cuda", max_tokens=n_seq * length, max_rows=n_seq)
    seqs = [list(range(3, 3 + length))] * n_seq
    N = n_seq * length
    eng._bind(seqs, None)                        # the host layout once; the timed part is the device program

    def fn():
        eng._bind = lambda s, t: (N, [length] * n_seq)
        eng.forward(seqs)
    wbytes = sum(int(torch.tensor(v).prod()) * 2 for k, v in shapes.items() if k.startswith("layers."))
    flops = 2.0 * N * layers * (4 * hidden * hidden + 2 * hidden * ffn) + 4.0 * layers * n_seq * length * length * hidden
    return [fn], wbytes, flops


def quant_decode_case(layers=4):
    """Eager batch-1 decode steps of the Q4_K / Q8_0 Llama-3-8B stack cut to ``layers`` layers (a launch list shows
    the share of the packed GEMV, attention and the row kernels); bytes = the packed weights of those layers."""
    from poot_b200.models.config import PRESETS
    from poot_b200.runtime.engine import DecoderEngine
    from poot_b200.runtime.session import FixedBatchSession
    from poot_b200.runtime.weights import random_quant_weights
    cfg = PRESETS["llama-3-8b"]()
    cfg.n_layers = layers
    w = random_quant_weights(cfg, "cuda", seed=0)
    max_len = 768
    bps = max_len // 16
    eng = DecoderEngine(w, num_blocks=bps, max_seqs=1, max_tokens=128, max_blocks_per_seq=bps, use_graphs=False)
    s = FixedBatchSession(eng, 1, max_len)
    s.len_t = torch.full((1,), 200, dtype=torch.int32)
    return [lambda: s.decode([1])], w.nbytes(), 0.0


def tp_oneshot_pair_case(world=2, T=64, H=4096, Kl=7168):
    """The fused row-parallel GEMM + one-shot all-reduce + reduce/RMSNorm pair of a tensor-parallel decode step with
    every rank of the group emulated on ONE GPU (a profiler captures single-GPU programs only): each rank has its own
    flag block, inbox, step counter and weight shard in this GPU's memory, so the "peer" stores land locally.  Launch
    order per round: every rank's step-begin, every rank's GEMM, then every rank's reduce+norm - a kernel that waits on
    flags is enqueued on the same stream after the kernels that set them, so nothing waits on a later launch.  One call
    of the returned function is one round; the time reported is per kernel launch (2 * world + world launches a round)."""
    from ctypes import c_float, c_int, c_void_p
    from poot_b200.ops._lib import check
    P = c_void_p
    K.register_signature("poot_tp_begin_step", [P, P, P])
    K.register_signature("poot_tp_norm", [P, P, P, P, P, c_int, c_int, c_float, c_int, c_int, c_int, c_int, c_int,
                                          c_int, c_int, P, P, P, P, P, P])
    K.register_signature("poot_gemm_skinny_tp", [c_int, P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                                 c_int, c_int, c_int, c_int, c_int, P, P, P, P, c_int, c_int, P, P, P])
    begin, norm, gemm = K.fn("poot_tp_begin_step"), K.fn("poot_tp_norm"), K.fn("poot_gemm_skinny_tp")
    MAX_ROWS, RS_SITES, AG_SITES = 128, 1, 2
    dev = torch.device("cuda")
    flags = [torch.zeros(256, dtype=torch.int32, device=dev) for _ in range(world)]
    inbox = [torch.zeros(2 * world * MAX_ROWS * H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    epoch = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(world)]
    ticket = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(world)]
    copies = 3          # rotate weight copies so that every launch streams cold weights (inputs larger than L2)
    W = [[rnd(H, Kl, scale=0.02) for _ in range(copies)] for _ in range(world)]
    x = [rnd(T, Kl, scale=0.5) for _ in range(world)]
    h = [torch.zeros(T, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    wn = torch.ones(H, dtype=torch.bfloat16, device=dev)
    xo = [torch.zeros(T, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    fpeer = (c_void_p * world)(*[f.data_ptr() for f in flags])
    ipeer = (c_void_p * world)(*[b.data_ptr() for b in inbox])
    st = K.status_word(dev)
    ck = K.skinny_cluster(H, Kl)
    it = [0]

    def one_round():
        s = K._stream()
        c = it[0] % copies
        it[0] += 1
        for r in range(world):
            check(begin(epoch[r].data_ptr(), st.data_ptr(), s), "begin")
        for r in range(world):
            check(gemm(K.EPI_STORE, x[r].data_ptr(), W[r][c].data_ptr(), None, H, Kl, Kl, H, ck, world, r, MAX_ROWS, -1,
                       AG_SITES, 0, RS_SITES, epoch[r].data_ptr(), flags[r].data_ptr(), fpeer, ipeer, H, T,
                       ticket[r].data_ptr(), st.data_ptr(), s), "gemm_skinny_tp")
        for r in range(world):
            check(norm(h[r].data_ptr(), inbox[r].data_ptr(), wn.data_ptr(), None, xo[r].data_ptr(), T, H, 1e-5, world, r,
                       MAX_ROWS, 0, AG_SITES, 0, RS_SITES, epoch[r].data_ptr(), flags[r].data_ptr(), fpeer,
                       ticket[r].data_ptr(), st.data_ptr(), s), "tp_norm")
    # per launch: the weight shard streams once per GEMM; the reduce reads world partial tiles
    per_round_bytes = world * (H * Kl * 2 + T * Kl * 2 + (world + 1) * T * H * 2 + T * H * 2)
    return [one_round], per_round_bytes, 2.0 * world * T * H * Kl


CASES = {
    "dense-decode-gemv-qkv": lambda: gemm_case(1, 6144, 4096, "skinny"),
    "dense-decode-gemv-o": lambda: gemm_case(1, 4096, 4096, "skinny"),
    "dense-decode-gemv-gate-up": lambda: gemm_case(1, 28672, 4096, "skinny"),
    "dense-decode-gemv-down": lambda: gemm_case(1, 4096, 14336, "skinny"),
    "dense-decode-gemv-lm-head": lambda: gemm_case(1, 128256, 4096, "skinny"),
    "simt-decode-gemv-gate-up": lambda: gemm_case(1, 28672, 4096, "gemv"),
    "batched-decode-gemm-m8-gate-up": lambda: gemm_case(8, 28672, 4096, "skinny"),
    "batched-decode-gemm-m64-qkv": lambda: gemm_case(64, 6144, 4096, "skinny"),
    "batched-decode-gemm-m64-o": lambda: gemm_case(64, 4096, 4096, "skinny"),
    "batched-decode-gemm-m64-gate-up": lambda: gemm_case(64, 28672, 4096, "skinny"),
    "batched-decode-gemm-m64-down": lambda: gemm_case(64, 4096, 14336, "skinny"),
    "batched-decode-gemm-m64-lm-head": lambda: gemm_case(64, 128256, 4096, "skinny"),
    "prefill-gemm-m512-qkv": lambda: gemm_case(512, 6144, 4096, "tiled"),
    "prefill-gemm-m512-gate-up": lambda: gemm_case(512, 28672, 4096, "tiled"),
    "prefill-gemm-m512-down": lambda: gemm_case(512, 4096, 14336, "tiled"),
    "prefill-gemm-m2048-gate-up": lambda: gemm_case(2048, 28672, 4096, "tiled"),
    "prefill-gemm-m8192-k4096-n4096": lambda: gemm_case(8192, 4096, 4096, "tiled"),
    "attention-decode-b1-ctx4096": lambda: attn_case(1, 4096),
    "attention-decode-b64-ctx1024": lambda: attn_case(64, 1024),
    "attention-decode-b64-ctx4096": lambda: attn_case(64, 4096),
    "prefill-attention-2048": lambda: flash_case(2048),
    "prefill-attention-8192": lambda: flash_case(8192),
    "attention-general-d256-b64-ctx1024": lambda: general_attn_case(64, 1024, 8, 4, 256, 256),
    "attention-general-latent-b16-ctx1024": lambda: general_attn_case(16, 1024, 128, 128, 192, 128),
    "scan-delta-rule-decode-b64": lambda: gdn_case(64, 1),
    "scan-delta-rule-prefill-512": lambda: gdn_case(1, 512),
    "scan-ssd-decode-b64": lambda: ssd_case(64, 1),
    "scan-ssd-prefill-512": lambda: ssd_case(1, 512),
    "causal-conv-decode-b64": lambda: conv_case(64, 1),
    "causal-conv-prefill-512": lambda: conv_case(1, 512),
    "replace-rows-1377x2048": lambda: replace_rows_case(1377, 2048),
    "encoder-minilm-b32-len128": lambda: encoder_case(32, 128),
    "quant-decode-steps-q4k-4-layers": lambda: quant_decode_case(4),
    "tp-oneshot-gemm-norm-pair-emulated-w2-m64": lambda: tp_oneshot_pair_case(2, 64, 4096, 7168),
    "expert-routing-softmax-512x128-top8": lambda: route_case(512, 128, 8, "softmax"),
    "expert-routing-sigmoid-groups-512x256-top8": lambda: route_case(512, 256, 8, "sigmoid"),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", action="append")
    ap.add_argument("--pdl", type=int, default=1)
    ap.add_argument("--once", action="store_true")
    a = ap.parse_args()
    K.set_pdl(bool(a.pdl))
    bw, fl, src = peaks()
    for name in (a.case or list(CASES)):
        fns, nbytes, flops = CASES[name]()
        if a.once:
            for f in fns[:1]:
                f()
            torch.cuda.synchronize()
            print(json.dumps({"case": name, "ran": 1}))
            continue
        us = time_graph(fns)
        t_mem, t_fl = nbytes / bw * 1e6, flops / fl * 1e6
        roof = max(t_mem, t_fl)
        print(json.dumps({"case": name, "us": round(us, 2), "roofline_us": round(roof, 2),
                          "bound": "memory" if t_mem >= t_fl else "compute", "frac_of_" + src: round(roof / us, 3),
                          "GBs": round(nbytes / us / 1e3, 1), "TFLOPs": round(flops / us / 1e6, 1)}), flush=True)
        del fns
        torch.cuda.empty_cache()
    K.check_status()


if __name__ == "__main__":
    main()
