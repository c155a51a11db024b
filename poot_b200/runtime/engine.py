"""Per-rank device engine: static step buffers, paged KV pools, the kernel program of one step, and
CUDA-graph capture / replay of that program.

A *step* runs ``T`` query tokens (decode: one per sequence row; prefill: a chunk of one or more sequences)
through the stack and samples one token for each of ``B`` logit rows.  All step inputs live in fixed device
buffers that the host overwrites in place before a replay, so one captured graph per ``(T, B, sampler)`` shape
serves every position - the record-on-first-step / replay design of the reference executor
(crates/poot-executor/src/engine.rs:2454-2700, crates/poot-ptx-runtime/src/graph.rs:11-56), here with one
process per GPU and no host work between kernels.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from ..models.config import DecoderConfig
from ..ops import cuda_ops as K
from .rope import rope_tables
from .weights import DecoderWeights

KV_BLOCK = K.KV_BLOCK


@dataclass
class StepShape:
    tokens: int         # T: query tokens in the step
    logit_rows: int     # B: rows that get logits + a sampled token
    sampler: int = 0    # 0 greedy, 1..3 Gumbel family rule
    chain: bool = False  # append the device-side advance (decode chaining)
    adjust: bool = False    # apply the sparse logit adjustments (bias, penalties) before sampling
    guided: bool = False    # also add the dense guided-decoding mask
    logprobs: bool = False  # record the picked token's log-probability
    lora: bool = False      # some row of the step selects a resident adapter (adds the per-row low-rank terms)
    embeds: bool = False    # rows of another modality replace the embeddings of flagged tokens (``bind_embeds``)
    mrope: bool = False     # sectioned rotary: the step's cos / sin rows were assembled per token (``bind_rope_streams``)


class KVPool:
    """Paged K/V pools, one pair per layer: ``[num_blocks, Hkv_local, 16, D]`` bf16."""

    def __init__(self, cfg: DecoderConfig, num_blocks: int, device, tp_world: int = 1, n_layers: Optional[int] = None):
        self.num_blocks = num_blocks
        self.hkv = max(cfg.n_kv_heads // tp_world, 1)
        shape = (cfg.n_layers if n_layers is None else n_layers, 2, num_blocks, self.hkv, KV_BLOCK, cfg.head_dim)
        self.buf = torch.zeros(shape, dtype=torch.bfloat16, device=device)

    def k(self, layer: int) -> torch.Tensor:
        return self.buf[layer, 0]

    def v(self, layer: int) -> torch.Tensor:
        return self.buf[layer, 1]

    @staticmethod
    def bytes_per_block(cfg: DecoderConfig, tp_world: int = 1) -> int:
        return cfg.n_layers * 2 * max(cfg.n_kv_heads // tp_world, 1) * KV_BLOCK * cfg.head_dim * 2


class DecoderEngine:
    """Runs the decoder program of one rank.  ``comm`` (optional) supplies the tensor-parallel collectives."""

    def __init__(self, weights: DecoderWeights, num_blocks: int, max_seqs: int, max_tokens: int,
                 max_blocks_per_seq: int, comm=None, device=None, use_graphs: bool = True, link=None,
                 carry: bool = False):
        """``carry``: every step also leaves the closing-norm hidden state of each of its token rows in ``carry_out``
        (what the model's multi-token-prediction layer reads).  An engine built over such a layer's own weights
        (``cfg.mtp_head``) reads ``carry_in`` beside its tokens and always exports its own closing state."""
        cfg = weights.cfg
        self.stage = weights.stage          # None, or this rank's layer range of a pipeline
        self.link = link                    # hand-off of the residual stream between stages
        if self.stage is not None and self.stage.count > 1:
            from .weights import UnsupportedOnDevice
            if link is None:
                raise ValueError("a pipeline stage needs a link to its neighbours")
            if comm is not None:
                raise UnsupportedOnDevice("pipeline stages are not themselves tensor-parallel groups")
        gaps = cfg.device_gaps()
        if gaps:
            from .weights import UnsupportedOnDevice
            raise UnsupportedOnDevice(f"{cfg.family}: the device program does not implement " + ", ".join(gaps))
        if (cfg.residual_scale != 1.0 or cfg.logit_scale != 1.0) and not getattr(weights, "_scales_folded", False):
            from .weights import fold_scales
            fold_scales(weights)
        self.cfg, self.w, self.comm = cfg, weights, comm
        self.device = torch.device(device if device is not None else weights.layers[0].wo.device)
        self.tp = weights.tp_world
        self.hq = cfg.n_heads // self.tp
        self.hkv = max(cfg.n_kv_heads // self.tp, 1)
        self.max_seqs, self.max_tokens, self.max_blocks = max_seqs, max_tokens, max_blocks_per_seq
        self.use_graphs = use_graphs
        self.tp_mode = "auto"   # "auto": one-shot all-reduce for small steps, reduce-scatter/all-gather above; "rs_ag"
        self.kv = KVPool(cfg, num_blocks, self.device, self.tp,
                         n_layers=sum(1 for i in range(len(weights.layers)) if cfg.mixer_of(weights.layer0 + i) == "attention") or 1)
        dev, i32 = self.device, torch.int32
        if comm is not None and getattr(comm, "fused", False):
            max_tokens = max(max_tokens, 128)  # padded rows of the fused tensor-parallel path
            self.max_tokens = max_tokens
        T, D, H = max_tokens, cfg.head_dim, cfg.hidden
        # ---- step inputs (written in place by the host, or by the advance kernel) ----
        self.tokens = torch.zeros(T, dtype=i32, device=dev)
        self.positions = torch.zeros(T, dtype=i32, device=dev)
        self.slots = torch.full((T,), -1, dtype=i32, device=dev)
        self.row_seq = torch.zeros(T, dtype=i32, device=dev)
        self.row_ctx = torch.zeros(T, dtype=i32, device=dev)
        self.block_tables = torch.zeros(max_seqs, max_blocks_per_seq, dtype=i32, device=dev)
        self.logit_idx = torch.zeros(max_seqs, dtype=torch.int64, device=dev)
        self.samp_params = torch.zeros(max_seqs, 4, dtype=torch.float32, device=dev)
        self.samp_topk = torch.zeros(max_seqs, dtype=i32, device=dev)
        self.samp_seeds = torch.zeros(max_seqs, dtype=i32, device=dev)
        # ---- activations ----
        bf = torch.bfloat16
        ffn_local = (cfg.moe_ffn if cfg.is_moe else cfg.ffn) // (1 if cfg.is_moe else self.tp)
        if cfg.is_moe and (cfg.first_dense_layers or cfg.dense_layers):      # leading dense layers of a routed model
            ffn_local = max(ffn_local, cfg.ffn)
        self.h = torch.zeros(T, H, dtype=bf, device=dev)
        self.x = torch.zeros(T, H, dtype=bf, device=dev)
        self.qkv = torch.zeros(T, (self.hq + 2 * self.hkv) * D, dtype=bf, device=dev)
        self.q = torch.zeros(T, self.hq * D, dtype=bf, device=dev)
        self.attn = torch.zeros(T, self.hq * D, dtype=bf, device=dev)
        self.act = torch.zeros(T, ffn_local, dtype=bf, device=dev)
        # split-K partial slices and split-KV scratch are only used by small steps (few tiles / few CTAs)
        self.max_splits = 8
        self.small_T = min(T, 256)
        self.partials = torch.zeros(self.max_splits, self.small_T, H, dtype=torch.float32, device=dev)
        self.hl = torch.zeros(max_seqs, H, dtype=bf, device=dev)
        self.xl = torch.zeros(max_seqs, H, dtype=bf, device=dev)
        self.logits = torch.zeros(max_seqs, cfg.vocab, dtype=torch.float32, device=dev)
        vl = cfg.vocab // self.tp
        if self.tp == 1:
            self.logits_local = self.logits
        else:
            rows = max(max_seqs, 128)
            self.logits_local = torch.zeros(rows, vl, dtype=torch.float32, device=dev)
            self.logits_sel = torch.zeros(max_seqs, vl, dtype=torch.float32, device=dev)
            self.logits_gather = torch.zeros(self.tp * max_seqs * vl, dtype=torch.float32, device=dev)
            G = K.argmax_groups(vl)
            self.argmax_part_local = torch.zeros(max_seqs * G * 3, dtype=torch.int32, device=dev)
            self.argmax_part_all = torch.zeros(self.tp * max_seqs * G * 3, dtype=torch.int32, device=dev)
        self.picked = torch.zeros(max_seqs, 2, dtype=i32, device=dev)
        self.logprobs = torch.zeros(max_seqs, dtype=torch.float32, device=dev)
        self.adj_idx = self.adj_val = self.guided_mask = None   # allocated on first use
        # tensor-core prefill attention: tiles cut on the host per step, rows they cover masked out of the per-row kernel
        # head_dim 256, latent attention, sink logits and ALiBi are served by the general attention kernel
        self.attn_general = cfg.head_dim not in (64, 128) or cfg.is_mla or cfg.attn_sinks or cfg.pos == "alibi"
        self.alibi = None
        if cfg.pos == "alibi":
            from ..tensor import alibi_slopes
            sl = alibi_slopes(cfg.n_heads, cfg.alibi_slopes, cfg.alibi_bias_max)
            self.alibi = torch.tensor(sl[weights.tp_rank * self.hq:(weights.tp_rank + 1) * self.hq], dtype=torch.float32, device=dev)
        self.flash_ok = cfg.head_dim == 128 and cfg.attn_softcap == 0
        self._flash_only = False      # set by bind: every row of the bound step is covered by a tile
        self.attn_tiles = torch.zeros(self._tile_slots(T, max_seqs), 4, dtype=i32, device=dev)
        self.row_ctx_simt = torch.zeros(T, dtype=i32, device=dev)
        pin = torch.cuda.is_available()
        self._h_tiles = torch.zeros(self.attn_tiles.shape, dtype=i32, pin_memory=pin)
        self._h_ctx_simt = torch.zeros(T, dtype=i32, pin_memory=pin)
        self.argmax_scratch = K.argmax_scratch(max_seqs, cfg.vocab, dev)
        self.attn_splits_max = 16
        ts = self.small_T
        self.attn_scratch = (torch.zeros(ts * self.hq * self.attn_splits_max * D, dtype=torch.float32, device=dev),
                             torch.zeros(ts * self.hq * self.attn_splits_max * 2, dtype=torch.float32, device=dev))
        import dataclasses as _dc
        cos, sin = rope_tables(_dc.replace(cfg, rope_dim=cfg.qk_rope_dim) if cfg.is_mla else cfg, cfg.max_position)
        self.cos, self.sin = cos.to(dev), sin.to(dev)
        self.cos_local = self.sin_local = self.cos_none = self.sin_none = None
        if cfg.rope_theta_local is not None:     # windowed layers rotate with their own base and no scaling
            import dataclasses
            from ..models.config import RopeScaling
            c2, s2 = rope_tables(dataclasses.replace(cfg, rope_theta=cfg.rope_theta_local, rope_scaling=RopeScaling()),
                                 cfg.max_position)
            self.cos_local, self.sin_local = c2.to(dev), s2.to(dev)
        if cfg.pos != "rope" or (cfg.rope_layers is not None and not all(cfg.rope_layers)):   # no position signal: the identity rotation
            self.cos_none, self.sin_none = torch.ones_like(self.cos), torch.zeros_like(self.sin)
        # attention layers own K/V pool entries; recurrent layers own state entries
        kinds = [cfg.mixer_of(weights.layer0 + i) for i in range(len(weights.layers))]
        self._kv_of = {i: n for n, i in enumerate(i for i, k in enumerate(kinds) if k == "attention")}
        if cfg.is_mla:
            dq = cfg.qk_nope_dim + cfg.qk_rope_dim
            self.mla_q = torch.zeros(T, cfg.n_heads * dq, dtype=bf, device=dev)
            self.mla_qa = torch.zeros(T, max(cfg.q_lora_rank, 8), dtype=bf, device=dev)
            self.mla_kva = torch.zeros(T, cfg.kv_lora_rank + cfg.qk_rope_dim, dtype=bf, device=dev)
            self.mla_ckv = torch.zeros(T, cfg.kv_lora_rank, dtype=bf, device=dev)
            self.mla_kvb = torch.zeros(T, cfg.n_heads * (cfg.qk_nope_dim + cfg.v_head_dim), dtype=bf, device=dev)
            if cfg.index_topk:
                # sparse attention indexer: its own key pool per attention layer, the step's indexer queries, raw keys and
                # head weights, one score per (row, visible position) and the kept positions of every row
                ni, Di = cfg.index_n_heads, cfg.index_head_dim
                self.idx_pool = torch.zeros(max(len(self._kv_of), 1), num_blocks, 16, Di, dtype=bf, device=dev)
                self.idx_q = torch.zeros(T, ni * Di, dtype=bf, device=dev)
                self.idx_kraw = torch.zeros(T, Di, dtype=bf, device=dev)
                self.idx_w = torch.zeros(T, (ni + 7) // 8 * 8, dtype=torch.float32, device=dev)
                self.idx_scores = torch.zeros(T, max_blocks_per_seq * 16, dtype=torch.float32, device=dev)
                self.idx_sel = torch.full((T, cfg.index_topk), -1, dtype=i32, device=dev)
        self._gdn_of = {i: n for n, i in enumerate(i for i, k in enumerate(kinds) if k == "gdn")}
        if self._gdn_of:
            nk, nv, Dg, Kc = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim, cfg.gdn_conv
            C = (2 * nk + nv) * Dg
            self.gdn_C, self.gdn_N = C, C + nv * Dg + 2 * nv
            self.gdn_in = torch.zeros(T, self.gdn_N, dtype=bf, device=dev)
            self.gdn_conv_out = torch.zeros(T, C, dtype=bf, device=dev)
            self.gdn_y = torch.zeros(T, nv * Dg, dtype=bf, device=dev)
            self.gdn_conv_state = torch.zeros(len(self._gdn_of), max_seqs, Kc - 1, C, dtype=torch.float32, device=dev)
            self.gdn_state = torch.zeros(len(self._gdn_of), max_seqs, nv, Dg, Dg, dtype=torch.float32, device=dev)
            # one segment per sequence piece of the step: (first row, rows, sequence row, first position); zero rows = unused
            self.seg_table = torch.zeros(max_seqs, 4, dtype=i32, device=dev)
            self._h_segs = torch.zeros(max_seqs, 4, dtype=i32, pin_memory=torch.cuda.is_available())
        self._ssm_of = {i: n for n, i in enumerate(i for i, k in enumerate(kinds) if k == "mamba")}
        if self._ssm_of:
            nhm, P, N, G, Kc = cfg.ssm_heads, cfg.ssm_head_dim, cfg.ssm_state, cfg.ssm_groups, cfg.ssm_conv
            I = nhm * P
            C = I + 2 * G * N
            self.ssm_I, self.ssm_C = I, C
            self.ssm_in = torch.zeros(T, -(-(I + C + nhm) // 8) * 8, dtype=bf, device=dev)
            self.ssm_conv_out = torch.zeros(T, C, dtype=bf, device=dev)
            self.ssm_y = torch.zeros(T, I, dtype=bf, device=dev)
            self.ssm_conv_state = torch.zeros(len(self._ssm_of), max_seqs, Kc - 1, C, dtype=torch.float32, device=dev)
            self.ssm_state = torch.zeros(len(self._ssm_of), max_seqs, nhm, N, P, dtype=torch.float32, device=dev)
            if not self._gdn_of:
                self.seg_table = torch.zeros(max_seqs, 4, dtype=i32, device=dev)
                self._h_segs = torch.zeros(max_seqs, 4, dtype=i32, pin_memory=torch.cuda.is_available())
        if cfg.attn_gate:
            self.gate = torch.zeros(T, self.hq * D, dtype=bf, device=dev)
        if not cfg.plain_block:
            if comm is not None:
                # the fused programs are written for the pre-norm SwiGLU rope layer; other attention stacks shard the
                # Megatron way over the library collectives.  Latent attention and recurrent mixers have no sharding rule
                # (crates/poot-graph-plan/src/passes/sharding.rs:86-96: ``NoRule``).
                from .weights import UnsupportedOnDevice
                if getattr(comm, "fused", False):
                    raise UnsupportedOnDevice(f"{cfg.family}: the fused tensor-parallel programs are built for the pre-norm "
                                              "SwiGLU rope layer only; shard this family over the library collectives")
                if cfg.is_mla or cfg.layer_kinds is not None or cfg.attn_gate:
                    raise UnsupportedOnDevice(f"{cfg.family}: no sharding rule for latent attention, gated attention or recurrent mixers")
            self.proj = torch.zeros(T, H, dtype=bf, device=dev)          # projection output waiting for its post norm
            if cfg.act != "silu":
                self.gu = torch.zeros(T, 2 * ffn_local, dtype=bf, device=dev)
            if cfg.qk_norm_wide:
                self.qn = torch.zeros(T, self.hq * D, dtype=bf, device=dev)
                self.kn = torch.zeros(T, self.hkv * D, dtype=bf, device=dev)
        self.scale = float(cfg.attn_scale) if cfg.attn_scale is not None else 1.0 / math.sqrt(D)
        if comm is not None:
            comm.attach(self)
        # Families whose layer the planner lowers completely run the compiled plan's launch list (runtime/program.py);
        # everything else keeps the hand-sequenced program below.
        self.program = None
        self.carry = bool(carry or cfg.mtp_head)
        self.carry_out = self.carry_in = None
        if self.carry:
            if comm is not None or (self.stage is not None and self.stage.count > 1):
                raise ValueError("the hidden-state carry is exported by the single-device engine")
            self.carry_out = torch.zeros(max_tokens, cfg.hidden, dtype=torch.bfloat16, device=self.device)
        if cfg.mtp_head:
            if getattr(weights, "mtp", None) is None:
                raise ValueError("weights of a multi-token-prediction layer carry its input norms and projection")
            H_ = cfg.hidden
            self.carry_in = torch.zeros(max_tokens, H_, dtype=torch.bfloat16, device=self.device)
            self.mtp_e = torch.zeros(max_tokens, H_, dtype=torch.bfloat16, device=self.device)
            self.mtp_c = torch.zeros(max_tokens, H_, dtype=torch.bfloat16, device=self.device)
            self.mtp_zero = torch.zeros(max_tokens, H_, dtype=torch.bfloat16, device=self.device)
            self.mtp_first = torch.zeros(max_tokens, dtype=torch.int32, device=self.device)   # 1 = absolute position 0
        from .program import ProgramExecutor
        if not self.carry:
            self.program = ProgramExecutor.build_for(self)
        self.lora = None                    # bank of resident adapters, created by enable_adapters()
        self.embed_rows = self.embed_flags = None   # staging of rows that replace embeddings, created by bind_embeds()
        self.rope_cos_tok = self.rope_sin_tok = None  # per-token rotary rows of a sectioned rope, created by bind_rope_streams()
        self._stage: Optional[str] = None    # "body" / "suffix" while one stage of a cut step is launched (run_late)
        self._suffix_in: Dict[Tuple, torch.Tensor] = {}     # the logits view each cut shape's suffix reads
        self._graphs: Dict[Tuple, torch.cuda.CUDAGraph] = {}
        self.launches_per_step: Dict[Tuple, int] = {}
        self._launch_counter = 0

    def bind_embeds(self, flags: torch.Tensor, rows: torch.Tensor) -> None:
        """Stage the rows that replace token embeddings in the next step: ``flags[T]`` int32 (1 = replace) and
        ``rows[T, hidden]`` (any float dtype; rows without a flag are ignored).  The buffers have fixed addresses, so a
        captured step graph replays over them."""
        if getattr(self.comm, "fused", False) or (self.stage is not None and not self.stage.first):
            raise ValueError("rows in place of embeddings: not in the fused tensor-parallel programs, and on the first "
                             "pipeline stage only")
        if self.embed_rows is None:
            self.embed_rows = torch.zeros(self.max_tokens, self.cfg.hidden, dtype=torch.bfloat16, device=self.device)
            self.embed_flags = torch.zeros(self.max_tokens, dtype=torch.int32, device=self.device)
        T = flags.numel()
        self.embed_flags[:T].copy_(flags, non_blocking=True)
        self.embed_rows[:T].copy_(rows, non_blocking=True)

    def bind_carry(self, rows: torch.Tensor, positions: torch.Tensor) -> None:
        """Stage the hidden-state carry of the next step of a multi-token-prediction layer: ``rows[T, hidden]`` (any
        float dtype) and the step's positions (the embedding at absolute position 0 is zeroed)."""
        if self.carry_in is None:
            raise ValueError("this engine is not a multi-token-prediction layer")
        T = rows.shape[0]
        self.carry_in[:T].copy_(rows, non_blocking=True)
        self.mtp_first[:T].copy_((positions[:T] == 0).to(torch.int32), non_blocking=True)

    def bind_rope_streams(self, streams: torch.Tensor) -> None:
        """Stage the rotary rows of the next step under a sectioned rope: ``streams[3, T]`` int32 are the (time, row,
        column) positions of every token; channel pair ``j`` of a token's row is read from the table at the position of
        the stream that owns ``j``.  The rows land in fixed buffers indexed by the token's place in the step, so the
        rotary kernel reads them with positions ``0..T-1`` and a captured step graph replays over them."""
        cfg = self.cfg
        if not cfg.mrope_sections:
            raise ValueError(f"{cfg.family}: rotary position streams need a sectioned rope")
        if getattr(self.comm, "fused", False):
            raise ValueError("rotary position streams are not read by the fused tensor-parallel programs")
        half = cfg.rot // 2
        if self.rope_cos_tok is None:
            dev = self.device
            self.rope_cos_tok = torch.zeros(self.max_tokens, half, dtype=torch.float32, device=dev)
            self.rope_sin_tok = torch.zeros(self.max_tokens, half, dtype=torch.float32, device=dev)
            self.rope_iota = torch.arange(self.max_tokens, dtype=torch.int32, device=dev)
            owner = [i % 3 for i, n in enumerate(cfg.mrope_sections) for _ in range(n)]
            if len(owner) != half:
                raise ValueError(f"mrope sections {cfg.mrope_sections} do not cover {half} channel pairs")
            self._rope_owner = torch.tensor(owner, dtype=torch.long, device=dev).view(1, 1, half)
        T = streams.shape[1]
        idx = streams.to(device=self.device, dtype=torch.long)                       # [3, T]
        own = self._rope_owner.expand(1, T, half)
        self.rope_cos_tok[:T].copy_(self.cos[idx].gather(0, own)[0])
        self.rope_sin_tok[:T].copy_(self.sin[idx].gather(0, own)[0])

    def enable_adapters(self, slots: int = 8, max_rank: int = 64):
        """Create the bank of resident LoRA adapters (per-row selection); see ``runtime/lora_bank.py``."""
        from .lora_bank import LoraBank, LoraBankError
        if self.comm is not None or (self.stage is not None and self.stage.count > 1):
            raise LoraBankError("per-row adapters are built for the single-device engine")
        if isinstance(self.w.layers[0].wqkv, K.QuantWeight):
            raise LoraBankError("per-row adapters need bf16 projections")
        self.lora = LoraBank(self.cfg, len(self.w.layers), slots, max_rank, self.max_tokens, self.device)
        if getattr(self, "gu", None) is None:
            ffn_local = self.cfg.ffn // self.tp
            self.gu = torch.zeros(self.max_tokens, 2 * ffn_local, dtype=torch.bfloat16, device=self.device)
        if getattr(self, "proj", None) is None:
            self.proj = torch.zeros(self.max_tokens, self.cfg.hidden, dtype=torch.bfloat16, device=self.device)
        return self.lora

    # ------------------------------------------------------------------ kernel program
    def host_embedding(self) -> int:
        """Keep the token-embedding table in host memory.  A table that only a row gather reads never needs to be a
        device buffer: a step needs ``T`` of its rows, never the table.  The table moves to pinned host memory; ``bind``
        - which knows the step's token ids on the host - copies the *stored* bytes of the rows the step gathers into a
        small device slot (a packed table's rows stay packed: they are decoded by the same row-gather kernel, over the
        slot), and the step's embed launch reads row ``t`` of the slot for token ``t``.  Returns the device bytes freed.
        Refused for a table that is also the output head (it has a second reader), for a tensor-parallel rank and for
        chained decode, whose tokens never visit the host.  The reference's hosted gather sites:
        crates/poot-graph-plan/src/passes/hosted_gather.rs:1-8."""
        w = self.w
        if w.embed is None or w.lm_head is w.embed:
            raise ValueError("the embedding table is also the output head: not a gather-only table")
        if self.comm is not None or (self.stage is not None and self.stage.count > 1):
            raise ValueError("hosted embedding rows are built for the single-device engine")
        pin = self.device.type == "cuda"
        T = self.max_tokens
        if isinstance(w.embed, K.QuantWeight):
            q = w.embed
            row_bytes = q.packed.numel() // q.N
            host = q.packed.view(q.N, row_bytes).cpu()
            slot = torch.zeros(T, row_bytes, dtype=torch.uint8, device=self.device)
            freed = q.packed.numel()
            w.embed = K.QuantWeight(q.fmt, slot.view(-1), T, q.K) if self.device.type == "cuda" else q
            self._hosted = {"table": host.pin_memory() if pin else host, "slot": slot, "packed": True,
                            "stage": torch.zeros(T, row_bytes, dtype=torch.uint8, pin_memory=pin)}
        else:
            host = w.embed.cpu()
            freed = w.embed.numel() * w.embed.element_size()
            slot = torch.zeros(T, host.shape[1], dtype=host.dtype, device=self.device)
            w.embed = slot
            self._hosted = {"table": host.pin_memory() if pin else host, "slot": slot, "packed": False,
                            "stage": torch.zeros(T, host.shape[1], dtype=host.dtype, pin_memory=pin)}
        self.embed_iota = torch.arange(T, dtype=torch.int32, device=self.device)
        self._graphs.clear()
        return freed

    def _embed_ids(self, T: int, lo: int = 0) -> torch.Tensor:
        """Row ids of the embed launch: the step's tokens, or 0..T-1 over the hosted slot."""
        if getattr(self, "_hosted", None) is not None:
            return self.embed_iota[lo:lo + T]
        return self.tokens[lo:lo + T]

    def enable_expert_pool(self, slots: int, manager) -> None:
        """Pooled experts: ``slots`` resident experts per routed layer, the rest in pinned host memory (runtime/moe.py)."""
        from .moe import enable_expert_pool
        enable_expert_pool(self, slots, manager)
        self._graphs.clear()

    def _count(self, n: int = 1):
        self._launch_counter += n

    def _linear(self, x, W, epi, out, resid=None):
        self._count()
        return K.linear(x, W, epi, out, resid)

    def _proj_to_residual(self, x, W, T, h=None, out=None):
        """``out = h + x @ W^T`` (o_proj / down_proj; in place on the residual stream ``self.h`` by default).  Returns
        pending fp32 partial slices (the caller's next norm adds them to ``h``) or None.

        Small-N, large-K projections at decode batch sizes do not fill 148 SMs with one K pass, so they split K
        and leave the reduction to the next RMSNorm (which reads the residual stream anyway).
        """
        h = self.h[:T] if h is None else h
        out = h if out is None else out
        N, Kdim = W.shape
        if T <= 128 or isinstance(W, K.QuantWeight):
            self._linear(x, W, K.EPI_RESID, out, h)
            return None
        tiles =((T + 127) // 128) * ((N + 63) // 64)
        if tiles < 100 and Kdim >= 1024 and T <= self.small_T:
            splits = max(1, min(self.max_splits, 148 // tiles, Kdim // 512))
            if splits > 1:
                p = self.partials[:splits, :T]
                self._count()
                K.gemm(x, W, K.EPI_PARTIAL, out=p, bn=64, splits=splits)
                return p
        self._linear(x, W, K.EPI_RESID, out, h)
        return None

    def _norm(self, w, T, pending, bias=None):
        h, x = self.h[:T], self.x[:T]
        self._count()
        if self.cfg.norm_kind == "layer":
            if pending is not None:
                self._count()
                K.reduce_partials(h, pending, h)
            K.layernorm(h, w, bias, self.cfg.norm_eps, out=x)
            return x
        if pending is None:
            K.rmsnorm(h, w, self.cfg.norm_eps, out=x)
        else:
            K.rmsnorm(h, w, self.cfg.norm_eps, out=x, partials=pending, h_out=h)
        return x

    def _attention(self, l: int, R: int, T: int, B: int, count: bool = True, q=None, out=None) -> None:
        """Attention of the step's ``R`` rows (``T`` of them live) into ``self.attn``.

        Steps that carry prefill pieces (more tokens than sampling rows) run two kernels: the per-row paged kernel
        over the rows left to it (its context length is 0 on rows the tiles cover) and the tensor-core flash kernel
        over the tiles ``bind`` cut from the step's segments.  Pure decode steps run the per-row kernel alone."""
        cfg, D = self.cfg, self.cfg.head_dim
        q = self.q[:R] if q is None else q
        out = self.attn[:R] if out is None else out
        if self.attn_general:
            # head widths the tuned kernels do not serve: the general kernel over every live row
            if count:
                self._count()
            K.attn_general(q, self.kv.k(self._kv_of[l]), self.kv.v(self._kv_of[l]), self.block_tables, self.row_seq[:R],
                           self.row_ctx[:R], self.hq, self.hkv, D, D, self.scale, out, softcap=cfg.attn_softcap,
                           window=cfg.window_of(self.w.layer0 + l), alibi=self.alibi, sinks=self.w.layers[l].sinks)
            return
        flash = self.flash_ok and T > B
        splits = self._attn_splits(R)
        simt = not (flash and self._flash_only)      # every row sits in a tile: the per-row kernel has nothing to do
        if count:
            self._count(((2 if splits > 1 else 1) if simt else 0) + (1 if flash else 0))
        if simt:
            K.attn_paged(q, self.kv.k(self._kv_of[l]), self.kv.v(self._kv_of[l]), self.block_tables, self.row_seq[:R],
                         (self.row_ctx_simt if flash else self.row_ctx)[:R], self.hq, self.hkv, D, self.scale,
                         out=out, splits=splits, scratch=self.attn_scratch, softcap=cfg.attn_softcap,
                         window=cfg.window_of(self.w.layer0 + l))
        if flash:
            K.attn_flash_prefill(q, self.kv.k(self._kv_of[l]), self.kv.v(self._kv_of[l]), self.block_tables,
                                 self.attn_tiles[:self._tile_slots(T, B)], self.hq, self.hkv, self.scale,
                                 out=out, window=cfg.window_of(self.w.layer0 + l))

    def _tile_slots(self, T: int, B: int) -> int:
        """Tile slots a (T, B) step can need: full tiles plus one ragged tile per sequence."""
        return (T + 127) // 128 + B

    def _attn_splits(self, T: int) -> int:
        ctas = T * self.hkv * max(1, (self.cfg.n_rep + 3) // 4)
        if ctas >= 148 or T > self.small_T:
            return 1
        return max(1, min(self.attn_splits_max, 296 // ctas))

    def _fused_shape(self, shape: StepShape) -> bool:
        """Whether this step runs one of the fused tensor-parallel programs (kernels that wait on other ranks).

        A step is either fused or it rides the library collectives, never both: a fused step's graph holds no library
        collective (the greedy pick is exchanged through the symmetric block), and a step that needs the full logits on
        every rank (sampling rules, logit adjustments, log-probabilities) takes the library path as a whole."""
        cfg, w, comm = self.cfg, self.w, self.comm
        if comm is None or not getattr(comm, "fused", False):
            return False
        if shape.sampler != 0 or shape.adjust or shape.logprobs:
            return False
        if isinstance(w.layers[0].wqkv, K.QuantWeight) or isinstance(w.layers[0].wo, K.QuantWeight):
            return False
        T = shape.tokens
        if cfg.is_moe:
            # expert parallelism rides the one-shot path: the experts' combine is the fused all-reduce (one expert per
            # rank pushes from its GEMM epilogue, several per rank from the combine kernel)
            fusable = w.ep_world == self.tp and w.layers[0].ex_wgu is not None
            if fusable and self.tp_mode == "rs_ag" and getattr(comm, "ep_cap", 0) and w.layers[0].sh_wgu is None:
                return bool(comm.rows_for(T))        # token-sharded stream: experts reached by dispatch / combine exchanges
            return bool(fusable and comm.oneshot_ok(T))
        if comm.oneshot_ok(T) and self.tp_mode != "rs_ag":
            return True
        return bool(comm.rows_for(T))

    def forward(self, shape: StepShape) -> None:
        """Launch the whole step on the current stream (eagerly or under capture)."""
        cfg, w = self.cfg, self.w
        T, B, D = shape.tokens, shape.logit_rows, cfg.head_dim
        if self._stage == "suffix":             # second stage of a step cut at its late-input point: the sampler suffix only
            self._launch_counter = 0
            return self._sample(shape, self._suffix_in[self._key(shape)])
        self._fused_step = False
        if shape.chain and getattr(self, "_hosted", None) is not None:
            raise ValueError("chained decode feeds tokens back on the device; hosted embedding rows are copied from the host")
        if self.program is not None and self.program.accepts(shape):
            return self.program.run(shape)      # the plain decoder layer: a walk over the compiled plan's launch list
        if self._fused_shape(shape):
            self._fused_step = True
            if self.comm.oneshot_ok(T) and (self.tp_mode != "rs_ag" or (cfg.is_moe and not getattr(self.comm, "ep_cap", 0))):
                return self._forward_tp_oneshot(shape)
            return self._forward_tp_fused(shape, self.comm.rows_for(T))
        self._launch_counter = 0
        h = self.h[:T]
        staged = self.stage is not None and self.stage.count > 1
        if staged and shape.chain:
            raise ValueError("chained decode feeds tokens back on one device; a pipeline's sampler and embedding are on different stages")
        if staged and not self.stage.first:
            self.link.recv_hidden(h)             # the residual stream as the previous stage left it
        else:
            self._count()
            if isinstance(w.embed, K.QuantWeight):
                K.quant_row_gather(self._embed_ids(T), w.embed, out=h)
            else:
                K.embed_gather(self._embed_ids(T), w.embed, out=h)
            if cfg.embed_scale != 1.0:
                K.scale_(h, cfg.embed_scale)
            if shape.embeds:
                self._count()
                K.replace_rows_(h, self.embed_rows[:T], self.embed_flags[:T])
            if w.embed_norm is not None:
                self._count()
                K.layernorm(h, w.embed_norm, w.embed_norm_b, cfg.norm_eps, out=h)
            if cfg.mtp_head:
                # h = eh_proj . [enorm(embedding of the token after the position, zero at position 0) ; hnorm(carry)],
                # as two projections over the halves of eh_proj, the second accumulating onto the first
                m = w.mtp
                self._count(3)
                K.replace_rows_(h, self.mtp_zero[:T], self.mtp_first[:T])
                K.rmsnorm(h, m["enorm"], cfg.norm_eps, out=self.mtp_e[:T])
                K.rmsnorm(self.carry_in[:T], m["hnorm"], cfg.norm_eps, out=self.mtp_c[:T])
                self._linear(self.mtp_e[:T], m["we"], K.EPI_STORE, h)
                self._linear(self.mtp_c[:T], m["wh"], K.EPI_RESID, h, h)
        pending = None
        lora = shape.lora and self.lora is not None
        post = cfg.block != "pre"           # a norm sits between each projection and its residual add
        for l, L in enumerate(w.layers):
            if cfg.layer_ffn is not None:       # blocks of one mixer each (a token mixer OR an FFN), each behind its own norm
                pending = self._single_mixer_block(l, L, T, B, pending)
                continue
            x = h if cfg.block == "post" else self._norm(L.ln1, T, pending, L.ln1_b)
            if L.kind == "mla":
                pending = self._mla_mixer(l, L, x, T)
                x = self._norm(L.ln2, T, pending)
                if cfg.moe_layer(w.layer0 + l):
                    pending = self._moe(l, L, x, T)
                else:
                    act = self._linear(x, L.wgu, K.EPI_SWIGLU, self.act[:T])
                    pending = self._proj_to_residual(act, L.wdown, T)
                continue
            if L.kind == "gdn":
                pending = self._gdn_mixer(l, L, x, T)
                x = self._norm(L.ln2, T, pending)
                if cfg.moe_layer(w.layer0 + l):
                    pending = self._moe(l, L, x, T)
                else:
                    act = self._linear(x, L.wgu, K.EPI_SWIGLU, self.act[:T])
                    pending = self._proj_to_residual(act, L.wdown, T)
                continue
            qkv = self._linear(x, L.wqkv, K.EPI_STORE, self.qkv[:T])
            if L.bqkv is not None:
                K.bias_add_(qkv, L.bqkv)
            if lora:
                self.lora.apply(self, "qkv", l, x, qkv, T)
            qn, kn = L.q_norm, L.k_norm
            if cfg.qk_norm_wide:            # one norm over the whole q / k projection: done here, not per head in the rope kernel
                self._wide_qk_norm(qkv, L, T)
                qn = kn = None
            cos, sin = self._rope_tables_of(w.layer0 + l)
            rope_at = self.positions[:T]
            if shape.mrope:                     # rows assembled per token by bind_rope_streams: row t is token t's
                cos, sin, rope_at = self.rope_cos_tok, self.rope_sin_tok, self.rope_iota[:T]
            self._count()
            kvl = self._kv_of[l]
            K.rope_kv_write(qkv, self.q[:T], self.kv.k(kvl), self.kv.v(kvl), rope_at, self.slots[:T],
                            cos, sin, self.hq, self.hkv, D, cfg.rot, qn, kn, cfg.norm_eps)
            self._attention(l, T, T, B)
            if L.wgate is not None:             # gated attention: the output is scaled by sigmoid of a projection of the layer input
                gate = self._linear(x, L.wgate, K.EPI_STORE, self.gate[:T])
                self._count()
                K.sigmoid_mul(self.attn[:T], gate)
            if post:
                self._proj_post_norm(self.attn[:T], L.wo, L.post1, T, ("o", l) if lora else None)
            elif self.comm is not None:
                pending = self.comm.row_parallel(self, self.attn[:T], L.wo, T)
                if L.bo is not None:            # the bias joins the reduced sum once
                    K.bias_add_(h, L.bo)
            else:
                pending = self._proj_to_residual(self.attn[:T], L.wo, T)
                if lora:
                    self.lora.apply(self, "o", l, self.attn[:T], h, T)
                if L.bo is not None:
                    K.bias_add_(h, L.bo)
            x = h if cfg.block == "post" else self._norm(L.ln2, T, pending, L.ln2_b)
            if cfg.moe_layer(w.layer0 + l):
                pending = self._moe(l, L, x, T)
            elif not cfg.gated_ffn:             # down(act(up(x) + b) ) + b: no gate
                up = self._linear(x, L.wgu, K.EPI_STORE, self.act[:T])
                if L.bgu is not None:
                    K.bias_add_(up, L.bgu)
                self._count()
                K.act_(up, cfg.act)
                pending = (self.comm.row_parallel(self, up, L.wdown, T) if self.comm is not None
                           else self._proj_to_residual(up, L.wdown, T))
                if L.bdown is not None:
                    K.bias_add_(h, L.bdown)
            else:
                if cfg.act == "silu" and not lora:
                    act = self._linear(x, L.wgu, K.EPI_SWIGLU, self.act[:T])
                else:                       # plain projection (+ adapter term), then the gated activation over (gate, up) pairs
                    gu = self._linear(x, L.wgu, K.EPI_STORE, self.gu[:T])
                    if lora:
                        self.lora.apply(self, "gu", l, x, gu, T)
                    self._count()
                    act = K.gated_act(gu, True, cfg.act, out=self.act[:T])
                if post:
                    self._proj_post_norm(act, L.wdown, L.post2, T, ("down", l) if lora else None)
                elif self.comm is not None:
                    pending = self.comm.row_parallel(self, act, L.wdown, T)
                else:
                    pending = self._proj_to_residual(act, L.wdown, T)
                    if lora:
                        self.lora.apply(self, "down", l, act, h, T)
        if pending is not None:
            self._count()
            K.reduce_partials(h, pending, h)
        if staged and not self.stage.last:
            self.link.send_hidden(h)
            if self.stage.first:                 # the driver's rank: wait for the last stage's sampled tokens
                self.link.return_picked(self.picked[:B], self.logprobs[:B] if shape.logprobs else None)
            return
        xl = self.xl[:B]
        if self.carry:
            # the closing norm runs over every token row (the carry), the logit rows are gathered from its output
            self._count()
            if cfg.norm_kind == "layer":
                K.layernorm(h, w.final_norm, w.final_norm_b, cfg.norm_eps, out=self.carry_out[:T])
            else:
                K.rmsnorm(h, w.final_norm, cfg.norm_eps, out=self.carry_out[:T])
            if B == T:
                xl = self.carry_out[:T]
            else:
                self._count()
                K.gather_rows(self.carry_out[:T], self.logit_idx[:B], xl)
        else:
            hl = self.hl[:B]
            if B == T:
                hl = h
            else:
                self._count()
                K.gather_rows(h, self.logit_idx[:B], hl)
            self._count()
            if cfg.norm_kind == "layer":
                K.layernorm(hl, w.final_norm, w.final_norm_b, cfg.norm_eps, out=xl)
            else:
                K.rmsnorm(hl, w.final_norm, cfg.norm_eps, out=xl)
        self._linear(xl, w.lm_head, K.EPI_F32, self.logits_local[:B])
        if cfg.final_softcap > 0:
            self._count()
            K.softcap_(self.logits_local[:B], cfg.final_softcap)
        self._sample(shape, self.logits_local[:B])
        if staged:
            self.link.return_picked(self.picked[:B], self.logprobs[:B] if shape.logprobs else None)

    def _single_mixer_block(self, l: int, L, T: int, B: int, pending):
        """One block of a stack whose blocks hold a single mixer (nemotron-h): Mamba2, plain attention, a dense FFN or
        routed experts, always as ``h += mixer(norm(h))``."""
        cfg, w, D = self.cfg, self.w, self.cfg.head_dim
        if L.kind == "mamba":
            pending = self._mamba_mixer(l, L, self._norm(L.ln1, T, pending), T)
        elif L.kind == "attention":
            x = self._norm(L.ln1, T, pending)
            qkv = self._linear(x, L.wqkv, K.EPI_STORE, self.qkv[:T])
            cos, sin = self._rope_tables_of(w.layer0 + l)
            kvl = self._kv_of[l]
            self._count()
            K.rope_kv_write(qkv, self.q[:T], self.kv.k(kvl), self.kv.v(kvl), self.positions[:T], self.slots[:T], cos, sin,
                            self.hq, self.hkv, D, cfg.rot, None, None, cfg.norm_eps)
            self._attention(l, T, T, B)
            pending = self._proj_to_residual(self.attn[:T], L.wo, T)
        if cfg.has_ffn(w.layer0 + l):
            x = self._norm(L.ln2, T, pending)
            if cfg.moe_layer(w.layer0 + l):
                pending = self._moe(l, L, x, T)
            else:
                up = self._linear(x, L.wgu, K.EPI_STORE, self.act[:T])
                if L.bgu is not None:
                    K.bias_add_(up, L.bgu)
                self._count()
                K.act_(up, cfg.act)
                pending = (self.comm.row_parallel(self, up, L.wdown, T) if self.comm is not None
                           else self._proj_to_residual(up, L.wdown, T))
                if L.bdown is not None:
                    K.bias_add_(self.h[:T], L.bdown)
        return pending

    def _mamba_mixer(self, l: int, L, x, T: int):
        """Mamba2 layer (components/mamba2.rs): one GEMM for z | (x | B | C) | dt, causal conv + SiLU continuing each
        sequence's window, the selective state-space recurrence over each sequence's state, the gated RMSNorm within
        channel groups, out-projection into the residual stream."""
        cfg, si = self.cfg, self._ssm_of[l]
        I, C = self.ssm_I, self.ssm_C
        proj = self._linear(x, L.wqkv, K.EPI_STORE, self.ssm_in[:T])
        self._count(3)
        K.causal_conv_silu(proj, I, C, L.ssm["conv"], self.ssm_conv_state[si], self.seg_table, self.ssm_conv_out[:T],
                           bias=L.ssm["conv_bias"])
        K.ssd_scan(self.ssm_conv_out[:T], proj, I + C, L.ssm["dt_bias"], L.ssm["a_log"], L.ssm["d"], self.ssm_state[si],
                   self.seg_table, self.ssm_y[:T], cfg.ssm_heads, cfg.ssm_groups, cfg.ssm_state, cfg.ssm_head_dim)
        G = cfg.ssm_groups
        K.gated_rmsnorm(self.ssm_y[:T], proj, 0, L.ssm["gate_norm"], cfg.norm_eps, self.ssm_y[:T], G, I // G, gate_first=True)
        return self._proj_to_residual(self.ssm_y[:T], L.wo, T)

    def _mla_mixer(self, l: int, L, x, T: int):
        """Multi-head latent attention in its expanded form (components/mla.rs): low-rank query and key/value
        projections with their norms, the rotary on the rotary parts only, keys ``[no-position | shared rotary]`` and
        values written to the paged pools, attention with key width ``dn + dr`` and value width ``dv``, out-projection."""
        cfg, m = self.cfg, L.mla
        nh, dn, dr, dv = cfg.n_heads, cfg.qk_nope_dim, cfg.qk_rope_dim, cfg.v_head_dim
        if "q_a" in m:
            qa = self._linear(x, m["q_a"], K.EPI_STORE, self.mla_qa[:T, :cfg.q_lora_rank])
            self._count()
            K.rmsnorm(qa, m["q_a_norm"], cfg.mla_eps, out=qa)
            q = self._linear(qa, m["q_b"], K.EPI_STORE, self.q[:T])
        else:
            q = self._linear(x, m["q"], K.EPI_STORE, self.q[:T])
        kva = self._linear(x, m["kv_a"], K.EPI_STORE, self.mla_kva[:T])
        ckv = self.mla_ckv[:T]
        ckv.copy_(kva[:, :cfg.kv_lora_rank])
        self._count(3)
        K.rmsnorm(ckv, m["kv_a_norm"], cfg.mla_eps, out=ckv)
        kvb = self._linear(ckv, m["kv_b"], K.EPI_STORE, self.mla_kvb[:T])
        kvl = self._kv_of[l]
        K.mla_qkv_write(q, kvb, kva, cfg.kv_lora_rank, self.mla_q[:T], self.kv.k(kvl), self.kv.v(kvl), self.positions[:T],
                        self.slots[:T], self.cos, self.sin, nh, dn, dr, dv)
        attn = self.attn[:T, :nh * dv]
        sel = self._index_select(kvl, m, x, qa, T) if cfg.index_topk else None
        K.attn_general(self.mla_q[:T], self.kv.k(kvl), self.kv.v(kvl), self.block_tables, self.row_seq[:T], self.row_ctx[:T],
                       nh, nh, dn + dr, dv, self.scale, attn, window=cfg.window_of(self.w.layer0 + l), sel=sel)
        return self._proj_to_residual(attn, L.wo, T)

    def _index_select(self, kvl: int, m, x, qa, T: int):
        """Sparse attention indexer (components/dsa.rs): score every visible key of every row with the light multi-head
        scorer over the layer's index pool and keep each row's ``index_topk`` best; the result is the selection list
        the attention kernel walks."""
        cfg = self.cfg
        ni, Di, dr = cfg.index_n_heads, cfg.index_head_dim, cfg.qk_rope_dim
        iq = self._linear(qa, m["idx_q"], K.EPI_STORE, self.idx_q[:T])
        kraw = self._linear(x, m["idx_k"], K.EPI_STORE, self.idx_kraw[:T])
        w = self._linear(x, m["idx_w"], K.EPI_F32, self.idx_w[:T])
        self._count(4)
        K.index_q_rope(iq, self.positions[:T], self.cos, self.sin, ni, Di, dr)
        K.index_k_write(kraw, m["idx_k_norm"], m["idx_k_norm_bias"], 1e-6, self.positions[:T], self.slots[:T], self.cos,
                        self.sin, self.idx_pool[kvl], dr)
        K.index_scores(iq, w, self.idx_pool[kvl], self.block_tables, self.row_seq[:T], self.row_ctx[:T], self.idx_scores[:T],
                       ni, Di, self.idx_scores.shape[1], Di ** -0.5)
        return K.index_select(self.idx_scores[:T], self.row_ctx[:T], self.idx_sel[:T])

    def _gdn_mixer(self, l: int, L, x, T: int):
        """Gated delta net layer (components/gdn.rs): one GEMM for q | k | v | z | b | a, causal conv + SiLU over
        (q | k | v) continuing each sequence's conv window, the gated delta rule over each sequence's state matrices,
        RMSNorm gated by SiLU(z), out-projection into the residual stream."""
        cfg, gi = self.cfg, self._gdn_of[l]
        nk, nv, Dg = cfg.gdn_k_heads, cfg.gdn_v_heads, cfg.gdn_head_dim
        C = self.gdn_C
        proj = self._linear(x, L.wqkv, K.EPI_STORE, self.gdn_in[:T])
        self._count(3)
        K.causal_conv_silu(proj, 0, C, L.gdn["conv"], self.gdn_conv_state[gi], self.seg_table, self.gdn_conv_out[:T])
        K.gdn_scan(self.gdn_conv_out[:T], proj, C + nv * Dg, C + nv * Dg + nv, L.gdn["dt_bias"], L.gdn["a_log"],
                   self.gdn_state[gi], self.seg_table, self.gdn_y[:T], nk, nv, Dg)
        K.gated_rmsnorm(self.gdn_y[:T], proj, C, L.gdn["gate_norm"], cfg.norm_eps, self.gdn_y[:T], nv, Dg)
        return self._proj_to_residual(self.gdn_y[:T], L.wo, T)

    def _rope_tables_of(self, l: int):
        cfg = self.cfg
        if self.cos_none is not None and (cfg.pos != "rope" or not cfg.rope_layers[l]):
            return self.cos_none, self.sin_none
        if self.cos_local is not None and cfg.window_of(l) > 0:
            return self.cos_local, self.sin_local
        return self.cos, self.sin

    def _proj_post_norm(self, x, W, norm_w, T: int, adapter_site=None) -> None:
        """``h += rmsnorm(x @ W^T) * norm_w`` (post-norm and sandwich blocks): projection, norm, residual add."""
        h, p = self.h[:T], self.proj[:T]
        self._linear(x, W, K.EPI_STORE, p)
        if adapter_site is not None:
            self.lora.apply(self, adapter_site[0], adapter_site[1], x, p, T)
        if self.comm is not None:                # a row-parallel projection: the norm needs the sum over the ranks
            self.comm.all_reduce(p)
        self._count(2)
        K.rmsnorm(p, norm_w, self.cfg.norm_eps, out=p)
        K.add(h, p, out=h)

    def _wide_qk_norm(self, qkv, L, T: int) -> None:
        """RMSNorm over the whole q projection and over the whole k projection of the fused qkv rows."""
        nq, nk = self.hq * self.cfg.head_dim, self.hkv * self.cfg.head_dim
        qn, kn = self.qn[:T], self.kn[:T]
        qn.copy_(qkv[:, :nq])
        kn.copy_(qkv[:, nq:nq + nk])
        if self.comm is not None:
            # the norm spans the heads of every rank: mean squares are summed over the ranks, then each rank scales
            # its own channels (library-collective path; plain tensor arithmetic, two small all-reduces per layer)
            for t, wt, width in ((qn, L.q_norm, nq * self.tp), (kn, L.k_norm, nk * self.tp)):
                ss = t.float().pow(2).sum(-1, keepdim=True)
                self.comm.all_reduce(ss)
                t.copy_((t.float() * torch.rsqrt(ss / width + self.cfg.norm_eps) * wt.float()).to(t.dtype))
            qkv[:, :nq].copy_(qn)
            qkv[:, nq:nq + nk].copy_(kn)
            return
        self._count(6)
        K.rmsnorm(qn, L.q_norm, self.cfg.norm_eps, out=qn)
        K.rmsnorm(kn, L.k_norm, self.cfg.norm_eps, out=kn)
        qkv[:, :nq].copy_(qn)
        qkv[:, nq:nq + nk].copy_(kn)

    def _sample(self, shape: StepShape, local_logits: torch.Tensor) -> None:
        """Sampler suffix over (possibly vocabulary-sharded) logits; every rank ends with the same ``picked``."""
        B, V = shape.logit_rows, self.cfg.vocab
        self.last_local_logits = local_logits  # [B, vocab / tp] of the step just launched
        if self._stage == "body":               # first stage of a cut step: everything up to the logits
            self._suffix_in[self._key(shape)] = local_logits
            return
        need_full = shape.sampler != 0 or shape.adjust or shape.logprobs
        logits = None
        if self.tp == 1:
            logits = local_logits
        else:
            vl = V // self.tp
            if not need_full:
                # greedy: exchange the stage-1 partial tables (a few KB), not the logits
                G = K.argmax_groups(vl)
                part = self.argmax_part_local[:B * G * 3].view(B, G, 3)
                self._count()
                K.argmax_partials(local_logits, self.w.tp_rank * vl, V, part)
                if getattr(self, "_fused_step", False):
                    self._count()
                    self.comm.argmax_exchange(part, B, G, V, self.picked[:B])
                else:
                    allp = self.argmax_part_all[:self.tp * B * G * 3].view(self.tp, B, G, 3)
                    self.comm.all_gather(allp, part)
                    self._count()
                    K.argmax_combine(allp, B, G, V, self.picked[:B])
            else:
                gathered = self.logits_gather[:self.tp * B * vl].view(self.tp, B, vl)
                self.comm.all_gather(gathered, local_logits.contiguous() if local_logits.stride(0) != vl else local_logits)
                logits = self.logits[:B]
                logits.view(B, self.tp, vl).copy_(gathered.permute(1, 0, 2))
        if logits is not None:
            if shape.adjust:
                from ..ops import suffix_ops
                self._count()
                if self.adj_idx is None:
                    self._alloc_adjust()
                suffix_ops.adjust_logits(logits, self.adj_idx[:B], self.adj_val[:B],
                                         self.guided_mask[:B] if shape.guided else None)
            self._count(2 if shape.sampler == 0 else 1)
            if shape.sampler == 0:
                K.argmax(logits, out=self.picked[:B], scratch=self.argmax_scratch)
            else:
                K.sample_gumbel(logits, self.samp_params[:B], self.samp_topk[:B], self.samp_seeds[:B], shape.sampler,
                                out=self.picked[:B])
            if shape.logprobs:
                from ..ops import suffix_ops
                self._count()
                suffix_ops.token_logprob(logits, self.picked[:B], out=self.logprobs[:B])
        if shape.chain:
            self._count()
            K.decode_advance(self.picked, self.tokens, self.positions, self.slots, self.row_ctx, self.block_tables,
                             self.row_seq, B)

    MAX_ADJ = 1024

    def _alloc_adjust(self) -> None:
        dev = self.device
        self.adj_idx = torch.full((self.max_seqs, self.MAX_ADJ), -1, dtype=torch.int32, device=dev)
        self.adj_val = torch.zeros(self.max_seqs, self.MAX_ADJ, 4, dtype=torch.float32, device=dev)
        self.guided_mask = torch.zeros(self.max_seqs, self.cfg.vocab, dtype=torch.float32, device=dev)

    def _forward_tp_oneshot(self, shape: StepShape) -> None:
        """Small steps on the fused tensor-parallel path with one-shot all-reduces: the o_proj / down_proj GEMM
        epilogues write their partial rows into every rank's inbox over NVLink, and the next kernel (residual add +
        RMSNorm) sums the inboxes in rank order.  One cross-rank synchronisation per projection, no library call."""
        cfg, w, comm = self.cfg, self.w, self.comm
        T, B, D = shape.tokens, shape.logit_rows, cfg.head_dim
        self._launch_counter = 0
        h, x = self.h[:T], self.x[:T]
        self._count(3)
        comm.begin_step()
        K.embed_gather(self.tokens[:T], w.embed, out=h)
        if cfg.embed_scale != 1.0:
            K.scale_(h, cfg.embed_scale)
        K.rmsnorm(h, w.layers[0].ln1, cfg.norm_eps, out=x)
        rs = -1
        for l, L in enumerate(w.layers):
            if l > 0:
                self._count()
                comm.norm_oneshot(h, L.ln1, x, T, cfg.norm_eps, rs_site=rs)
            splits = self._attn_splits(T)
            self._count(8 + (1 if splits > 1 else 0))
            K.linear(x, L.wqkv, K.EPI_STORE, self.qkv[:T])
            if L.bqkv is not None:
                K.bias_add_(self.qkv[:T], L.bqkv)
            K.rope_kv_write(self.qkv[:T], self.q[:T], self.kv.k(l), self.kv.v(l), self.positions[:T], self.slots[:T],
                            self.cos, self.sin, self.hq, self.hkv, D, cfg.rot, L.q_norm, L.k_norm, cfg.norm_eps)
            self._attention(l, T, T, B, count=False)
            rs += 1
            comm.gemm_allreduce(self.attn[:T], L.wo, T, rs_site=rs)
            comm.norm_oneshot(h, L.ln2, x, T, cfg.norm_eps, rs_site=rs)
            rs += 1
            if cfg.is_moe:
                from . import moe as _moe
                _moe.moe_forward(self, l, L, x, T, ep=("fused", comm, rs))
            else:
                K.linear(x, L.wgu, K.EPI_SWIGLU, self.act[:T])
                comm.gemm_allreduce(self.act[:T], L.wdown, T, rs_site=rs)
        if B == T:
            self._count()
            comm.norm_oneshot(h, w.final_norm, self.xl[:B], T, cfg.norm_eps, rs_site=rs)
        else:
            # reduce into h (normalised output unused), then gather the logit rows and normalise them
            self._count(3)
            comm.norm_oneshot(h, w.final_norm, x, T, cfg.norm_eps, rs_site=rs)
            K.gather_rows(h, self.logit_idx[:B], self.hl[:B])
            K.rmsnorm(self.hl[:B], w.final_norm, cfg.norm_eps, out=self.xl[:B])
        self._count()
        K.linear(self.xl[:B], w.lm_head, K.EPI_F32, self.logits_local[:B])
        self._sample(shape, self.logits_local[:B])
        self._count()
        comm.end_step()

    def _forward_tp_fused(self, shape: StepShape, R: int) -> None:
        """Decode-sized step on the fused tensor-parallel path: the residual stream is sharded by token rows
        (S rows per rank, R = world * S padded rows); every projection is one kernel that also does its collective."""
        cfg, w, comm = self.cfg, self.w, self.comm
        T, B, D = shape.tokens, shape.logit_rows, cfg.head_dim
        S = R // self.tp
        r0 = w.tp_rank * S
        self._launch_counter = 0
        self._count(2)
        comm.begin_step()
        K.embed_gather(self.tokens[r0:r0 + S], w.embed, out=comm.h_shard[:S])
        if cfg.embed_scale != 1.0:
            K.scale_(comm.h_shard[:S], cfg.embed_scale)
        ag, rs, pending_rs = 0, -1, -1       # pending_rs: the reduce-scatter site whose inboxes the next norm still has to add
        for l, L in enumerate(w.layers):
            self._count(5 + (1 if self._attn_splits(R) > 1 else 0))
            comm.norm(L.ln1, S, cfg.norm_eps, ag_site=ag, rs_site=pending_rs)
            comm.gemm(K.EPI_STORE, None, L.wqkv, self.qkv[:R], S, ag_site=ag)
            if L.bqkv is not None:
                K.bias_add_(self.qkv[:R], L.bqkv)
            K.rope_kv_write(self.qkv[:R], self.q[:R], self.kv.k(l), self.kv.v(l), self.positions[:R], self.slots[:R],
                            self.cos, self.sin, self.hq, self.hkv, D, cfg.rot, L.q_norm, L.k_norm, cfg.norm_eps)
            self._attention(l, R, T, B, count=False)
            rs += 1
            comm.gemm(K.EPI_STORE, self.attn[:R], L.wo, None, S, rs_site=rs)
            ag += 1
            if cfg.moe_layer(w.layer0 + l):
                # routed experts over the token-sharded stream: this rank's rows are normalised locally, each goes to
                # the ranks of its experts and its results come back (no all-gather, no reduce-scatter at this site)
                from . import moe as _moe
                x_own = self.x[:S]
                self._count()
                comm.norm_local(L.ln2, x_own, S, cfg.norm_eps, rs_site=rs)
                _moe.moe_forward_sharded(self, l, L, x_own, S, comm, site=l)
                rs += 1
                ag += 1
                pending_rs = -1
                continue
            self._count(3)
            comm.norm(L.ln2, S, cfg.norm_eps, ag_site=ag, rs_site=rs)
            comm.gemm(K.EPI_SWIGLU, None, L.wgu, self.act[:R], S, ag_site=ag)
            rs += 1
            comm.gemm(K.EPI_STORE, self.act[:R], L.wdown, None, S, rs_site=rs)
            ag += 1
            pending_rs = rs
        self._count(2)
        comm.norm(w.final_norm, S, cfg.norm_eps, ag_site=ag, rs_site=pending_rs)
        if R > self.logits_local.shape[0]:
            # prefill-sized step: only the sampling rows meet the head - picked out of the gathered rows once they landed
            comm.gather_rows(self.logit_idx[:B], self.xl[:B], B, S, ag_site=ag)
            local = self.logits_sel[:B]
            self._linear(self.xl[:B], w.lm_head, K.EPI_F32, local)
        else:
            comm.gemm(K.EPI_F32, None, w.lm_head, self.logits_local[:R], S, ag_site=ag)
            if B == T:
                local = self.logits_local[:B]
            else:
                self._count()
                local = self.logits_sel[:B]
                K.gather_rows(self.logits_local[:R], self.logit_idx[:B], local)
        self._sample(shape, local)
        self._count()
        comm.end_step()

    def _moe(self, l, L, x, T, h=None):
        from . import moe as _moe
        ep = ("nccl", self.comm) if (self.comm is not None and self.w.ep_world > 1) else None
        _moe.moe_forward(self, l, L, x, T, ep, h=h)
        if L.sh_wgu is not None:
            _moe.shared_expert(self, L, x, T, h=h)
        return None

    # ------------------------------------------------------------------ capture / replay
    def _key(self, shape: StepShape):
        flash_only = self.flash_ok and shape.tokens > shape.logit_rows and self._flash_only
        return (shape.tokens, shape.logit_rows, shape.sampler, shape.chain, shape.adjust, shape.guided, shape.logprobs,
                flash_only, shape.lora, shape.embeds, shape.mrope)

    def prepare(self, shape: StepShape, stage: Optional[str] = None) -> None:
        """Warm up and capture the step graph for ``shape`` (never done in the serving path afterwards).  ``stage``:
        one of the two stages of a step cut at its late-input point (``run_late``), captured as a graph of its own."""
        key = self._key(shape) + ((stage,) if stage else ())
        if key in self._graphs or not self.use_graphs:
            return
        if stage:
            self._stage = stage
            try:
                self._capture(shape, key)
            finally:
                self._stage = None
            return
        self._capture(shape, key)

    def _capture(self, shape: StepShape, key) -> None:
        # A program whose kernels wait on other ranks starts on every rank together: host rendezvous with the devices
        # idle before the eager warm-up forward, and again before the first replay of the captured graph.  Without it
        # a rank that finished its set-up seconds earlier would sit in device-side waits while its peers are still
        # building tensor maps, and would run out of its step budget for no fault of any rank.
        multi = self.comm is not None and self.tp > 1
        if multi:
            self.comm.rendezvous()
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self.forward(shape)  # warm-up: tensor-map cache, function attributes
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        if multi:
            K.check_status(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            self.forward(shape)
        self._graphs[key] = g
        self.launches_per_step[key] = self._launch_counter
        if multi:
            self.comm.rendezvous()

    def run(self, shape: StepShape, stage: Optional[str] = None) -> None:
        """Replay (or eagerly launch) one step; inputs must already be in the static buffers."""
        key = self._key(shape) + ((stage,) if stage else ())
        g = self._graphs.get(key)
        if g is None and self.use_graphs:
            self.prepare(shape, stage)
            g = self._graphs.get(key)
        if g is not None:
            g.replay()
            return
        self._stage = stage
        try:
            self.forward(shape)
        finally:
            self._stage = None
        self.launches_per_step[key] = self._launch_counter

    def run_late(self, shape: StepShape, late) -> None:
        """A step cut at its late-input point (crates/poot-executor/src/engine.rs "late_after"): the stages before the
        point are enqueued - everything up to the logits - then ``late()`` builds and binds what only the rest reads
        (the guided-decoding masks, the sparse logit adjustments) while the device is busy with the model body, then
        the sampler suffix is enqueued.  Each stage is its own captured graph."""
        if shape.chain:
            raise ValueError("a chained step feeds itself on the device; it has no late-input point")
        self.run(shape, "body")
        late()
        self.run(shape, "suffix")

    # ------------------------------------------------------------------ host-side input binding
    def bind(self, tokens, positions, slots, row_seq, row_ctx, logit_idx, block_tables=None,
             non_blocking: bool = True) -> None:
        """Copy one step's inputs (pinned host tensors) into the static device buffers."""
        T = tokens.numel()
        self.tokens[:T].copy_(tokens, non_blocking=non_blocking)
        hosted = getattr(self, "_hosted", None)
        if hosted is not None:                  # the rows this step gathers, as stored, into the device slot
            rows = hosted["stage"][:T]
            torch.index_select(hosted["table"], 0, tokens.long().clamp(0, hosted["table"].shape[0] - 1), out=rows)
            hosted["slot"][:T].copy_(rows, non_blocking=non_blocking)
        self.positions[:T].copy_(positions, non_blocking=non_blocking)
        self.slots[:T].copy_(slots, non_blocking=non_blocking)
        self.row_seq[:T].copy_(row_seq, non_blocking=non_blocking)
        self.row_ctx[:T].copy_(row_ctx, non_blocking=non_blocking)
        if self.comm is not None and getattr(self.comm, "fused", False):
            R = self.comm.rows_for(T)
            if R > T:  # padding rows of the fused path: no KV write, empty context
                self.tokens[T:R].zero_()
                self.positions[T:R].zero_()
                self.slots[T:R].fill_(-1)
                self.row_ctx[T:R].zero_()
                self.row_seq[T:R].zero_()
        B = logit_idx.numel()
        self.logit_idx[:B].copy_(logit_idx, non_blocking=non_blocking)
        if self._gdn_of or self._ssm_of:
            segs = K.step_segments(row_seq.numpy(), positions.numpy(), row_ctx.numpy())
            if segs.shape[0] > self._h_segs.shape[0]:
                raise ValueError("a step carries more sequence pieces than the engine has rows")
            self._h_segs.zero_()
            self._h_segs[:segs.shape[0]] = torch.from_numpy(segs)
            self.seg_table.copy_(self._h_segs, non_blocking=non_blocking)
        if self.flash_ok and T > B:
            tiles, covered = K.flash_tiles(row_seq.numpy(), positions.numpy())
            n = self._tile_slots(T, B)
            self._h_tiles[:n].zero_()
            self._h_tiles[:tiles.shape[0]] = torch.from_numpy(tiles)
            self._h_ctx_simt[:T] = row_ctx
            self._h_ctx_simt[:T][torch.from_numpy(covered)] = 0
            self._flash_only = bool(covered.all())
            self.attn_tiles[:n].copy_(self._h_tiles[:n], non_blocking=non_blocking)
            self.row_ctx_simt[:T].copy_(self._h_ctx_simt[:T], non_blocking=non_blocking)
            if self.row_ctx_simt.shape[0] > T:
                self.row_ctx_simt[T:].zero_()
        if block_tables is not None:
            self.block_tables[:block_tables.shape[0], :block_tables.shape[1]].copy_(block_tables,
                                                                                     non_blocking=non_blocking)
