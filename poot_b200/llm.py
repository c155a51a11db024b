"""The call a user makes: load a checkpoint (or a random-init preset), get a driver, a tokenizer and ``generate``.

Mirrors the reference's ``ModelHandle`` -> ``Driver`` pairing (crates/poot-llm/src/driver/handle.rs:233,
crates/poot-llm/src/driver/run.rs:136-248): the handle resolves the family and weights, the driver owns rows,
paged K/V and the prefix cache, and a step engine runs the device program.  KV capacity is sized from the device
memory left after the weights are resident.
"""
from __future__ import annotations

import os
from typing import Iterable, List, Optional

from .driver.driver import Driver
from .driver.kvcache import BLOCK, blocks_for
from .driver.sampler import SamplingParams
from .models.config import DecoderConfig, PRESETS
from .text.codec import ByteTokenizer, GgufTokenizer, HfTokenizer, StreamDecoder


def _stage_and_link(cfg, pp_rank: int, pp_world: int, link):
    """This process's layer range of a pipeline over ``pp_world`` processes, and the link to its neighbours."""
    if pp_world <= 1:
        return None, None
    from .driver.placement import pipeline_cuts
    from .parallel.pipeline import PipelineLink
    from .runtime.weights import StageSpec
    l0, l1 = pipeline_cuts(cfg, pp_world)[pp_rank]
    return StageSpec(pp_rank, pp_world, l0, l1), (link or PipelineLink(pp_rank, pp_world))


def _tokenizer_for(handle):
    if handle is None:
        return None
    if handle.kind == "hf":
        p = os.path.join(handle.source, "tokenizer.json")
        if os.path.exists(p):
            return HfTokenizer(p)
    elif "tokenizer.ggml.tokens" in handle.store.metadata:
        return GgufTokenizer(handle.store.metadata)
    return None


class LLM:
    """A resident model with its serving driver."""

    def __init__(self, cfg: DecoderConfig, driver: Driver, tokenizer, engine=None, handle=None, comm=None):
        self.cfg, self.driver, self.tokenizer, self.engine, self.handle, self.comm = cfg, driver, tokenizer, engine, handle, comm
        self.draft = None           # draft policy of the model itself (its multi-token-prediction layer), when it has one

    # ---- construction --------------------------------------------------------------------------------------------
    @staticmethod
    def _assemble(cfg, weights, tokenizer, rows, max_seq, prefill_chunk, kv_fraction, comm, handle, num_blocks=None,
                  prefix_caching=True, prefill_budget=None, link=None, mtp=None):
        """``mtp``: ``(device weights of the model's multi-token-prediction layer, k)``; the layer gets a one-block engine
        of its own whose K/V pool is addressed through the target's block tables."""
        import torch
        from .driver.engines import DeviceStepEngine
        from .runtime.engine import DecoderEngine, KVPool
        dev = weights.layers[0].wo.device
        max_seq = min(max_seq, cfg.max_position)
        if num_blocks is None:      # capacity fit against the memory left after the weights are resident
            from .driver import capacity
            free, _ = torch.cuda.mem_get_info(dev)
            shapes = capacity.fit(cfg, free, rows, max_seq, max(prefill_chunk, prefill_budget or 0), weights.tp_world,
                                  kv_fraction=kv_fraction)
            rows, max_seq, num_blocks = shapes.rows, shapes.max_seq, shapes.num_blocks
            prefill_chunk = min(prefill_chunk, max_seq)
            if comm is not None or link is not None:      # every rank must agree: take the smallest fit over the group
                import torch.distributed as dist
                t = torch.tensor([rows, max_seq, prefill_chunk, num_blocks], dtype=torch.int64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MIN)
                rows, max_seq, prefill_chunk, num_blocks = (int(v) for v in t.tolist())
        step_prefill = max(prefill_chunk, min(prefill_budget or 0, rows * prefill_chunk))
        max_tokens = max(step_prefill, rows) + rows             # prefill tokens of a step + one decode row per sequence
        # pipeline stages launch eagerly: their steps contain point-to-point transfers whose capture is not relied on
        if mtp is not None:
            from .driver.features import Feature, check as _check, require_mtp
            require_mtp(cfg)
            _check([Feature.DRAFT_MTP] + ([Feature.TENSOR_PLACEMENT] if comm is not None else [])
                   + ([Feature.PIPELINE_PLACEMENT] if link is not None else []))
            prefix_caching = False     # a block's last position in the layer's cache depends on the token after it
        eng = DecoderEngine(weights, num_blocks, rows, max_tokens, blocks_for(max_seq), comm=comm, link=link,
                            use_graphs=link is None and dev.type == "cuda", carry=mtp is not None)
        tokenizer = tokenizer or ByteTokenizer(cfg.vocab, bos=cfg.bos_token, eos=cfg.eos_token)
        eos = getattr(tokenizer, "eos", None)
        if cfg.is_recurrent:
            from .driver.features import Feature, check
            check([Feature.RECURRENT_STATE] + ([Feature.TENSOR_PLACEMENT] if comm is not None else []))
            prefix_caching = False         # a prefix hit skips tokens whose recurrent state is not cached
        drv = Driver(DeviceStepEngine(eng), num_blocks, rows, max_seq, cfg.vocab, prefill_chunk=prefill_chunk,
                     prefix_caching=prefix_caching, eos_token=eos if eos is not None else cfg.eos_token,
                     prefill_budget=step_prefill)
        llm = LLM(cfg, drv, tokenizer, eng, handle, comm)
        if mtp is not None:
            from .driver.speculate import MtpDraft
            layer_weights, k = mtp
            layer = DecoderEngine(layer_weights, num_blocks, rows, max_tokens, blocks_for(max_seq),
                                  use_graphs=dev.type == "cuda")
            llm.mtp_engine = layer
            llm.draft = MtpDraft(DeviceStepEngine(layer), k).attach(drv)
        return llm

    @staticmethod
    def load(path: str, device="cuda", rows: int = 32, max_seq: int = 4096, prefill_chunk: int = 512,
             kv_fraction: float = 0.85, keep_packed: bool = True, tp_rank: int = 0, tp_world: int = 1, comm=None,
             num_blocks: Optional[int] = None, lora: Optional[str] = None, prefill_budget: Optional[int] = None,
             pp_rank: int = 0, pp_world: int = 1, link=None, draft_mtp: int = 0) -> "LLM":
        """``path``: a Hugging Face directory (config.json + safetensors) or a ``.gguf`` file; ``lora``: a PEFT adapter
        directory merged into the projections at load; ``pp_rank`` / ``pp_world``: this process's stage of a layer
        pipeline (it loads only its layers)."""
        from .driver.handle import ModelHandle, device_weights
        handle = ModelHandle.load(path)
        if lora is not None:
            from .load.lora import load_adapter
            handle.apply_adapter(load_adapter(lora))
        stage, link = _stage_and_link(handle.cfg, pp_rank, pp_world, link)
        weights = device_weights(handle, device, tp_rank, tp_world, keep_packed, stage=stage)
        mtp = None
        if draft_mtp:
            from .driver.features import Feature, Unavailable, require_mtp
            from .driver.handle import mtp_device_weights
            require_mtp(handle.cfg)
            if not handle.has_mtp:
                raise Unavailable(Feature.DRAFT_MTP, f"{path} does not store the model's multi-token-prediction layer")
            mtp = (mtp_device_weights(handle, device, weights), draft_mtp)
        return LLM._assemble(handle.cfg, weights, _tokenizer_for(handle), rows, max_seq, prefill_chunk, kv_fraction,
                             comm, handle, num_blocks, prefill_budget=prefill_budget, link=link, mtp=mtp)

    @staticmethod
    def random(preset: str, device="cuda", rows: int = 32, max_seq: int = 4096, prefill_chunk: int = 512,
               kv_fraction: float = 0.85, seed: int = 0, std: float = 0.02, tp_rank: int = 0, tp_world: int = 1,
               comm=None, num_blocks: Optional[int] = None, prefill_budget: Optional[int] = None, pp_rank: int = 0,
               pp_world: int = 1, link=None, draft_mtp: int = 0, **over) -> "LLM":
        """Random-init weights of a named architecture (benchmarks and tests: no checkpoint on disk).  ``draft_mtp``:
        also draw a multi-token-prediction layer (the configuration must name one: ``mtp_layers=1``) and draft with it."""
        from .runtime.weights import random_weights, share_tables
        import dataclasses
        cfg = dataclasses.replace(PRESETS[preset](), **over)
        stage, link = _stage_and_link(cfg, pp_rank, pp_world, link)
        if draft_mtp:
            from .driver.features import require_mtp
            require_mtp(cfg)                    # refused before a byte of weights is drawn
        weights = random_weights(cfg, device, seed=seed, std=std, tp_rank=tp_rank, tp_world=tp_world, stage=stage)
        mtp = None
        if draft_mtp:
            from .models.config import mtp_config
            mtp = (share_tables(random_weights(mtp_config(cfg), device, seed=seed + 1, std=std), weights), draft_mtp)
        return LLM._assemble(cfg, weights, None, rows, max_seq, prefill_chunk, kv_fraction, comm, None, num_blocks,
                             prefill_budget=prefill_budget, link=link, mtp=mtp)

    @staticmethod
    def fake(vocab: int = 1000, rows: int = 8, max_seq: int = 512, num_blocks: int = 256, prefill_chunk: int = 64,
             fail_at_step: Optional[int] = None, prefill_budget: Optional[int] = None) -> "LLM":
        """A driver over the deterministic host engine (next token = last + 1): serving logic without a device."""
        from .driver.engines import FakeStepEngine
        tk = ByteTokenizer(vocab)
        drv = Driver(FakeStepEngine(vocab, max(prefill_chunk, prefill_budget or 0) + rows, fail_at_step), num_blocks, rows,
                     max_seq, vocab, prefill_chunk=prefill_chunk, eos_token=tk.eos, prefill_budget=prefill_budget)
        return LLM(None, drv, tk)

    @staticmethod
    def oracle(path: str, rows: int = 4, max_seq: int = 512, num_blocks: int = 128, prefill_chunk: int = 64,
               lora: Optional[str] = None, prefill_budget: Optional[int] = None, draft_mtp: int = 0, packed: bool = False) -> "LLM":
        """A checkpoint served by the CPU oracle: every supported family end to end on the host, in f32, through the
        same driver (paged K/V, prefix cache, sampling rules) as the device engine.  Slow; meant for checking a
        family or a checkpoint without a device."""
        from .driver.engines import OracleStepEngine
        from .driver.handle import ModelHandle
        handle = ModelHandle.load(path)
        if lora is not None:
            from .load.lora import load_adapter
            handle.apply_adapter(load_adapter(lora))
        mtp = None
        if draft_mtp:
            from .driver.features import Feature, Unavailable, require_mtp
            require_mtp(handle.cfg)
            if not handle.has_mtp:
                raise Unavailable(Feature.DRAFT_MTP, f"{path} does not store the model's multi-token-prediction layer")
            mtp = (handle.mtp_oracle_weights(), draft_mtp)
        if packed:
            # quantised matrices stay as stored and are decoded inside the contractions by the native loops
            if lora is not None or mtp is not None:
                raise ValueError("the packed oracle serves a plain checkpoint (no adapter, no draft layer)")
            weights, formats = handle.packed_oracle_weights()
            return LLM.oracle_from(handle.model, weights, _tokenizer_for(handle), rows, max_seq, num_blocks, prefill_chunk, handle,
                                   prefill_budget, weight_formats=formats)
        return LLM.oracle_from(handle.model, handle.oracle_weights(), _tokenizer_for(handle), rows, max_seq, num_blocks,
                               prefill_chunk, handle, prefill_budget, mtp=mtp)

    @staticmethod
    def graph(path: str, device: str = "cuda", rows: int = 4, max_seq: int = 512, num_blocks: int = 128, prefill_chunk: int = 64,
              dtype: str = "bf16", prefill_budget: Optional[int] = None) -> "LLM":
        """A checkpoint served by the general device executor: the family's step graphs evaluated equation by equation
        with tensors on ``device`` (weights in ``dtype``, arithmetic in f32, pools resident and written in place).  Every
        family the registry traces runs this way, including those without a hand-written device program; it is
        launch-bound, so the hand-written engine (``LLM.load``) is the one to use where it has a program."""
        import torch
        from .driver.engines import GraphStepEngine
        from .driver.handle import ModelHandle
        handle = ModelHandle.load(path)
        cfg = handle.cfg
        max_seq = min(max_seq, cfg.max_position)
        step_prefill = max(prefill_chunk, min(prefill_budget or 0, rows * prefill_chunk))
        wd = {"bf16": torch.bfloat16, "f32": torch.float32}[dtype]
        eng = GraphStepEngine(handle.model, handle.oracle_weights(), num_blocks, rows, step_prefill + rows, blocks_for(max_seq),
                              device=device, weight_dtype=wd)
        tokenizer = _tokenizer_for(handle)
        eos = getattr(tokenizer, "eos", None)
        from .driver.features import Feature, check
        check([Feature.RECURRENT_STATE] if cfg.is_recurrent else [])
        drv = Driver(eng, num_blocks, rows, max_seq, cfg.vocab, prefill_chunk=prefill_chunk, prefix_caching=not cfg.is_recurrent,
                     eos_token=eos if eos is not None else cfg.eos_token, prefill_budget=step_prefill)
        return LLM(cfg, drv, tokenizer, None, handle, None)

    @staticmethod
    def oracle_from(model, weights, tokenizer=None, rows: int = 4, max_seq: int = 512, num_blocks: int = 128,
                    prefill_chunk: int = 64, handle=None, prefill_budget: Optional[int] = None, mtp=None,
                    weight_formats=None) -> "LLM":
        """``mtp``: ``(weights of the multi-token-prediction layer, k)``: the layer drafts ``k`` tokens per round for a
        lone greedy sequence (``LLM.draft``); the model's configuration must store such a layer."""
        from .driver.engines import OracleStepEngine
        cfg = model.cfg
        max_seq = min(max_seq, cfg.max_position)
        step_prefill = max(prefill_chunk, min(prefill_budget or 0, rows * prefill_chunk))
        eng = OracleStepEngine(model, weights, num_blocks, rows, step_prefill + rows, blocks_for(max_seq),
                               carry=mtp is not None, weight_formats=weight_formats)
        tokenizer = tokenizer or ByteTokenizer(cfg.vocab, bos=cfg.bos_token, eos=cfg.eos_token)
        eos = getattr(tokenizer, "eos", None)
        # a prefix hit skips tokens; a recurrent layer's state after those tokens is not in the K/V cache, so recurrent
        # families run without the prefix cache (the reference snapshots recurrent state instead)
        from .driver.features import Feature, check
        check([Feature.RECURRENT_STATE] if cfg.is_recurrent else [])
        drv = Driver(eng, num_blocks, rows, max_seq, cfg.vocab, prefill_chunk=prefill_chunk,
                     prefix_caching=not cfg.is_recurrent and mtp is None,
                     eos_token=eos if eos is not None else cfg.eos_token, prefill_budget=step_prefill)
        llm = LLM(cfg, drv, tokenizer, None, handle, None)
        if mtp is not None:
            # a block's last position depends on the token after it, so prefix reuse is off under this policy
            from .driver.features import Feature
            from .driver.speculate import MtpDraft
            from .models.config import mtp_config
            from .models.model import Model
            from .driver.features import require_mtp
            require_mtp(cfg)
            check([Feature.DRAFT_MTP] + ([Feature.RECURRENT_STATE] if cfg.is_recurrent else []))
            mtp_weights, k = mtp
            layer = model.mtp_model()
            runner = OracleStepEngine(layer, mtp_weights, num_blocks, rows, step_prefill + rows, blocks_for(max_seq))
            llm.draft = MtpDraft(runner, k).attach(drv)
        return llm

    # ---- generation ----------------------------------------------------------------------------------------------
    def generate_tokens(self, prompt: Iterable[int], params: Optional[SamplingParams] = None, on_token=None,
                        embeds=None, rope_positions=None) -> List[int]:
        """``embeds``: ``(positions, rows)`` replacing the embeddings of those prompt tokens (image rows of a VLM);
        ``rope_positions[3, len(prompt)]``: the prompt's rotary position streams under a sectioned rope."""
        p = params or SamplingParams()
        if (self.draft is not None and embeds is None and rope_positions is None and p.greedy and not p.needs_adjust
                and not p.logprobs):
            from .driver.speculate import generate_speculative
            return generate_speculative(self.driver, list(prompt), p, self.draft, on_token)
        return self.driver.generate(list(prompt), params, on_token, embeds=embeds, rope_positions=rope_positions)

    def generate(self, prompt: str, params: Optional[SamplingParams] = None, on_text=None) -> str:
        dec = StreamDecoder(self.tokenizer)
        out: List[str] = []

        def tok(t):
            if t == self.driver.eos_token:
                return
            piece = dec.push(t)
            if piece:
                out.append(piece)
                if on_text is not None:
                    on_text(piece)

        self.driver.generate(self.tokenizer.encode(prompt), params, tok)
        tail = dec.flush()
        if tail:
            out.append(tail)
            if on_text is not None:
                on_text(tail)
        return "".join(out)

    def chat(self, messages: List[dict], params: Optional[SamplingParams] = None, template: Optional[str] = None,
             on_text=None) -> str:
        from .text.chat import render_chat
        family = self.cfg.family if self.cfg is not None else "llama"
        text = render_chat(messages, template, family, True)
        return self.generate(text, params, on_text)

    def close(self) -> None:
        if self.comm is not None:
            self.comm.close()
