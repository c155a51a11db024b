"""The device executor of a compiled plan: walks the launch list of ``plan/lower.py`` over one arena.

For the families whose layer the planner lowers completely (the pre-norm RMSNorm / rope / SwiGLU decoder layer with or
without q/k/v biases, per-head q/k norms and routed experts: llama, mistral, mixtral, qwen2, qwen3, qwen3-moe, phi3 ...)
the engine's step is this walk, not a hand-written sequence: the model is traced once into the graph IR, compiled
(passes, per-equation plans), lowered to launches, and every launch is bound here to a launcher, its weights (by the
canonical names the plan carries) and its operand buffers.  Buffers are views into ONE arena laid out by the lifetime
colouring of the launch program (``LaunchProgram.row_bytes``, bytes per token row scaled by the engine's row capacity),
so adding a family of this shape means writing its graph, not editing the engine.

Row-count dependent choices stay with the launchers (``ops.cuda_ops.linear`` picks the skinny or the tiled tcgen05 GEMM,
``DecoderEngine._attention`` the per-row or the tensor-core kernel, ``_proj_to_residual`` split-K with the reduction
deferred into the next norm), so one launch program serves every step shape and each shape is captured as its own CUDA
graph by the engine as before.

Reference: the plan walk of crates/poot-executor/src/engine.rs:2454-2700 over the ``Program`` of
crates/poot-graph-plan/src/compile.rs:923-1210.
"""
from __future__ import annotations

import re
from typing import Dict, Optional

import torch

from ..ops import cuda_ops as K
from ..plan.lower import Launch, LaunchProgram, LoweringRefused, lower

_LAYER = re.compile(r"^layers\.(\d+)\.(.+)$")
_GROUPS = {("attn_q", "attn_k", "attn_v"): "wqkv", ("ffn_gate", "ffn_up"): "wgu", ("attn_o",): "wo", ("ffn_down",): "wdown",
           ("attn_norm",): "ln1", ("ffn_norm",): "ln2"}


class ProgramExecutor:
    def __init__(self, engine, lp: LaunchProgram):
        self.e, self.lp = engine, lp
        dev = engine.device
        self.split = next((n for n, l in enumerate(lp.launches) if l.op == "rows"), len(lp.launches))
        # two row domains: token rows (up to max_tokens) before the logit rows are selected, sampling rows after
        t_rows, b_rows = engine.max_tokens, engine.max_seqs
        t_bytes = max((lp.row_bytes[l.out][0] + lp.row_bytes[l.out][1] for l in lp.launches[:self.split]), default=0)
        b_bytes = max((lp.row_bytes[l.out][0] + lp.row_bytes[l.out][1] for l in lp.launches[self.split:]
                       if l.epi != "f32"), default=0)
        self.arena = torch.zeros(t_rows * t_bytes + b_rows * b_bytes, dtype=torch.uint8, device=dev)
        self.arena_bytes = self.arena.numel()
        self.separate_bytes = t_rows * sum(lp.row_bytes[l.out][1] for l in lp.launches[:self.split])
        self.buf: Dict[int, torch.Tensor] = {}
        base_b = t_rows * t_bytes
        for n, l in enumerate(lp.launches):
            if l.epi == "f32":
                continue                        # the logits live in the engine's static buffer (the sampler suffix reads it)
            off, size = lp.row_bytes[l.out]
            rows = t_rows if n < self.split else b_rows
            start = off * rows + (0 if n < self.split else base_b)
            raw = self.arena[start:start + rows * l.width * l.dtype_bytes]
            self.buf[l.out] = raw.view(torch.bfloat16).view(rows, l.width)
        self.bound = [self._bind(l) for l in lp.launches]

    # ---- construction ------------------------------------------------------------------------------------------------
    @staticmethod
    def eligible(engine) -> bool:
        cfg, w = engine.cfg, engine.w
        if not cfg.plain_block or engine.comm is not None or engine.attn_general:
            return False
        if engine.stage is not None and engine.stage.count > 1:
            return False
        if cfg.layer_ffn is not None or cfg.mlp_bias or cfg.embed_scale != 1.0 or cfg.shared_width:
            return False
        return all(L.kind == "attention" and L.wgate is None and L.bo is None for L in w.layers)

    @staticmethod
    def build_for(engine) -> Optional["ProgramExecutor"]:
        """The executor for this engine's model, or None when the family is outside what the lowering covers (the
        engine then runs its hand-sequenced program)."""
        if not ProgramExecutor.eligible(engine):
            return None
        from ..models.model import Model, StepSpec
        from ..plan.compile import compile_graph
        try:
            g = Model(engine.cfg).trace(StepSpec(rows=2, tokens=2, capacity=64, paged=True, pool_slots=16 * 8))
            return ProgramExecutor(engine, lower(compile_graph(g)))
        except (LoweringRefused, KeyError, AttributeError):
            return None

    def _bind(self, l: Launch):
        """Weights (and biases) of a launch, resolved from the plan's canonical names to the engine's tensors."""
        w = self.e.w
        if l.op == "embed":
            return w.embed
        if l.op == "gemm" and l.epi == "f32":
            return w.lm_head
        if l.op in ("rope_kv", "attention", "rows"):
            return None
        roles = []
        for n in l.weights:
            m = _LAYER.match(n)
            roles.append(m.group(2) if m else n)
        if l.op == "rmsnorm" and roles == ["final_norm"]:
            return w.final_norm
        if l.op == "moe":
            return w.layers[l.layer - w.layer0]
        attr = _GROUPS.get(tuple(roles))
        if attr is None:
            raise LoweringRefused(f"no weight binding for {l.weights}")
        L = w.layers[l.layer - w.layer0]
        t = getattr(L, attr)
        if t is None:
            raise LoweringRefused(f"layer {l.layer} has no {attr}")
        if l.bias:
            if attr != "wqkv" or L.bqkv is None:
                raise LoweringRefused(f"no bias binding for {l.bias}")
            return (t, L.bqkv)
        return t

    def accepts(self, shape) -> bool:
        """Steps whose extras the launch list does not carry (resident adapters, rows of another modality, staged
        rotary rows) run the engine's hand-sequenced program."""
        return not (shape.lora or shape.embeds or shape.mrope)

    # ---- the walk ------------------------------------------------------------------------------------------------------
    def run(self, shape) -> None:
        e, cfg, w = self.e, self.e.cfg, self.e.w
        T, B, D = shape.tokens, shape.logit_rows, cfg.head_dim
        e._launch_counter = 0
        pending = None                          # (partials, residual value, output value) of a deferred split-K reduction
        buf = self.buf
        alias: Dict[int, torch.Tensor] = {}     # values that are another value's bytes for this step shape

        def flush():
            nonlocal pending
            if pending is not None:
                p, rv, ov = pending
                e._count()
                K.reduce_partials(buf[rv][:T], p, buf[ov][:T])
                pending = None

        for n, (l, bound) in enumerate(zip(self.lp.launches, self.bound)):
            rows = T if n < self.split else B
            if l.op == "embed":
                e._count()
                h = buf[l.out][:T]
                table = e.w.embed               # (rebound when the table moved to the host: the slot of gathered rows)
                if isinstance(table, K.QuantWeight):
                    K.quant_row_gather(e._embed_ids(T), table, out=h)
                else:
                    K.embed_gather(e._embed_ids(T), table, out=h)
            elif l.op == "rmsnorm":
                out = buf[l.out][:rows]
                e._count()
                if pending is not None and pending[2] == l.x:
                    p, rv, ov = pending         # the norm reads the residual stream anyway: it adds the split-K slices
                    K.rmsnorm(buf[rv][:T], bound, cfg.norm_eps, out=out, partials=p, h_out=buf[ov][:T])
                    pending = None
                else:
                    K.rmsnorm(alias.get(l.x, buf[l.x])[:rows], bound, cfg.norm_eps, out=out)
            elif l.op == "gemm":
                x = buf[l.x][:rows]
                if l.epi == "f32":
                    e._linear(x, bound, K.EPI_F32, e.logits_local[:B])
                elif l.epi == "swiglu":
                    e._linear(x, bound, K.EPI_SWIGLU, buf[l.out][:rows])
                elif l.epi == "resid":
                    flush()
                    p = e._proj_to_residual(x, bound, T, h=buf[l.resid][:T], out=buf[l.out][:T])
                    if p is not None:
                        pending = (p, l.resid, l.out)
                else:
                    W, bias = bound if isinstance(bound, tuple) else (bound, None)
                    out = e._linear(x, W, K.EPI_STORE, buf[l.out][:rows])
                    if bias is not None:
                        K.bias_add_(out, bias)
            elif l.op == "rope_kv":
                L = w.layers[l.layer - w.layer0]
                cos, sin = e._rope_tables_of(l.layer)
                kvl = e._kv_of[l.layer - w.layer0]
                e._count()
                K.rope_kv_write(buf[l.x][:T], buf[l.out][:T], e.kv.k(kvl), e.kv.v(kvl), e.positions[:T], e.slots[:T], cos, sin,
                                e.hq, e.hkv, D, cfg.rot, L.q_norm, L.k_norm, cfg.norm_eps)
            elif l.op == "attention":
                e._attention(l.layer - w.layer0, T, T, B, q=buf[l.x][:T], out=buf[l.out][:T])
            elif l.op == "moe":
                flush()
                h = buf[l.out][:T]
                if l.resid is not None and buf[l.resid].data_ptr() != buf[l.out].data_ptr():
                    h.copy_(buf[l.resid][:T])
                e._moe(l.layer - w.layer0, bound, buf[l.x][:T], T, h=h)
            elif l.op == "rows":
                flush()
                if B == T:                      # every row samples: the selected rows are the residual stream itself
                    alias[l.out] = buf[l.x]
                else:
                    e._count()
                    K.gather_rows(buf[l.x][:T], e.logit_idx[:B], buf[l.out][:B])
            else:                               # pragma: no cover - lower() only emits the kinds above
                raise LoweringRefused(l.op)
        flush()
        e._sample(shape, e.logits_local[:B])
