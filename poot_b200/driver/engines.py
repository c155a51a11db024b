"""Step engines behind the driver: the device engine adapter and the recording fake.

``DeviceStepEngine`` binds a padded ``StepInputs`` into the device engine's static buffers (one pinned staging
copy per field), replays the prepared step graph and reads back ``(token, non_finite_index)`` per sampling row -
never the logits (crates/poot-llm/src/driver/step.rs:776, suffix.rs:255).  ``FakeStepEngine`` records every step
and answers deterministically, which is how the scheduling and admission logic is tested without a GPU (the
reference's recording ``ServeEngine``, crates/poot-serve/src/tests/recording_engine.rs).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import numpy as np

from .driver import StepInputs


class FakeStepEngine:
    """Next token = (last fed token of the row + 1) mod vocab (moved to the next token a guided mask allows);
    records the steps it was asked to run."""

    def __init__(self, vocab: int = 1000, max_tokens: int = 256, fail_at_step: Optional[int] = None):
        self.vocab, self.max_tokens = vocab, max_tokens
        self.steps: List[StepInputs] = []
        self.block_tables = {}
        self.fail_at_step = fail_at_step

    def write_block_table(self, row: int, blocks) -> None:
        self.block_tables[row] = list(blocks)

    def run_step(self, inp: StepInputs) -> Tuple[np.ndarray, Optional[np.ndarray]]:
        if self.fail_at_step is not None and len(self.steps) == self.fail_at_step:
            raise RuntimeError("injected engine fault")
        self.steps.append(inp)
        self.last_run_ms, self.last_device_ms, self.last_launches = 0.0, None, 0
        self._last_first = []
        B = len(inp.logit_idx)
        picked = np.zeros((B, 2), np.int32)
        picked[:, 1] = -1
        for b in range(inp.live_rows):
            tok = (int(inp.tokens[inp.logit_idx[b]]) + 1) % self.vocab
            mask = (inp.adjust or {}).get("guided", {}).get(b) if inp.adjust else None
            if mask is not None:      # a guided row: the first allowed token at or after the candidate, cyclically
                ok = np.flatnonzero(np.asarray(mask) == 0.0)
                later = ok[ok >= tok]
                tok = int(later[0] if len(later) else ok[0])
            picked[b, 0] = tok
            self._last_first.append((int(inp.tokens[inp.logit_idx[b]]) + 1) % self.vocab)
        return picked, (np.zeros(B, np.float32) if inp.want_logprobs else None)


    def last_logits(self, rows: int) -> np.ndarray:
        """Synthetic logits of the last step: the favourite scores 0, every next id half a nat less."""
        out = np.zeros((rows, self.vocab), np.float32)
        ids = np.arange(self.vocab)
        for b in range(rows):
            out[b] = -0.5 * ((ids - self._last_first[b]) % self.vocab)
        return out

    def copy_block(self, src: int, dst: int) -> None:
        self.copies = getattr(self, "copies", []) + [(src, dst)]


class DeviceStepEngine:
    """Adapter from ``StepInputs`` to :class:`poot_b200.runtime.engine.DecoderEngine`."""

    def __init__(self, engine):
        import torch
        self.torch = torch
        self.e = engine
        self.max_tokens = engine.max_tokens
        n = engine.max_tokens
        pin = torch.cuda.is_available()

        def buf(shape, dtype):
            t = torch.zeros(shape, dtype=dtype)
            return t.pin_memory() if pin else t

        self.h_tokens, self.h_pos, self.h_slots = buf(n, torch.int32), buf(n, torch.int32), buf(n, torch.int32)
        self.h_seq, self.h_ctx = buf(n, torch.int32), buf(n, torch.int32)
        B = engine.max_seqs
        self.h_lidx = buf(B, torch.int64)
        self.h_params, self.h_topk, self.h_seeds = buf((B, 4), torch.float32), buf(B, torch.int32), buf(B, torch.int32)
        self.h_picked, self.h_logprobs = buf((B, 2), torch.int32), buf(B, torch.float32)
        self.h_bt = buf((engine.max_seqs, engine.max_blocks), torch.int32)
        self.h_status = buf(16, torch.int32)   # the device control block, read back with every step's result
        self.h_carry = None                    # host copy of the hidden-state carry, made when the engine exports one
        self.last_hidden = None
        self.status_hook = None                # tests: callable returning (code, detail) in place of the device's block
        self.device_timing = False           # bracket each step with CUDA events (opt-in: it adds a synchronisation)
        self.late_inputs = True              # guided-decoding masks may arrive as callables: built at the step's late-input point
        self.late_steps = 0
        self.bounds_checked = False          # the checked kernel library is loaded: read its record after every step
        if pin and engine.device.type == "cuda":
            from ..ops import cuda_ops as K
            if K.bounds_checking():
                self.bounds_checked = True
                K.set_bounds_limits(pool_slots=engine.kv.num_blocks * 16, pool_blocks=engine.kv.num_blocks,
                                    state_rows=engine.max_seqs)
        self.last_device_ms = None           # None = not measured
        self.last_run_ms = None
        self.last_launches = 0

    @property
    def carry(self) -> bool:
        """The engine leaves every token row's closing hidden state in ``last_hidden`` after a step."""
        return self.e.carry

    @property
    def block_tables(self):
        return self.e.block_tables

    @block_tables.setter
    def block_tables(self, tables) -> None:
        """Read another engine's block tables (a multi-token-prediction layer addresses its cache through the target's);
        set before the first step, which captures the tensor's address."""
        if tuple(tables.shape) != tuple(self.e.block_tables.shape):
            raise ValueError("block tables of different geometry cannot be shared")
        self.e.block_tables = tables

    def write_block_table(self, row: int, blocks) -> None:
        n = len(blocks)
        self.h_bt[row, :n] = self.torch.as_tensor(blocks, dtype=self.torch.int32)
        self.e.block_tables[row, :n].copy_(self.h_bt[row, :n], non_blocking=True)

    def run_step(self, inp: StepInputs):
        from ..runtime.engine import StepShape
        torch, e = self.torch, self.e
        T, B = len(inp.tokens), len(inp.logit_idx)
        for dst, src in ((self.h_tokens, inp.tokens), (self.h_pos, inp.positions), (self.h_slots, inp.slots),
                         (self.h_seq, inp.row_seq), (self.h_ctx, inp.row_ctx)):
            dst[:T] = torch.from_numpy(src)
        self.h_lidx[:B] = torch.from_numpy(inp.logit_idx)
        e.bind(self.h_tokens[:T], self.h_pos[:T], self.h_slots[:T], self.h_seq[:T], self.h_ctx[:T], self.h_lidx[:B])
        if inp.sampler != 0:
            self.h_params[:B] = torch.from_numpy(inp.params)
            self.h_topk[:B] = torch.from_numpy(inp.top_k)
            self.h_seeds[:B] = torch.from_numpy(inp.seeds)
            e.samp_params[:B].copy_(self.h_params[:B], non_blocking=True)
            e.samp_topk[:B].copy_(self.h_topk[:B], non_blocking=True)
            e.samp_seeds[:B].copy_(self.h_seeds[:B], non_blocking=True)
        guided = False
        late = None
        if inp.adjust is not None:
            if e.adj_idx is None:
                e._alloc_adjust()
            e.adj_idx[:B].copy_(torch.from_numpy(inp.adjust["idx"]), non_blocking=False)
            e.adj_val[:B].copy_(torch.from_numpy(inp.adjust["val"]), non_blocking=False)
            if inp.adjust["guided"]:
                guided = True
                rows = inp.adjust["guided"]

                def bind_masks():
                    e.guided_mask[:B].zero_()
                    for r, m in rows.items():
                        m = m() if callable(m) else m           # built now: the model body is already on the device
                        e.guided_mask[r].copy_(torch.from_numpy(np.ascontiguousarray(m, dtype=np.float32)))

                if any(callable(m) for m in rows.values()):
                    late = bind_masks
                else:
                    bind_masks()
        lora = False
        if inp.adapter_rows is not None:
            if e.lora is None:
                raise RuntimeError("a sequence names an adapter slot but the engine has no adapter bank")
            lora = e.lora.bind_rows(inp.adapter_rows, T)
        if inp.carry is not None:
            e.bind_carry(torch.from_numpy(np.ascontiguousarray(inp.carry[:T])), torch.from_numpy(inp.positions[:T]))
        embeds = inp.embed_flags is not None
        if embeds:
            e.bind_embeds(torch.from_numpy(inp.embed_flags[:T]), torch.from_numpy(inp.embed_rows[:T]))
        mrope = inp.rope_positions is not None
        if mrope:
            e.bind_rope_streams(torch.from_numpy(inp.rope_positions[:, :T]))
        shape = StepShape(T, B, inp.sampler, False, inp.adjust is not None, guided, inp.want_logprobs, lora, embeds, mrope)
        import time as _time
        t0 = _time.perf_counter()
        ev = None
        if self.device_timing:
            ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
            ev[0].record()
        if late is not None:
            e.run_late(shape, late)
            self.late_steps += 1
        else:
            e.run(shape)
        if ev is not None:
            ev[1].record()
        self.h_picked[:B].copy_(e.picked[:B], non_blocking=True)
        if inp.want_logprobs:
            self.h_logprobs[:B].copy_(e.logprobs[:B], non_blocking=True)
        if e.carry:
            if self.h_carry is None:
                self.h_carry = torch.zeros(e.max_tokens, e.cfg.hidden, dtype=torch.bfloat16)
                if torch.cuda.is_available():
                    self.h_carry = self.h_carry.pin_memory()
            self.h_carry[:T].copy_(e.carry_out[:T], non_blocking=True)
        on_device = e.device.type == "cuda"
        if on_device:
            # the control block rides the same stream as the result: no extra synchronisation
            from ..ops import cuda_ops as K
            self.h_status.copy_(K.status_word(e.device), non_blocking=True)
            torch.cuda.current_stream().synchronize()
        self._raise_on_failed_wait(on_device)
        if e.carry:
            self.last_hidden = self.h_carry[:T].float().numpy()
        self.last_run_ms = (_time.perf_counter() - t0) * 1e3
        self.last_device_ms = ev[0].elapsed_time(ev[1]) if ev is not None else None
        self.last_launches = e.launches_per_step.get(e._key(shape), 0)
        return self.h_picked[:B].numpy().copy(), (self.h_logprobs[:B].numpy().copy() if inp.want_logprobs else None)

    # ---- recurrent state: snapshot / restore of sequence rows (speculative rollback) ---------------------------------
    _STATE_NAMES = ("gdn_state", "gdn_conv_state", "ssm_state", "ssm_conv_state")

    @property
    def has_recurrent_state(self) -> bool:
        return any(getattr(self.e, n, None) is not None for n in self._STATE_NAMES)

    def snapshot_rows(self, rows) -> None:
        """Copy the recurrent state of the sequence rows ``rows`` into the shadow set.  Folding a token into a recurrent
        state is not invertible, so a speculative round keeps a copy of the rows it verifies and a partial accept copies
        them back and replays the kept tokens (crates/poot-llm/src/driver/snapshot.rs:1-17).  K/V needs no copy: a slot
        past the committed length is overwritten before it is ever visible."""
        torch = self.torch
        idx = torch.as_tensor(list(rows), dtype=torch.long, device=self.e.device)
        if getattr(self, "_shadow", None) is None:
            self._shadow = {n: torch.zeros_like(getattr(self.e, n)) for n in self._STATE_NAMES
                            if getattr(self.e, n, None) is not None}
        for n, sh in self._shadow.items():
            sh.index_copy_(1, idx, getattr(self.e, n).index_select(1, idx))

    def restore_rows(self, rows) -> None:
        torch = self.torch
        if getattr(self, "_shadow", None) is None:
            raise RuntimeError("restore_rows without a snapshot")
        idx = torch.as_tensor(list(rows), dtype=torch.long, device=self.e.device)
        for n, sh in self._shadow.items():
            getattr(self.e, n).index_copy_(1, idx, sh.index_select(1, idx))

    def abort(self) -> None:
        """Watchdog / signal-handler hook: every pending and future wait on another rank gives up at once."""
        if self.e.device.type == "cuda":
            from ..ops import cuda_ops as K
            K.request_abort(self.e.device)

    def abort_cleanup(self) -> None:
        """Clean-up after a failed step: make pending waits give up, let the device go idle, clear the control block."""
        if self.e.device.type != "cuda":
            return
        from ..ops import cuda_ops as K
        K.request_abort(self.e.device)
        try:
            self.torch.cuda.synchronize(self.e.device)
        finally:
            K.clear_abort(self.e.device)
        st = K.status_word(self.e.device)
        st[0:4].zero_()
        st[8:9].zero_()

    def reset_state(self) -> None:
        """The engine's part of a complete reset: recurrent and convolution state start from zero, the K/V pool's
        contents are dropped by the owner (its blocks return to the free list), and a tensor-parallel group starts its
        cross-rank counters over together."""
        e = self.e
        for name in ("gdn_state", "gdn_conv_state", "ssm_state", "ssm_conv_state"):
            t = getattr(e, name, None)
            if t is not None:
                t.zero_()
        comm = getattr(e, "comm", None)
        if comm is not None and hasattr(comm, "reset"):
            comm.reset()

    def _raise_on_failed_wait(self, on_device: bool) -> None:
        """A wait that gave up inside the step makes its tokens invalid: they must not reach a client.  The typed
        error leaves through the scheduler's guard, which fails the live requests and marks the engine dead."""
        if self.bounds_checked and on_device:
            from ..ops import cuda_ops as K
            K.check_bounds()                   # raises DeviceIndexOutOfRange: the step's tokens are discarded
        if self.status_hook is not None:
            code, detail = self.status_hook()
        elif on_device:
            code, detail = int(self.h_status[0]), int(self.h_status[1])
        else:
            return
        if code != 0:
            from ..ops import cuda_ops as K
            if on_device and self.status_hook is None:
                st = K.status_word(self.e.device)
                st[0:2].zero_()
                st[8:9].zero_()
            raise K.DeviceWaitTimeout(f"device wait timed out in {K.describe_status(code, detail)}; the step's "
                                      "tokens were discarded", code, detail)

    def last_logits(self, rows: int) -> np.ndarray:
        """Whole-vocabulary logits of the last step's sampling rows (single-rank engines only)."""
        if self.e.tp != 1:
            raise RuntimeError("ranks of a tensor-parallel engine hold vocabulary shards")
        return self.e.logits[:rows].float().cpu().numpy()

    def copy_block(self, src: int, dst: int) -> None:
        """Copy one K/V block in every layer (a forked sequence gets its own copy of the partial last block)."""
        self.e.kv.buf[:, :, dst].copy_(self.e.kv.buf[:, :, src])
        if getattr(self.e, "idx_pool", None) is not None:        # the sparse indexer's keys of the block travel with it
            self.e.idx_pool[:, dst].copy_(self.e.idx_pool[:, src])


class OracleStepEngine:
    """The CPU oracle behind the driver: every supported family runs end to end on the host.

    A step's ragged token list is cut into its per-sequence segments; each segment is one evaluation of the family's
    traced graph (``rows=1``, ``tokens=len(segment)``) whose paged K/V pools are this engine's state, read through
    the sequence's block table and written at the step's slots - the same maps the device program gets.  Sampling,
    logit adjustment and log-probabilities follow the rules the device kernels implement
    (crates/poot-eval/src/ops/sampling.rs:61-183).  This is the reference's ``poot-eval`` used as an executor: slow,
    exact in f32, and independent of any device kernel.
    """

    def __init__(self, model, weights, num_blocks: int, max_seqs: int, max_tokens: int, max_blocks_per_seq: int,
                 options=None, graph_transform=None, carry: bool = False, weight_formats=None):
        """``carry``: every step also keeps the closing-norm hidden state of each of its tokens (``last_hidden``), the
        input of a multi-token-prediction layer; the graphs are then traced with a logit row at every position.
        ``weight_formats``: name -> block format of the weights that ``weights`` holds as packed bytes; the step graphs
        declare them as stored, their contractions and row gathers are formed (``recognize_packed``) and evaluated by
        the native loops, so a quantised checkpoint is served at its packed size."""
        from ..oracle.eval import EvalOptions
        from .kvcache import BLOCK
        self.model, self.weights = model, weights
        self.block = BLOCK
        self.num_blocks, self.max_seqs, self.max_tokens, self.max_blocks = num_blocks, max_seqs, max_tokens, max_blocks_per_seq
        self.options = options or EvalOptions(matmul_precision="exact", native=bool(weight_formats))
        self.weight_formats = tuple(sorted((weight_formats or {}).items()))
        self.spec_extra = {}                         # further StepSpec fields of this engine's graphs (weight storage type)
        if self.weight_formats and graph_transform is None:
            def graph_transform(g):
                from ..plan import passes
                g = g.copy()
                passes.recognize_packed(g)
                return g
        self.graph_transform = graph_transform
        self.block_tables = np.zeros((max_seqs, max_blocks_per_seq), np.int32)
        self.state = {}
        self.graphs = {}
        self.steps = 0
        self._logits: Optional[np.ndarray] = None
        self.carry = carry or bool(getattr(model.cfg, "mtp_head", False))
        self.last_hidden: Optional[np.ndarray] = None
        self.last_run_ms, self.last_device_ms, self.last_launches = None, None, 0

    def write_block_table(self, row: int, blocks) -> None:
        self.block_tables[row, :len(blocks)] = np.asarray(blocks, np.int32)

    def _graph(self, tokens: int, capacity: int, embeds: bool = False, mrope: bool = False, all_rows: bool = False):
        all_rows = all_rows or self.carry
        key = (tokens, capacity, embeds, mrope, all_rows)
        if key not in self.graphs:
            from ..models.model import StepSpec
            g = self.model.trace(StepSpec(rows=1, tokens=tokens, capacity=capacity, paged=True,
                                          pool_slots=self.num_blocks * self.block, embeds=embeds, mrope=mrope,
                                          carry=self.carry, logit_rows="all" if all_rows else "last",
                                          weight_formats=self.weight_formats, **self.spec_extra))
            self.graphs[key] = self.graph_transform(g) if self.graph_transform is not None else g
        return self.graphs[key]

    def _segment(self, row: int, tokens: np.ndarray, positions: np.ndarray, slots: np.ndarray, ctx: int,
                 embed_flags: Optional[np.ndarray] = None, embed_rows: Optional[np.ndarray] = None,
                 rope_positions: Optional[np.ndarray] = None, carry: Optional[np.ndarray] = None, all_rows: bool = False):
        """Logits of the segment's last token, or with ``all_rows`` (a verify step reads a logit row per token) of every
        token; with ``carry`` engines ``(logits, hidden)`` of every token."""
        from ..oracle.eval import eval_graph
        blocks = max(1, -(-ctx // self.block))
        cap_blocks = 1
        while cap_blocks < blocks:
            cap_blocks *= 2
        cap_blocks = min(cap_blocks, self.max_blocks)
        cap = cap_blocks * self.block
        embeds = embed_flags is not None and bool(embed_flags.any())
        mrope = rope_positions is not None and bool(getattr(self.model.cfg, "mrope_sections", None))
        g = self._graph(len(tokens), cap, embeds, mrope, all_rows)
        bt = self.block_tables[row, :cap_blocks].astype(np.int64)
        read = (bt[:, None] * self.block + np.arange(self.block)[None, :]).reshape(1, cap).astype(np.int32)
        inputs = {"tokens": tokens.reshape(1, -1).astype(np.int32), "positions": positions.reshape(1, -1).astype(np.int32),
                  "read_map": read, "write_map": slots.astype(np.int32)}
        if mrope:
            inputs["rope_positions"] = np.ascontiguousarray(rope_positions, dtype=np.int32)
        if embeds:
            inputs["embed_flags"], inputs["embed_rows"] = embed_flags.astype(np.int32), embed_rows.astype(np.float32)
        if getattr(self.model.cfg, "mtp_head", False):
            if carry is None:
                raise ValueError("a multi-token-prediction layer steps over a hidden-state carry")
            inputs["carry"] = np.ascontiguousarray(carry, dtype=np.float32)
        fresh = int(positions[0]) == 0        # a sequence's first segment starts its recurrences from zero
        keys = {}
        for i in g.inputs:
            if i.storage == "const":
                inputs[i.name] = self.weights[i.name]
            elif i.storage == "state":
                # paged pools are shared by every sequence; recurrent state (conv taps, scan carry) belongs to the row
                key = (row, i.name) if getattr(i, "state_role", None) == "recurrent" else i.name
                if key not in self.state or (isinstance(key, tuple) and fresh):
                    self.state[key] = self._new_state(g.types[i.value])
                inputs[i.name] = self.state[key]
                keys[i.name] = key
        outputs = self._evaluate(g, inputs)
        for o in g.outputs:
            if o.role == "state_next":
                self.state[keys[o.state_of]] = outputs[o.name]
        if self.carry:
            return outputs["logits"], outputs["hidden"]
        return outputs["logits"] if all_rows else outputs["logits"][0]

    # ---- where the step's values live (overridden by the device evaluator) ---------------------------------------------
    def _new_state(self, ty):
        return np.zeros(ty.shape, dtype=np.float32)

    def _evaluate(self, g, inputs):
        from ..oracle.eval import eval_graph
        return eval_graph(g, inputs, self.options).outputs

    def run_step(self, inp: StepInputs):
        import time as _time
        from ..oracle.sampling import sample_rows
        t0 = _time.perf_counter()
        T, B = inp.live_tokens or len(inp.tokens), len(inp.logit_idx)
        vocab = self.model.cfg.vocab
        logits = np.zeros((B, vocab), np.float32)
        want = {int(i): b for b, i in enumerate(inp.logit_idx[:inp.live_rows])}
        hidden = np.zeros((T, self.model.cfg.hidden), np.float32) if self.carry else None
        start = 0
        while start < T:
            row = int(inp.row_seq[start])
            end = start + 1
            while end < T and int(inp.row_seq[end]) == row and int(inp.positions[end]) == int(inp.positions[end - 1]) + 1:
                end += 1
            if int(inp.row_ctx[start]) > 0:       # padding tokens have no context and write nothing
                ef = inp.embed_flags[start:end] if inp.embed_flags is not None else None
                er = inp.embed_rows[start:end] if inp.embed_flags is not None else None
                several = any(i in want for i in range(start, end - 1))          # a verify step: a logit row inside the segment
                out = self._segment(row, inp.tokens[start:end], inp.positions[start:end], inp.slots[start:end],
                                    int(inp.row_ctx[end - 1]), ef, er,
                                    inp.rope_positions[:, start:end] if inp.rope_positions is not None else None,
                                    inp.carry[start:end] if inp.carry is not None else None, all_rows=several)
                if self.carry or several:
                    seg_logits = out[0] if self.carry else out
                    if self.carry:
                        hidden[start:end] = out[1]
                    for i in range(start, end):
                        if i in want:
                            logits[want[i]] = seg_logits[i - start]
                elif end - 1 in want:
                    logits[want[end - 1]] = out
            start = end
        if inp.adjust is not None:
            idx, val = inp.adjust["idx"], inp.adjust["val"]
            for b in range(inp.live_rows):
                for t, v in zip(idx[b], val[b]):
                    if 0 <= t < vocab:
                        l = np.float32(logits[b, t] + v[0])
                        logits[b, t] = np.float32((l * v[1] if l > 0 else l * v[2]) + v[3])
                m = inp.adjust["guided"].get(b)
                if m is not None:
                    m = np.asarray(m, np.float32)
                    fmin = np.finfo(np.float32).min
                    logits[b] = np.where(m <= fmin, fmin, logits[b] + m).astype(np.float32)
        picked = sample_rows(logits, inp.params, inp.top_k, inp.seeds, inp.sampler)
        lp = None
        if inp.want_logprobs:
            mx = logits.max(-1, keepdims=True)
            lse = mx[:, 0] + np.log(np.exp(logits - mx).sum(-1))
            lp = (logits[np.arange(B), picked[:, 0]] - lse).astype(np.float32)
        self._logits = logits
        self.last_hidden = hidden
        self.steps += 1
        self.last_run_ms = (_time.perf_counter() - t0) * 1e3
        return picked, lp

    def last_logits(self, rows: int) -> np.ndarray:
        return self._logits[:rows]

    def _copy(self, v):
        return v.copy()

    # ---- recurrent state: snapshot / restore of sequence rows (speculative rollback), as on the device engine ---------
    @property
    def has_recurrent_state(self) -> bool:
        return bool(getattr(self.model.cfg, "is_recurrent", False))

    def snapshot_rows(self, rows) -> None:
        """Keep a copy of the recurrent state (conv windows, scan carries) of the sequence rows ``rows``: folding a
        token into it is not invertible, so a speculative round that rejects a draft restores the rows and replays
        what it keeps (crates/poot-llm/src/driver/snapshot.rs:1-17)."""
        rows = set(int(r) for r in rows)
        self._shadow = {k: self._copy(v) for k, v in self.state.items() if isinstance(k, tuple) and k[0] in rows}
        self._shadow_rows = rows

    def restore_rows(self, rows) -> None:
        if getattr(self, "_shadow", None) is None:
            raise RuntimeError("restore_rows without a snapshot")
        for k in [k for k in self.state if isinstance(k, tuple) and k[0] in self._shadow_rows]:
            del self.state[k]                      # a state first written after the snapshot starts from zero again
        self.state.update({k: self._copy(v) for k, v in self._shadow.items()})

    def copy_block(self, src: int, dst: int) -> None:
        b = self.block
        for name, pool in self.state.items():
            if isinstance(name, str) and name.endswith("_pool"):          # every paged pool: K/V, latent, indexer keys
                pool[dst * b:(dst + 1) * b] = pool[src * b:(src + 1) * b]


class GraphStepEngine(OracleStepEngine):
    """The general device executor behind the driver: the family's traced step graphs evaluated with tensors on
    ``device`` (``oracle/torch_eval.py``), weights uploaded once, paged pools and recurrent state resident there and
    written in place.  Every family the registry traces runs through it, including those the hand-written engine has
    no program for; one library or extension launch per equation, so it is launch-bound, and the logits come back to
    the host for the driver's sampling rules (crates/poot-executor: a planned program walked equation by equation)."""

    def __init__(self, model, weights, num_blocks: int, max_seqs: int, max_tokens: int, max_blocks_per_seq: int, device="cuda",
                 weight_dtype=None, carry: bool = False):
        import torch
        super().__init__(model, weights, num_blocks, max_seqs, max_tokens, max_blocks_per_seq, carry=carry)
        self.torch, self.device = torch, torch.device(device)
        self.weight_dtype = weight_dtype or torch.float32
        if self.weight_dtype == torch.bfloat16:       # the graphs declare the weights as stored and widen them where they are used
            from ..tensor import DType
            self.spec_extra = {"weight_dtype": DType.BF16}

        def up(a):
            t = torch.from_numpy(np.ascontiguousarray(a))
            return t.to(self.device, dtype=self.weight_dtype if t.dtype.is_floating_point else t.dtype)
        self.weights = {n: up(a) for n, a in weights.items()}
        self._owners = {}
        self._commit = {}

    def _new_state(self, ty):
        from ..oracle.torch_eval import StateTensor, torch_dtype
        st = StateTensor(tuple(ty.shape), torch_dtype(ty.dtype), self.device)
        self._owners[st.view.data_ptr()] = st
        return st.view

    def _copy(self, v):
        return v.clone()

    def _evaluate(self, g, inputs):
        from ..oracle.torch_eval import eval_graph_torch, torch_dtype
        torch = self.torch
        feed, in_place = {}, {}
        for i in g.inputs:
            if i.name not in inputs:
                continue
            v = inputs[i.name]
            want = torch_dtype(g.types[i.value].dtype)
            if not isinstance(v, torch.Tensor):
                v = torch.from_numpy(np.ascontiguousarray(v)).to(self.device)
            feed[i.name] = v if v.dtype == want else v.to(want)
            st = self._owners.get(feed[i.name].data_ptr()) if i.storage == "state" else None
            if st is not None:
                in_place[i.value] = st
        plan = self._commit.get(id(g))
        if plan is None:                                  # which updates may overwrite their state: proven once per graph
            from ..plan.state_commit import plan_state_commit
            plan = self._commit[id(g)] = set(plan_state_commit(g).inplace)
        out = eval_graph_torch(g, feed, self.device, in_place, donated=plan)
        res = {}
        for o in g.outputs:
            v = out[o.name]
            if o.role == "state_next":
                if v.data_ptr() not in self._owners:            # a recurrent state: a fresh tensor each step
                    v = v.contiguous()
                res[o.name] = v
            else:
                res[o.name] = v.float().cpu().numpy()
        return res

    def copy_block(self, src: int, dst: int) -> None:
        b = self.block
        for name, pool in self.state.items():
            if isinstance(name, str) and name.endswith("_pool"):
                pool[dst * b:(dst + 1) * b].copy_(pool[src * b:(src + 1) * b])
