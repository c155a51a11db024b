"""Sentence embeddings and cross-encoder scores from an encoder checkpoint.

``Embedder`` is the ``encode`` counterpart of ``LLM``: it loads a BERT-family directory, tokenises, pads the batch
on the right, evaluates the traced encoder graph and pools on the host (the reference's ``poot embed`` and the
``/v1/embeddings`` / ``/v1/rerank`` routes: crates/poot-models/src/architectures/bert.rs:1-11,
crates/poot-serve/src/handlers.rs).  The graph evaluator is the CPU oracle; a padded token is never attended to,
so a text's vector does not depend on what it is batched with.
"""
from __future__ import annotations

import os
import threading
import time
from typing import List, Optional, Sequence, Tuple

import numpy as np


class EmbedError(ValueError):
    pass


class PairTokenizer:
    """Adds the ``[CLS] a [SEP] (b [SEP])`` frame a BERT checkpoint expects around a tokenizer's plain encoding."""

    def __init__(self, tk, cls_id: int, sep_id: int):
        self.tk, self.cls, self.sep = tk, cls_id, sep_id

    def _plain(self, text: str) -> List[int]:
        try:
            return list(self.tk.encode(text, add_bos=False))
        except TypeError:
            return list(self.tk.encode(text))

    def encode(self, a: str, b: Optional[str] = None) -> Tuple[List[int], List[int]]:
        ids = [self.cls] + self._plain(a) + [self.sep]
        types = [0] * len(ids)
        if b is not None:
            second = self._plain(b) + [self.sep]
            ids += second
            types += [1] * len(second)
        return ids, types


class Embedder:
    def __init__(self, model, weights, tokenizer: PairTokenizer, name: str = "bert"):
        self.model, self.weights, self.tk, self.name = model, weights, tokenizer, name
        self.cfg = model.cfg
        self.graphs = {}
        self.lock = threading.Lock()
        self.engine = None               # device program (runtime/encoder_engine.py); None: the host evaluator

    def to_device(self, device="cuda", max_tokens: int = 4096, max_rows: int = 64) -> "Embedder":
        """Run the encoder on the B200 engine (bf16) instead of the host evaluator."""
        import torch
        from .runtime.encoder_engine import EncoderEngine
        tensors = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in self.weights.items()}
        self.engine = EncoderEngine(self.cfg, tensors, device, max_tokens, max_rows)
        return self

    @staticmethod
    def load(path: str, backend: str = "oracle", device="cuda") -> "Embedder":
        """``backend``: ``oracle`` (host evaluator, f32) or ``device`` (the B200 engine, bf16)."""
        if backend not in ("oracle", "device"):
            raise EmbedError(f"backend {backend!r}: oracle or device")
        emb = Embedder._load(path)
        return emb.to_device(device) if backend == "device" else emb

    @staticmethod
    def _load(path: str) -> "Embedder":
        from .driver.handle import ModelHandle
        handle = ModelHandle.load(path)
        if getattr(handle.model, "kind", "decoder") != "encoder":
            raise EmbedError(f"{path}: family {handle.cfg.family!r} is a decoder; embeddings need an encoder checkpoint")
        tkfile = os.path.join(path, "tokenizer.json")
        if os.path.exists(tkfile):
            from .text.codec import HfTokenizer
            tk = HfTokenizer(tkfile)
            cls_id = tk.tk.token_to_id("[CLS]")
            sep_id = tk.tk.token_to_id("[SEP]")
            if cls_id is None or sep_id is None:
                raise EmbedError("tokenizer has no [CLS] / [SEP]")
        else:       # no tokenizer beside the weights: bytes, with the two highest ids as the frame
            from .text.codec import ByteTokenizer
            tk = ByteTokenizer(handle.cfg.vocab)
            cls_id, sep_id = handle.cfg.vocab - 2, handle.cfg.vocab - 1
        return Embedder(handle.model, handle.oracle_weights(), PairTokenizer(tk, cls_id, sep_id), os.path.basename(path.rstrip("/")))

    # ---- evaluation ----------------------------------------------------------------------------------------------
    def forward(self, ids: Sequence[Sequence[int]], types: Optional[Sequence[Sequence[int]]] = None) -> np.ndarray:
        """``hidden[rows, T, H]`` (embedders) or ``scores[rows, labels]`` (classifier checkpoints) for right-padded rows."""
        from .oracle.eval import EvalOptions, eval_graph
        c = self.cfg
        R = len(ids)
        longest = max(len(x) for x in ids)
        if longest > c.max_position:
            raise EmbedError(f"input of {longest} tokens exceeds the model's {c.max_position} positions")
        if self.engine is not None:
            with self.lock:
                if c.labels:
                    return self.engine.scores(ids, types).cpu().numpy()
                rows = self.engine.forward(ids, types)
                hid = np.zeros((R, longest, c.hidden), np.float32)
                for r, x in enumerate(rows):
                    hid[r, :x.shape[0]] = x.cpu().numpy()
                return hid
        T = min(-(-longest // 16) * 16, c.max_position)
        tok = np.full((R, T), c.pad_token, np.int32)
        typ = np.zeros((R, T), np.int32)
        real = np.zeros((R, T), np.int32)
        for r, x in enumerate(ids):
            tok[r, :len(x)] = x
            real[r, :len(x)] = 1
            if types is not None:
                typ[r, :len(x)] = types[r]
        with self.lock:
            if (R, T) not in self.graphs:
                self.graphs[(R, T)] = self.model.trace(R, T)
            g = self.graphs[(R, T)]
            inputs = {"tokens": tok, "positions": np.arange(T, dtype=np.int32)[None].repeat(R, 0), "token_type": typ,
                      "real_tokens": real}
            for i in g.inputs:
                if i.storage == "const":
                    inputs[i.name] = self.weights[i.name]
            out = eval_graph(g, inputs, EvalOptions(matmul_precision="exact")).outputs
        return out["scores"] if c.labels else out["hidden"]

    def embed_ids(self, ids: Sequence[Sequence[int]], pooling: str = "mean", normalize: bool = True) -> np.ndarray:
        if self.cfg.labels:
            raise EmbedError("the checkpoint is a classifier (cross-encoder): it scores pairs, it does not embed")
        if pooling not in ("mean", "cls"):
            raise EmbedError(f"pooling {pooling!r}: mean or cls")
        hid = self.forward(ids)
        out = np.zeros((len(ids), self.cfg.hidden), np.float32)
        for r, x in enumerate(ids):
            out[r] = hid[r, 0] if pooling == "cls" else hid[r, :len(x)].mean(0)
        if normalize:
            out /= np.maximum(np.linalg.norm(out, axis=-1, keepdims=True), 1e-12)
        return out

    def embed(self, texts: Sequence[str], pooling: str = "mean", normalize: bool = True) -> Tuple[np.ndarray, int]:
        ids = [self.tk.encode(t)[0] for t in texts]
        return self.embed_ids(ids, pooling, normalize), sum(len(x) for x in ids)

    def rerank(self, query: str, documents: Sequence[str]) -> Tuple[np.ndarray, int]:
        """Relevance of each document to the query: the classifier logit of the pair (cross-encoders), or the cosine of
        the two embeddings when the checkpoint is an embedder."""
        if self.cfg.labels:
            pairs = [self.tk.encode(query, d) for d in documents]
            s = self.forward([p[0] for p in pairs], [p[1] for p in pairs])
            return s[:, 0].astype(np.float32), sum(len(p[0]) for p in pairs)
        vec, n = self.embed([query] + list(documents))
        return (vec[1:] @ vec[0]).astype(np.float32), n


class EmbedEngine:
    """What the HTTP layer needs from an engine when the served model is an encoder: health, metrics, drain."""

    def __init__(self, embedder: Embedder, metrics):
        self.embedder, self.metrics = embedder, metrics
        self.state, self.cause, self.timing, self.driver = "serving", None, None, None
        self.tk = embedder.tk.tk
        self.inflight = 0
        self._lock = threading.Lock()

    def health(self) -> dict:
        h = {"status": self.state}
        if self.state == "serving":
            h.update({"backend": "oracle" if self.embedder.engine is None else "b200", "kind": "encoder", "max_seq": self.embedder.cfg.max_position})
        return h

    def run(self, fn):
        if self.state != "serving":
            raise RuntimeError("draining")
        with self._lock:
            self.inflight += 1
        t0 = time.monotonic()
        self.metrics.inc("poot_requests_total")
        try:
            out = fn()
            self.metrics.inc("poot_requests_completed_total")
            return out
        except Exception:
            self.metrics.inc("poot_requests_errored_total")
            raise
        finally:
            self.metrics.observe("poot_request_e2e_ms", (time.monotonic() - t0) * 1e3)
            with self._lock:
                self.inflight -= 1

    def drain(self, timeout: float = 30.0) -> None:
        self.state = "draining"
        deadline = time.monotonic() + timeout
        while self.inflight and time.monotonic() < deadline:
            time.sleep(0.01)
