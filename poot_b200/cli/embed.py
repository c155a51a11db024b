"""``poot embed {similarity|rerank|cross} MODEL_DIR TEXT...`` (crates/poot-llm/src/bin/poot/embed.rs:1-80).

``similarity`` prints the cosine of each later text to the first; ``rerank`` ranks the documents after the query by
the cosine of their embeddings; ``cross`` ranks them by a cross-encoder's relevance logit."""
from __future__ import annotations

import sys
from typing import List

USAGE = "usage: poot embed {similarity|rerank|cross} [--backend auto|device|oracle] MODEL_DIR TEXT [TEXT ...]"


def _backend(argv: List[str]):
    """Strip ``--backend X`` (anywhere after the mode); ``auto`` is the device when one is present."""
    backend = "auto"
    rest = []
    i = 0
    while i < len(argv):
        if argv[i] == "--backend" and i + 1 < len(argv):
            backend = argv[i + 1]
            i += 2
            continue
        rest.append(argv[i])
        i += 1
    if backend not in ("auto", "device", "oracle"):
        raise ValueError(f"--backend {backend!r}: auto, device or oracle")
    if backend == "auto":
        import torch
        backend = "device" if torch.cuda.is_available() else "oracle"
    return backend, rest


def main_embed(argv: List[str], out=None) -> int:
    out = out or sys.stdout
    try:
        backend, argv = _backend(list(argv))
    except ValueError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    if len(argv) < 3 or argv[0] not in ("similarity", "rerank", "cross"):
        print(USAGE, file=sys.stderr)
        return 2
    mode, path, texts = argv[0], argv[1], argv[2:]
    from ..embed import Embedder, EmbedError
    try:
        emb = Embedder.load(path, backend=backend)
        if mode == "similarity":
            vec, _ = emb.embed(texts)
            print("pooling mean", file=out)
            for t, v in zip(texts[1:], vec[1:]):
                print(f"{float(v @ vec[0]):+.3f}  {t}", file=out)
            return 0
        if len(texts) < 2:
            print("error: a query and at least one document", file=sys.stderr)
            return 2
        if (mode == "cross") != bool(emb.cfg.labels):
            raise EmbedError("`cross` needs a cross-encoder checkpoint; `rerank` an embedding encoder")
        scores, _ = emb.rerank(texts[0], texts[1:])
        order = sorted(range(len(scores)), key=lambda i: (-float(scores[i]), i))
        for rank, i in enumerate(order):
            print(f"{rank + 1}. {float(scores[i]):+.3f}  {texts[1 + i]}", file=out)
        return 0
    except (EmbedError, FileNotFoundError, ValueError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
