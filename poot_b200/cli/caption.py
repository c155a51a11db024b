"""``caption MODEL_DIR IMAGE [QUESTION]``: caption an image with a vision-language checkpoint
(crates/poot-llm/src/bin/poot/caption.rs:26-37: positional checkpoint directory, image file and question, 64 greedy
tokens streamed to stdout; ``--backend`` picks the text stack's executor as the reference's device flags do).  The
image is decoded with Pillow; an animated file contributes its first frame."""
from __future__ import annotations

import argparse
import sys
from typing import List

DEFAULT_QUESTION = "Can you describe this image?"
MAX_NEW = 64


class _Strict(argparse.ArgumentParser):
    def error(self, message):
        raise ValueError(message)


def parse_caption(argv: List[str]) -> argparse.Namespace:
    p = _Strict(prog="poot caption", allow_abbrev=False)
    p.add_argument("model_dir")
    p.add_argument("image")
    p.add_argument("question", nargs="?", default=DEFAULT_QUESTION)
    p.add_argument("-n", "--predict", type=int, default=MAX_NEW)
    p.add_argument("--backend", default="auto", choices=("auto", "device", "oracle"))
    p.add_argument("-c", "--ctx-size", type=int, default=0, help="text window (0: 8192 on the device, 2048 on the oracle)")
    a = p.parse_args(argv)
    if a.predict <= 0:
        raise ValueError("--predict must be positive")
    if a.ctx_size < 0:
        raise ValueError("--ctx-size must not be negative")
    return a


def main_caption(argv: List[str]) -> int:
    try:
        args = parse_caption(argv)
    except ValueError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    from ..models.registry import UnsupportedFamily
    from ..vlm import NotVisionModel, VisionLLM
    try:
        from PIL import Image
        image = Image.open(args.image)
        if getattr(image, "n_frames", 1) > 1 and image.format == "PNG":
            # an animated PNG is a clip: the front end samples its frames (families without a video path refuse it)
            from ..models.image_prep import read_apng
            with open(args.image, "rb") as fh:
                image = read_apng(fh.read())
        else:
            image.load()
    except Exception as e:                                  # unreadable or undecodable file
        print(f"error: decode {args.image}: {e}", file=sys.stderr)
        return 1
    backend = args.backend
    if backend == "auto":
        import torch
        backend = "device" if torch.cuda.is_available() else "oracle"
    ctx = args.ctx_size or (8192 if backend == "device" else 2048)
    try:
        vlm = VisionLLM.load(args.model_dir, backend=backend, rows=1, max_seq=ctx)
    except (NotVisionModel, UnsupportedFamily, FileNotFoundError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    print(f"loaded {args.image}; model from {args.model_dir}", file=sys.stderr)

    def piece(text: str):
        sys.stdout.write(text)
        sys.stdout.flush()
    vlm.caption(image, args.question, args.predict, piece)
    sys.stdout.write("\n")
    return 0
