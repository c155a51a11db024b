"""Image preprocessing of the Idefics3 / SmolVLM front end: a decoded RGB image -> the channel-first square frames the
vision tower encodes, and the prompt text that stands for them
(crates/poot-models/src/multimodal/idefics3/preprocess.rs:1-30, 215-260; front.rs prompt expansion).

The pipeline follows the checkpoint's processor: scale the longest edge to ``longest_edge`` (even other edge, Lanczos),
round both edges up to multiples of the tower's ``tile``, cut ``rows x cols`` tiles row-major and append the whole
image resized to one tile (the "global" frame); an image no larger than one tile is a single frame.  Each frame is
rescaled and normalised per channel.  In the prompt every frame becomes ``rows_per_image`` image tokens behind a marker
naming its grid cell."""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import List, Tuple

import numpy as np

MAX_IMAGE_SIZE = 4096          # the longest-edge resize never exceeds this


@dataclass
class ImagePrep:
    longest_edge: int = 4 * 364
    tile: int = 364
    split: bool = True
    rescale: float = 1.0 / 255.0
    mean: Tuple[float, ...] = (0.5, 0.5, 0.5)
    std: Tuple[float, ...] = (0.5, 0.5, 0.5)
    fake_token: str = "<fake_token_around_image>"
    image_token: str = "<image>"
    global_token: str = "<global-img>"

    @staticmethod
    def from_dir(path: str, tile: int) -> "ImagePrep":
        """Read ``preprocessor_config.json`` beside the checkpoint; a missing file keeps the defaults at ``tile``."""
        p = ImagePrep(longest_edge=4 * tile, tile=tile)
        f = os.path.join(path, "preprocessor_config.json")
        if os.path.exists(f):
            with open(f) as fh:
                c = json.load(fh)
            p.longest_edge = int((c.get("size") or {}).get("longest_edge", p.longest_edge))
            p.tile = int((c.get("max_image_size") or {}).get("longest_edge", tile))
            p.split = bool(c.get("do_image_splitting", True))
            p.rescale = float(c.get("rescale_factor", p.rescale))
            p.mean = tuple(c.get("image_mean", p.mean))
            p.std = tuple(c.get("image_std", p.std))
        if p.tile != tile:
            raise ValueError(f"preprocessor tiles of {p.tile} pixels do not fit a vision tower of {tile}")
        return p


def resize_longest(h: int, w: int, longest: int) -> Tuple[int, int]:
    """``(height, width)`` with the longest edge at ``longest``, aspect kept, the other edge rounded up to even."""
    aspect = w / h
    if w >= h:
        w2 = longest
        h2 = int(w2 / aspect)
        h2 += h2 % 2
    else:
        h2 = longest
        w2 = int(h2 * aspect)
        w2 += w2 % 2
    h2, w2 = max(h2, 1), max(w2, 1)
    if w2 >= h2 and w2 > MAX_IMAGE_SIZE:
        w2, h2 = MAX_IMAGE_SIZE, int(MAX_IMAGE_SIZE / aspect)
    elif h2 > w2 and h2 > MAX_IMAGE_SIZE:
        h2, w2 = MAX_IMAGE_SIZE, int(MAX_IMAGE_SIZE * aspect)
    return max(h2, 1), max(w2, 1)


def resize_for_encoder(h: int, w: int, tile: int) -> Tuple[int, int]:
    """Round each edge up to a multiple of ``tile``, the short one following the long one's aspect."""
    aspect = w / h
    if w >= h:
        w = math.ceil(w / tile) * tile
        h = math.ceil(int(w / aspect) / tile) * tile
    else:
        h = math.ceil(h / tile) * tile
        w = math.ceil(int(h * aspect) / tile) * tile
    return h, w


def split_geometry(h: int, w: int, tile: int) -> Tuple[int, int]:
    """``(rows, cols)`` of tiles; ``(0, 0)`` when the image fits one tile and is not split."""
    if h > tile or w > tile:
        return math.ceil(h / tile), math.ceil(w / tile)
    return 0, 0


@dataclass
class Frames:
    pixels: np.ndarray                     # [frames, 3, tile, tile] f32, tiles row-major then the global frame
    rows: int = 0
    cols: int = 0


def _resized(img, h: int, w: int):
    from PIL import Image
    return img.resize((w, h), Image.LANCZOS)


def preprocess(img, prep: ImagePrep) -> Frames:
    """``img`` is a PIL image (any mode; converted to RGB)."""
    img = img.convert("RGB")
    w, h = img.size
    h, w = resize_longest(h, w, prep.longest_edge)
    img = _resized(img, h, w)
    frames, rows, cols = [], 0, 0
    if prep.split:
        h, w = resize_for_encoder(h, w, prep.tile)
        img = _resized(img, h, w)
        rows, cols = split_geometry(h, w, prep.tile)
        if rows:
            th, tw = math.ceil(h / rows), math.ceil(w / cols)
            for r in range(rows):
                for c in range(cols):
                    box = (c * tw, r * th, min((c + 1) * tw, w), min((r + 1) * th, h))
                    frames.append(img.crop(box))
            frames.append(_resized(img, prep.tile, prep.tile))
        else:
            frames.append(img)
    else:
        frames.append(_resized(img, prep.tile, prep.tile))
    out = np.zeros((len(frames), 3, prep.tile, prep.tile), dtype=np.float32)
    mean = np.asarray(prep.mean, dtype=np.float32)[:, None, None]
    std = np.asarray(prep.std, dtype=np.float32)[:, None, None]
    for i, f in enumerate(frames):
        if f.size != (prep.tile, prep.tile):
            f = _resized(f, prep.tile, prep.tile)
        a = np.asarray(f, dtype=np.float32).transpose(2, 0, 1)
        out[i] = (a * np.float32(prep.rescale) - mean) / std
    return Frames(out, rows, cols)


def image_prompt(prep: ImagePrep, rows: int, cols: int, rows_per_image: int) -> str:
    """The text one image becomes: per tile a marker, its grid-cell name and ``rows_per_image`` image tokens; the
    global frame last."""
    run = prep.image_token * rows_per_image
    if rows == 0 and cols == 0:
        return f"{prep.fake_token}{prep.global_token}{run}{prep.fake_token}"
    text = ""
    for r in range(rows):
        for c in range(cols):
            text += f"{prep.fake_token}<row_{r + 1}_col_{c + 1}>{run}"
        text += "\n"
    return text + f"\n{prep.fake_token}{prep.global_token}{run}{prep.fake_token}"
