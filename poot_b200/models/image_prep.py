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
from typing import List, Optional, Tuple

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


# ---- Qwen2.5-VL ----------------------------------------------------------------------------------------------------
CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


@dataclass
class QwenImagePrep:
    """Preprocessing of the Qwen2.5-VL front end (crates/poot-models/src/multimodal/qwen_vl/processor): resize both
    edges to multiples of ``patch * merge`` within a pixel budget (bicubic), normalise, and lay the pixels out as one
    row per ``temporal x patch x patch`` patch in (frame, merged row, merged column, row in cell, column in cell) order."""
    patch: int = 14
    merge: int = 2
    temporal: int = 2
    min_pixels: int = 56 * 56
    max_pixels: int = 28 * 28 * 1280
    rescale: float = 1.0 / 255.0
    mean: Tuple[float, ...] = CLIP_MEAN
    std: Tuple[float, ...] = CLIP_STD
    image_token: str = "<|image_pad|>"

    @staticmethod
    def from_dir(path: str, patch: int, merge: int, temporal: int) -> "QwenImagePrep":
        p = QwenImagePrep(patch=patch, merge=merge, temporal=temporal, min_pixels=(2 * patch * merge) ** 2,
                          max_pixels=(patch * merge) ** 2 * 1280)
        f = os.path.join(path, "preprocessor_config.json")
        if os.path.exists(f):
            with open(f) as fh:
                c = json.load(fh)
            size = c.get("size") or {}
            p.min_pixels = int(c.get("min_pixels") or size.get("shortest_edge") or p.min_pixels)
            p.max_pixels = int(c.get("max_pixels") or size.get("longest_edge") or p.max_pixels)
            p.rescale = float(c.get("rescale_factor", p.rescale))
            p.mean = tuple(c.get("image_mean", p.mean))
            p.std = tuple(c.get("image_std", p.std))
            for key, want in (("patch_size", patch), ("merge_size", merge), ("temporal_patch_size", temporal)):
                if key in c and int(c[key]) != want:
                    raise ValueError(f"preprocessor {key} {c[key]} does not fit the vision tower's {want}")
        return p


def smart_resize(h: int, w: int, factor: int, min_pixels: int, max_pixels: int) -> Tuple[int, int]:
    """``(height, width)``: both multiples of ``factor``, the area inside ``[min_pixels, max_pixels]``, aspect kept as
    closely as that allows."""
    if max(h, w) / min(h, w) > 200:
        raise ValueError(f"aspect ratio of a {h}x{w} image exceeds 200")
    hb, wb = round(h / factor) * factor, round(w / factor) * factor
    if hb * wb > max_pixels:
        beta = math.sqrt(h * w / max_pixels)
        hb = max(factor, math.floor(h / beta / factor) * factor)
        wb = max(factor, math.floor(w / beta / factor) * factor)
    elif hb * wb < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        hb, wb = math.ceil(h * beta / factor) * factor, math.ceil(w * beta / factor) * factor
    return hb, wb


@dataclass
class QwenImages:
    patches: np.ndarray                 # [sum t*h*w, C * temporal * patch * patch] f32
    grids: List[Tuple[int, int, int]]   # (t, h, w) patches of every image or video, in prompt order
    seconds: Optional[List[Optional[float]]] = None   # per grid: seconds one temporal step covers (None: a still image)

    def rows(self, merge: int) -> List[int]:
        return [t * h * w // (merge * merge) for t, h, w in self.grids]


def qwen_preprocess(img, prep: QwenImagePrep) -> QwenImages:
    """One still image (a PIL image): a single temporal step made of ``temporal`` copies of the frame."""
    from PIL import Image
    img = img.convert("RGB")
    w, h = img.size
    hb, wb = smart_resize(h, w, prep.patch * prep.merge, prep.min_pixels, prep.max_pixels)
    img = img.resize((wb, hb), Image.BICUBIC)
    a = np.asarray(img, dtype=np.float32).transpose(2, 0, 1) * np.float32(prep.rescale)
    a = (a - np.asarray(prep.mean, np.float32)[:, None, None]) / np.asarray(prep.std, np.float32)[:, None, None]
    p, m, tp = prep.patch, prep.merge, prep.temporal
    gh, gw = hb // p, wb // p
    x = np.broadcast_to(a[None], (tp, 3, hb, wb)).reshape(1, tp, 3, gh // m, m, p, gw // m, m, p)
    x = x.transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)
    return QwenImages(np.ascontiguousarray(x).reshape(gh * gw, 3 * tp * p * p), [(1, gh, gw)])


# ---- Qwen2.5-VL video ----------------------------------------------------------------------------------------------
MAX_VIDEO_FRAMES = 16 * 1024


@dataclass
class VideoClip:
    """Decoded frames of one clip with what frame sampling needs to know about the source."""
    frames: list                         # PIL images, source order
    fps: float                           # average source rate: frames / duration
    timestamps: List[float] = field(default_factory=list)    # start of each frame in seconds


@dataclass
class QwenVideoPrep:
    """Frame sampling and per-frame pixel budget of the video half of the processor (crates/poot-models/src/multimodal/
    qwen_vl/processor/video_sampling.rs, preprocess.rs): frames are taken uniformly at ``fps`` per second of source,
    between ``min_frames`` and ``max_frames`` and a whole number of temporal steps."""
    fps: float = 2.0
    min_frames: int = 4
    max_frames: int = 768
    min_pixels: int = 128 * 28 * 28
    max_pixels: int = 768 * 28 * 28

    @staticmethod
    def from_dir(path: str, patch: int, merge: int) -> "QwenVideoPrep":
        """Defaults scaled to the tower's merged cell, overridden by ``video_preprocessor_config.json`` where the
        checkpoint directory has one."""
        p = QwenVideoPrep(min_pixels=128 * (patch * merge) ** 2, max_pixels=768 * (patch * merge) ** 2)
        f = os.path.join(path, "video_preprocessor_config.json")
        if os.path.exists(f):
            with open(f) as fh:
                c = json.load(fh)
            size = c.get("size") or {}
            p.min_pixels = int(c.get("min_pixels") or size.get("shortest_edge") or p.min_pixels)
            p.max_pixels = int(c.get("max_pixels") or size.get("longest_edge") or p.max_pixels)
            p.fps = float(c.get("fps") or p.fps)
            p.min_frames, p.max_frames = int(c.get("min_frames") or p.min_frames), int(c.get("max_frames") or p.max_frames)
        if not (p.fps > 0 and 0 < p.min_frames <= p.max_frames and 0 < p.min_pixels <= p.max_pixels):
            raise ValueError(f"video preprocessing limits do not make sense: {p}")
        return p


def sample_video_frames(n_frames: int, source_fps: float, prep: QwenVideoPrep, temporal: int = 2) -> List[int]:
    """Indices of the frames the processor keeps: ``n_frames / source_fps * fps`` of them, clamped to ``[min_frames,
    max_frames]`` and to the clip's length, rounded down to whole temporal steps, spaced uniformly from frame 0."""
    if n_frames <= 0:
        raise ValueError("a video must hold at least one frame")
    if n_frames > MAX_VIDEO_FRAMES:
        raise ValueError(f"a video of {n_frames} frames; at most {MAX_VIDEO_FRAMES} are read")
    if not (math.isfinite(source_fps) and source_fps > 0):
        raise ValueError(f"source frame rate must be positive and finite, got {source_fps}")
    want = n_frames / source_fps * prep.fps
    want = min(min(max(want, prep.min_frames), prep.max_frames), n_frames)
    want = int(math.floor(want / temporal) * temporal)
    if want <= 0:                        # a clip shorter than one temporal step: every frame, padded by the caller
        return list(range(n_frames))
    return [int(x) for x in np.arange(0, n_frames, n_frames / want).astype(np.int64)[:want]]


def qwen_preprocess_video(clip: VideoClip, prep: QwenImagePrep, video: Optional[QwenVideoPrep] = None):
    """``(QwenImages with one (t, h, w) grid, seconds one temporal step covers)`` for one clip: sample, resize every kept
    frame to one size within the per-frame pixel budget, normalise, and lay ``temporal`` consecutive frames into each
    patch row (an odd tail repeats the last frame)."""
    from PIL import Image
    video = video or QwenVideoPrep()
    keep = sample_video_frames(len(clip.frames), clip.fps, video, prep.temporal)
    frames = [clip.frames[i].convert("RGB") for i in keep]
    while len(frames) % prep.temporal:
        frames.append(frames[-1])
    w, h = frames[0].size
    if any(f.size != (w, h) for f in frames):
        raise ValueError("the frames of one video differ in size")
    hb, wb = smart_resize(h, w, prep.patch * prep.merge, video.min_pixels, video.max_pixels)
    mean, std = np.asarray(prep.mean, np.float32)[:, None, None], np.asarray(prep.std, np.float32)[:, None, None]
    a = np.stack([(np.asarray(f.resize((wb, hb), Image.BICUBIC), dtype=np.float32).transpose(2, 0, 1) * np.float32(prep.rescale) - mean) / std
                  for f in frames])
    p, m, tp = prep.patch, prep.merge, prep.temporal
    gt, gh, gw = len(frames) // tp, hb // p, wb // p
    x = a.reshape(gt, tp, 3, gh // m, m, p, gw // m, m, p).transpose(0, 3, 6, 4, 7, 2, 1, 5, 8)
    # the rate the kept frames stand for: kept frames over the clip's duration
    sampled_fps = len(keep) / (len(clip.frames) / clip.fps)
    return QwenImages(np.ascontiguousarray(x).reshape(gt * gh * gw, 3 * tp * p * p), [(gt, gh, gw)]), prep.temporal / sampled_fps


def read_apng(data: bytes, max_pixels: int = 32 * 1024 * 1024) -> VideoClip:
    """An animated PNG as a clip (crates/poot-llm/src/multimodal/apng.rs): one animation cycle, every frame composed onto
    the canvas, the frame delays kept as timestamps; the source rate is frames over duration.  A still PNG is a
    one-frame clip at one frame per second."""
    import io
    from PIL import Image, ImageSequence
    img = Image.open(io.BytesIO(data))
    if img.format != "PNG":
        raise ValueError(f"a video is read from an animated PNG, not {img.format}")
    n = int(getattr(img, "n_frames", 1))
    if n > MAX_VIDEO_FRAMES or n * img.size[0] * img.size[1] > max_pixels:
        raise ValueError(f"an animation of {n} frames of {img.size[0]}x{img.size[1]} is over the decode budget")
    frames, stamps, t = [], [], 0.0
    for f in ImageSequence.Iterator(img):
        frames.append(f.convert("RGB").copy())
        stamps.append(t)
        t += float(f.info.get("duration", 0.0) or 0.0) / 1000.0
    if t <= 0.0:
        t = float(len(frames))           # no delays stated: one frame per second
        stamps = [float(i) for i in range(len(frames))]
    return VideoClip(frames, len(frames) / t, stamps)
