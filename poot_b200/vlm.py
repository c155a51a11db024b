"""Vision-language generation: image frames through the vision tower, their rows in place of the image tokens'
embeddings, then ordinary decoding (crates/poot-llm/src/bin/poot/caption.rs:38-120; the front-end session of
crates/poot-models/src/multimodal/front_end.rs).

``VisionLLM.load(dir)`` opens an Idefics3 / SmolVLM checkpoint.  ``prepare`` turns a question and a decoded image into
prompt tokens and normalised frames; ``generate`` encodes the frames once and opens a sequence on the text driver
whose image-token positions carry the image rows (``Driver.open(..., embeds=)``), so chunked prefill, the paged K/V
cache, the prefix cache (keyed on the rows' content) and sampling are the ordinary ones.  ``backend="oracle"`` runs the
text stack on the host evaluator, ``backend="device"`` on the B200 engine; the vision tower is evaluated on the host
in both (one pass per image)."""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import numpy as np

from .driver.handle import ModelHandle
from .models.image_prep import (ImagePrep, QwenImagePrep, QwenImages, QwenVideoPrep, VideoClip, image_prompt, preprocess, qwen_preprocess,
                                qwen_preprocess_video, read_apng)
from .models.vision import QwenVisionTower, mrope_positions, patchify, position_ids, qwen_vision_inputs
from .oracle.eval import EvalOptions, eval_graph
from .driver.sampler import SamplingParams
from .oracle.runner import BLOCK, OracleSession
from .text.chat import render_chat
from .text.codec import StreamDecoder, load_tokenizer

# the template SmolVLM checkpoints ship, used when a checkpoint directory carries none
VLM_TEMPLATE = ("<|im_start|>{% for message in messages %}{{message['role'] | capitalize}}"
                "{% if message['content'][0]['type'] == 'image' %}{{':'}}{% else %}{{': '}}{% endif %}"
                "{% for line in message['content'] %}{% if line['type'] == 'text' %}{{line['text']}}"
                "{% elif line['type'] == 'image' %}{{ '<image>' }}{% endif %}{% endfor %}<end_of_utterance>\n{% endfor %}"
                "{% if add_generation_prompt %}{{ 'Assistant:' }}{% endif %}")


# Qwen2.5-VL's template: ChatML turns, an image part written as one padded placeholder between the vision markers
QWEN_VL_TEMPLATE = ("{% for message in messages %}{% if loop.first and message['role'] != 'system' %}<|im_start|>system\n"
                    "You are a helpful assistant.<|im_end|>\n{% endif %}<|im_start|>{{ message['role'] }}\n"
                    "{% if message['content'] is string %}{{ message['content'] }}{% else %}{% for part in message['content'] %}"
                    "{% if part['type'] == 'image' %}<|vision_start|><|image_pad|><|vision_end|>"
                    "{% elif part['type'] == 'video' %}<|vision_start|><|video_pad|><|vision_end|>"
                    "{% elif part['type'] == 'text' %}{{ part['text'] }}{% endif %}{% endfor %}{% endif %}<|im_end|>\n{% endfor %}"
                    "{% if add_generation_prompt %}<|im_start|>assistant\n{% endif %}")

VIDEO_TOKEN = "<|video_pad|>"
MAX_IMAGE_BYTES = 32 * 1024 * 1024
MAX_IMAGE_PIXELS = 64 * 1024 * 1024
MAX_VIDEO_BYTES = 64 * 1024 * 1024


def video_clip(src) -> VideoClip:
    """A video part's payload as a clip: a ``VideoClip``, a list of PIL frames (taken as one frame per second), the bytes
    of an animated PNG, or a ``data:image/apng;base64,`` (or ``image/png``) URL of one.  Nothing is fetched."""
    import base64
    import binascii
    if isinstance(src, VideoClip):
        return src
    if isinstance(src, (list, tuple)) and src:
        return VideoClip(list(src), 1.0, [float(i) for i in range(len(src))])
    if isinstance(src, (bytes, bytearray)):
        return read_apng(bytes(src))
    if not isinstance(src, str) or not src.startswith("data:"):
        raise ValueError("a video is a data: URL of an animated PNG (base64); remote URLs are not fetched")
    head, sep, payload = src[5:].partition(",")
    if not sep or not head.endswith(";base64") or head.split(";")[0] not in ("image/apng", "image/png", "video/apng"):
        raise ValueError("a video URL must be data:image/apng;base64,...")
    if len(payload) > MAX_VIDEO_BYTES * 4 // 3 + 4:
        raise ValueError("video payload exceeds the size limit")
    try:
        raw = base64.b64decode(payload, validate=True)
    except (binascii.Error, ValueError):
        raise ValueError("video payload is not valid base64") from None
    return read_apng(raw)


def image_from_data_url(url):
    """Decode a ``data:image/...;base64,`` URL into a PIL image; anything else (a remote URL, an oversized or
    undecodable payload) is a ``ValueError``."""
    import base64
    import binascii
    import io
    if not isinstance(url, str) or not url.startswith("data:"):
        raise ValueError("image_url must be a data: URL (base64); remote URLs are not fetched")
    head, sep, payload = url[5:].partition(",")
    if not sep or not head.endswith(";base64"):
        raise ValueError("image_url must be base64-encoded (data:image/png;base64,...)")
    if len(payload) > MAX_IMAGE_BYTES * 4 // 3 + 4:
        raise ValueError("image payload exceeds the size limit")
    try:
        raw = base64.b64decode(payload, validate=True)
    except (binascii.Error, ValueError):
        raise ValueError("image payload is not valid base64") from None
    from PIL import Image
    try:
        img = Image.open(io.BytesIO(raw))
        if img.size[0] * img.size[1] > MAX_IMAGE_PIXELS:
            raise ValueError("image exceeds the pixel limit")
        img.load()
    except ValueError:
        raise
    except Exception as e:
        raise ValueError(f"image payload does not decode: {e}") from None
    return img


class NotVisionModel(ValueError):
    """The checkpoint's family has no vision front end."""


class VisionLLM:
    def __init__(self, handle: ModelHandle, tokenizer=None, template: Optional[str] = None, llm=None):
        if getattr(handle.model, "kind", "decoder") != "vlm":
            raise NotVisionModel("the checkpoint is not a vision-language model: its family has no front end")
        self.handle, self.model = handle, handle.model
        self.vision = self.model.vision
        self.vision_weights = {n: w.to_f32() for n, w in handle.canonical.items() if n.startswith("vision.")}
        self._weights = None
        self.tokenizer, self.template = tokenizer, template
        self.llm = llm                                # text driver (None: a bare oracle session per call)
        self.qwen = isinstance(self.vision, QwenVisionTower)      # sectioned rotary positions, patches of any grid
        if self.qwen:
            vc = self.vision.cfg
            self.prep = QwenImagePrep.from_dir(handle.source, vc.patch, vc.merge, vc.temporal)
            self.video_prep = QwenVideoPrep.from_dir(handle.source, vc.patch, vc.merge)
        else:
            self.prep = ImagePrep.from_dir(handle.source, self.vision.cfg.image_size)
        self._towers = {}
        self.vision_engine = None                     # device program of the tower (runtime/vision_engine.py); None: host evaluator
        self.rope_delta = 0                           # rotary position minus sequence index after the last prefilled prompt
        self.eos: List[int] = []                      # end tokens of generation_config.json, beside the tokenizer's

    @staticmethod
    def load(path: str, backend: str = "oracle", device="cuda", rows: int = 4, max_seq: int = 8192,
             prefill_chunk: int = 256, num_blocks: Optional[int] = None) -> "VisionLLM":
        """``max_seq`` / ``prefill_chunk`` default to the reference's caption window (8192 positions, pieces of 256)."""
        import json
        import os
        from .llm import LLM
        if backend == "oracle":
            llm = LLM.oracle(path, rows=rows, max_seq=max_seq, num_blocks=num_blocks or (rows * max_seq // BLOCK),
                             prefill_chunk=prefill_chunk)
        elif backend == "device":
            llm = LLM.load(path, device=device, rows=rows, max_seq=max_seq, prefill_chunk=prefill_chunk, num_blocks=num_blocks)
        else:
            raise ValueError(f"backend {backend!r}: oracle or device")
        handle = llm.handle
        tok, template = None, None
        if os.path.exists(os.path.join(path, "tokenizer.json")):
            tok = load_tokenizer(handle)
        for name, key in (("chat_template.json", "chat_template"), ("tokenizer_config.json", "chat_template")):
            f = os.path.join(path, name)
            if template is None and os.path.exists(f):
                with open(f) as fh:
                    template = json.load(fh).get(key)
        f = os.path.join(path, "chat_template.jinja")
        if template is None and os.path.exists(f):
            with open(f) as fh:
                template = fh.read()
        vlm = VisionLLM(handle, tok, template, llm)
        if backend == "device" and not vlm.qwen:
            vlm.tower_to_device(device)
        f = os.path.join(path, "generation_config.json")
        if os.path.exists(f):
            with open(f) as fh:
                e = json.load(fh).get("eos_token_id")
            vlm.eos = [int(x) for x in (e if isinstance(e, list) else [e]) if x is not None]
        return vlm

    def tower_to_device(self, device="cuda", max_frames: int = 17) -> bool:
        """Run the vision tower on the device engine when its head width allows it; otherwise it stays on the host."""
        import torch
        from .runtime.vision_engine import VisionEngine
        try:
            tensors = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in self.vision_weights.items()}
            self.vision_engine = VisionEngine(self.vision.cfg, tensors, device, max_frames)
        except ValueError:
            self.vision_engine = None
        return self.vision_engine is not None

    @property
    def weights(self):
        """Every weight in f32 for bare oracle sessions (decoded on first use; the served paths never need it)."""
        if self._weights is None:
            self._weights = self.handle.oracle_weights()
        return self._weights

    # ---- vision tower ----------------------------------------------------------------------------------------------
    def encode_images(self, pixels: np.ndarray) -> np.ndarray:
        """``pixels[frames, C, S, S]`` (normalised) -> ``[frames * rows_per_image, text_hidden]``; for Qwen2.5-VL the
        flattened patches and grids of ``QwenImages`` -> one row per merged cell."""
        c = self.vision.cfg
        if self.qwen:
            n = pixels.patches.shape[0]
            if n not in self._towers:
                self._towers[n] = self.vision.trace(n)
            g = self._towers[n]
            inputs = {"patches": np.asarray(pixels.patches, dtype=np.float32), **qwen_vision_inputs(c, pixels.grids)}
            for i in g.inputs:
                if i.storage == "const":
                    inputs[i.name] = self.vision_weights[i.name]
            return eval_graph(g, inputs, EvalOptions(matmul_precision="exact")).outputs["image_rows"]
        pixels = np.asarray(pixels, dtype=np.float32)
        n, ch, h, w = pixels.shape
        if (ch, h, w) != (c.channels, c.image_size, c.image_size):
            raise ValueError(f"frames of {(ch, h, w)}; the tower takes {(c.channels, c.image_size, c.image_size)}")
        if self.vision_engine is not None and n <= self.vision_engine.max_frames:
            return self.vision_engine.forward(pixels).float().cpu().numpy()
        if n not in self._towers:
            self._towers[n] = self.vision.trace(n)
        g = self._towers[n]
        inputs = {"patches": patchify(pixels, c.patch),
                  "pos_ids": np.tile(position_ids(c, c.per_side, c.per_side)[None, :], (n, 1))}
        for i in g.inputs:
            if i.storage == "const":
                inputs[i.name] = self.vision_weights[i.name]
        return eval_graph(g, inputs, EvalOptions(matmul_precision="exact")).outputs["image_rows"]

    # ---- prompt ----------------------------------------------------------------------------------------------------
    def prepare(self, question: str, image) -> tuple:
        """``(prompt tokens, frames)`` for one user turn holding ``image`` (a PIL image) and ``question``."""
        part = {"type": "video", "video": image} if isinstance(image, VideoClip) else {"type": "image", "image": image}
        return self.prepare_messages([{"role": "user", "content": [part, {"type": "text", "text": question}]}])

    def prepare_messages(self, messages: List[dict], template: Optional[str] = None) -> tuple:
        """Chat messages whose contents hold image parts -> ``(prompt tokens, frames of every image in order)``.
        An image part is ``{"type": "image_url", "image_url": {"url": "data:image/...;base64,..."}}`` (or ``{"type":
        "image", "image": <PIL image>}``); only ``data:`` URLs are read (the server fetches nothing)."""
        if self.tokenizer is None:
            raise ValueError("the checkpoint directory has no tokenizer.json")
        images, shaped = [], []
        for m in messages:
            c = m.get("content") if isinstance(m, dict) else None
            if isinstance(c, str):
                shaped.append({**m, "content": [{"type": "text", "text": c}]})
                continue
            parts = []
            for part in c or []:
                kind = part.get("type") if isinstance(part, dict) else None
                if kind == "text":
                    parts.append({"type": "text", "text": str(part.get("text", ""))})
                elif kind == "image_url":
                    images.append(image_from_data_url((part.get("image_url") or {}).get("url")))
                    parts.append({"type": "image"})
                elif kind == "image":
                    images.append(part.get("image"))
                    parts.append({"type": "image"})
                elif kind in ("video", "video_url") and self.qwen:
                    images.append(video_clip(part.get("video") if kind == "video" else (part.get("video_url") or {}).get("url")))
                    parts.append({"type": "video"})
                else:
                    raise ValueError(f"content part of type {kind!r}: text and image_url parts are read" +
                                     (", and video / video_url parts (an animated PNG)" if self.qwen else ""))
            shaped.append({**m, "content": parts})
        default = QWEN_VL_TEMPLATE if self.qwen else VLM_TEMPLATE
        text = render_chat(shaped, template or self.template or default, family=self.handle.cfg.family, keep_parts=True)
        import re
        marks = [self.prep.image_token] + ([VIDEO_TOKEN] if self.qwen else [])
        cut = re.split("(" + "|".join(re.escape(t) for t in marks) + ")", text)
        pieces, written = cut[0::2], cut[1::2]
        if len(pieces) != len(images) + 1:
            raise ValueError(f"the template wrote {len(pieces) - 1} image placeholders for {len(images)} images")
        out, frames, grids, seconds = pieces[0], [], [], []
        for img, mark, tail in zip(images, written, pieces[1:]):
            if self.qwen:
                if isinstance(img, VideoClip) != (mark == VIDEO_TOKEN):
                    raise ValueError("the template wrote an image placeholder for a video part (or the reverse)")
                if isinstance(img, VideoClip):
                    one, sec = qwen_preprocess_video(img, self.prep, self.video_prep)
                else:
                    one, sec = qwen_preprocess(img, self.prep), None
                frames.append(one.patches)
                grids += one.grids
                seconds.append(sec)
                out += mark * one.rows(self.vision.cfg.merge)[0] + tail
            else:
                fr = preprocess(img, self.prep)
                frames.append(fr.pixels)
                out += image_prompt(self.prep, fr.rows, fr.cols, self.vision.cfg.rows_per_image) + tail
        pixels = np.concatenate(frames, 0) if frames else None
        if self.qwen and frames:
            pixels = QwenImages(pixels, grids, seconds if any(x is not None for x in seconds) else None)
        return self.tokenizer.encode(out, add_bos=False), pixels

    # ---- generation ------------------------------------------------------------------------------------------------
    def _session(self, length: int) -> OracleSession:
        cap = -(-length // BLOCK) * BLOCK
        return OracleSession(self.model, self.weights, rows=1, capacity=cap, paged=True)

    def prefill(self, sess: OracleSession, tokens: Sequence[int], pixels: Optional[np.ndarray]) -> np.ndarray:
        """Feed the whole prompt; returns the last position's logits ``[1, vocab]``."""
        toks = np.asarray(tokens, dtype=np.int32).reshape(1, -1)
        flags = self._media(toks[0]).astype(np.int32)
        none = pixels is None or (not self.qwen and len(pixels) == 0)
        rope = None
        if self.qwen:
            # three rotary streams per token; the decode steps after this prompt continue at ``index + rope_delta``
            rope = self._mrope(toks[0], None if none else pixels)
            self.rope_delta = int(rope.max()) + 1 - toks.shape[1]
        if none:
            if flags.any():
                raise ValueError("the prompt holds image tokens but no image was given")
            return sess.step(toks, rope_positions=rope)
        rows = self.encode_images(pixels)
        if int(flags.sum()) != rows.shape[0]:
            raise ValueError(f"the prompt holds {int(flags.sum())} image tokens; the frames give {rows.shape[0]} rows")
        full = np.zeros((toks.shape[1], rows.shape[1]), dtype=np.float32)
        full[flags.astype(bool)] = rows
        return sess.step(toks, embed_rows=full, embed_flags=flags, rope_positions=rope)

    def image_inputs(self, tokens: Sequence[int], pixels: Optional[np.ndarray]):
        """``(positions, rows)`` for ``Driver.open(..., embeds=)``: the prompt's image-token positions and the rows the
        frames give, checked to agree in number."""
        toks = np.asarray(tokens, dtype=np.int64).reshape(-1)
        at = np.nonzero(self._media(toks))[0]
        if pixels is None or (not self.qwen and len(pixels) == 0):
            if len(at):
                raise ValueError("the prompt holds image tokens but no image was given")
            return None
        rows = self.encode_images(pixels)
        if len(at) != rows.shape[0]:
            raise ValueError(f"the prompt holds {len(at)} image tokens; the frames give {rows.shape[0]} rows")
        return at, rows

    def rope_inputs(self, tokens: Sequence[int], pixels) -> Optional[np.ndarray]:
        """Rotary position streams ``[3, len(tokens)]`` for ``Driver.open(..., rope_positions=)`` under a sectioned rope
        (``None`` for families with one position per token)."""
        if not self.qwen:
            return None
        return self._mrope(np.asarray(tokens).reshape(-1), pixels)

    def _media(self, toks: np.ndarray) -> np.ndarray:
        """Which prompt positions take a row of the vision tower: image placeholders and, for Qwen, video placeholders."""
        at = toks == self.model.image_token
        if self.qwen and self.vision.cfg.video_token >= 0:
            at = at | (toks == self.vision.cfg.video_token)
        return at

    def _mrope(self, toks: np.ndarray, pixels) -> np.ndarray:
        c = self.vision.cfg
        grids = [] if pixels is None else pixels.grids
        return mrope_positions(toks, self.model.image_token, grids, c.merge, video_token=c.video_token if c.video_token >= 0 else None,
                               seconds_per_step=None if pixels is None else pixels.seconds, tokens_per_second=c.tokens_per_second)

    def generate(self, tokens: Sequence[int], pixels: Optional[np.ndarray], max_new: int = 64,
                 eos: Optional[Sequence[int]] = None, on_token: Optional[Callable[[int], None]] = None) -> List[int]:
        """Greedy continuation of ``tokens`` (which hold one image token per image row); stops before a token of ``eos``."""
        stop = set(eos or ())
        if self.llm is None:
            sess = self._session(len(tokens) + max_new)
            logits = self.prefill(sess, tokens, pixels)
            out: List[int] = []
            for i in range(max_new):
                tok = int(np.argmax(logits[0]))
                if tok in stop:
                    break
                out.append(tok)
                if on_token is not None:
                    on_token(tok)
                if i + 1 < max_new:
                    rope = np.full((3, 1), sess.length + self.rope_delta, np.int32) if self.qwen else None
                    logits = sess.step(np.array([[tok]], dtype=np.int32), rope_positions=rope)
            return out
        drv = self.llm.driver
        params = SamplingParams(temperature=0.0, max_tokens=max_new, ignore_eos=True)
        sid = drv.open(list(tokens), params, embeds=self.image_inputs(tokens, pixels),
                       rope_positions=self.rope_inputs(tokens, pixels))
        out = []
        try:
            while len(out) < max_new:
                res = [r for r in drv.step([sid]) if r.seq_id == sid]
                if not res:
                    break
                if res[0].token is None:
                    continue
                tok = int(res[0].token)
                if tok in stop:
                    break
                drv.commit(sid, [tok])
                out.append(tok)
                if on_token is not None:
                    on_token(tok)
        finally:
            drv.release(sid)
        return out

    def caption(self, image, question: str = "Can you describe this image?", max_new: int = 64,
                on_piece: Optional[Callable[[str], None]] = None) -> str:
        tokens, pixels = self.prepare(question, image)
        dec = StreamDecoder(self.tokenizer)
        pieces: List[str] = []

        def emit(tok: int):
            piece = dec.push(tok)
            if piece:
                pieces.append(piece)
                if on_piece is not None:
                    on_piece(piece)
        eos = [t for t in (getattr(self.tokenizer, "eos", None), self.handle.cfg.eos_token, *self.eos) if t is not None]
        self.generate(tokens, pixels, max_new, eos, emit)
        tail = dec.flush()
        if tail:
            pieces.append(tail)
            if on_piece is not None:
                on_piece(tail)
        return "".join(pieces)
