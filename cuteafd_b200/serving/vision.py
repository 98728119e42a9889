"""Image inputs of chat requests: content parts -> placeholder tokens in the prompt + the vision tower's rows for them.

A message's content may be a list of parts; image parts come as OpenAI `{"type": "image_url", "image_url": {"url": "data:..."}}`
(also `input_image` of the Responses surface) or Anthropic `{"type": "image", "source": {"type": "base64", "data": ...}}`.
`VisionFrontEnd.prepare` pulls the images out in order, leaves a marker in the text, renders the prompt with the server's chat
template, tokenises the text between the markers and writes `start, pad x n, end` token ids where each image was (n = rows the tower
emits for that image), then runs the tower once over all images of the request.  The scheduler's request carries the prompt
positions of the pad tokens and the rows; the runner scatters them over the embeddings of the prefill chunks that hold them.
Requests with images bypass the prefix cache (the placeholder ids do not identify the image).

Reference: rust/crates/cuteafd-daemon/src/shared/vision.rs (encoder owner), families/deepseek_v41/v41_requests.rs (images in the
admission identity), native/families/deepseek_v41/cuda/v41_vision.cu (`span_kernel`: start / newline / end rows around the features).
"""
from __future__ import annotations

import base64
import threading

IMAGE_MARK = "\u0001<image>\u0001"


def _audio_payload(part: dict):
    """Bytes of an audio content part (OpenAI `input_audio`: base64 WAV); None for other parts."""
    if part.get("type") != "input_audio":
        return None
    a = part.get("input_audio") or {}
    if not isinstance(a.get("data"), str) or a.get("format", "wav") != "wav":
        raise ValueError("audio parts carry base64 WAV data")
    return base64.b64decode(a["data"])


def _image_payload(part: dict):
    """Bytes (or a data: URI string) of an image content part; None for other parts."""
    kind = part.get("type")
    if kind in ("image_url", "input_image"):
        u = part.get("image_url")
        u = u.get("url") if isinstance(u, dict) else u
        if not isinstance(u, str):
            raise ValueError("image part without a url")
        return u
    if kind == "image":
        src = part.get("source") or {}
        if src.get("type") == "base64" and isinstance(src.get("data"), str):
            return base64.b64decode(src["data"])
        if src.get("type") == "url":
            return src.get("url", "")
        raise ValueError("image part without a base64 source")
    return None


def split_media(messages: list) -> tuple[list, list]:
    """Messages with every image / audio part replaced by a text part holding `IMAGE_MARK`, and (kind, payload) pairs in prompt order."""
    out, media = [], []
    for m in messages:
        c = m.get("content") if isinstance(m, dict) else None
        if not isinstance(c, list):
            out.append(m)
            continue
        parts = []
        for p in c:
            img = _image_payload(p) if isinstance(p, dict) else None
            aud = _audio_payload(p) if isinstance(p, dict) and img is None else None
            if img is None and aud is None:
                parts.append(p)
            else:
                media.append(("image", img) if img is not None else ("audio", aud))
                parts.append({"type": "text", "text": IMAGE_MARK})
        out.append({**m, "content": parts})
    return out, media


def split_images(messages: list) -> tuple[list, list]:
    """Messages with every image part replaced by a text part holding `IMAGE_MARK`, and the payloads in prompt order."""
    out, images = [], []
    for m in messages:
        c = m.get("content") if isinstance(m, dict) else None
        if not isinstance(c, list):
            out.append(m)
            continue
        parts = []
        for p in c:
            payload = _image_payload(p) if isinstance(p, dict) else None
            if payload is None:
                parts.append(p)
            else:
                images.append(payload)
                parts.append({"type": "text", "text": IMAGE_MARK})
        out.append({**m, "content": parts})
    return out, images


def expand_prompt(text: str, counts: list[int], encode, start_id, pad_id, end_id) -> tuple[list[int], list[int]]:
    """Token ids of a rendered prompt whose images / clips sit at `IMAGE_MARK`, and the prompt positions of the pad tokens.  The ids are
    single values, or lists with one entry per item (image and audio placeholders differ)."""
    pieces = text.split(IMAGE_MARK)
    if len(pieces) != len(counts) + 1:
        raise ValueError("the prompt text contains the image marker itself")
    per_item = isinstance(pad_id, (list, tuple))
    starts, pads, ends = (start_id, pad_id, end_id) if per_item else ([start_id] * len(counts), [pad_id] * len(counts), [end_id] * len(counts))
    ids, positions = [], []
    for i, piece in enumerate(pieces):
        if piece:
            ids += encode(piece)
        if i < len(counts):
            start_id, pad_id, end_id = starts[i], pads[i], ends[i]
            if start_id is not None:
                ids.append(start_id)
            positions += range(len(ids), len(ids) + counts[i])
            ids += [pad_id] * counts[i]
            if end_id is not None:
                ids.append(end_id)
    return ids, positions


class VisionFrontEnd:
    """Owns the tower for a server.  `pad_id` / `start_id` / `end_id`: the tokenizer's image placeholder and its brackets
    (`image_token_id`, `vision_start_token_id`, `vision_end_token_id` of a Hugging Face config)."""

    def __init__(self, tower, pad_id: int | None = None, start_id: int | None = None, end_id: int | None = None, max_images: int = 8, *,
                 audio_tower=None, audio_pad_id: int | None = None, audio_start_id: int | None = None, audio_end_id: int | None = None):
        self.tower, self.pad_id, self.start_id, self.end_id, self.max_images = tower, pad_id, start_id, end_id, max_images
        self.audio_tower, self.audio_ids = audio_tower, (audio_start_id, audio_pad_id, audio_end_id)
        self._lock = threading.Lock()           # one encode at a time: the towers' buffers are shared
        self.images = self.image_tokens = self.clips = self.audio_tokens = 0

    def prepare(self, messages: list, render, encode):
        """`render(messages) -> str`, `encode(str) -> ids`.  Returns (prompt ids, embeds dict or None)."""
        import torch
        msgs, media = split_media(messages)
        if not media:
            return encode(render(messages)), None
        if len(media) > self.max_images:
            raise ValueError(f"{len(media)} images / clips in one request (limit {self.max_images})")
        items: list = [None] * len(media)              # per item: (input tensor, token count)
        for i, (kind, payload) in enumerate(media):
            if kind == "image":
                if self.tower is None:
                    raise ValueError("this server has no vision tower")
                from ..models.vision import image_tokens, load_image
                rgb = load_image(payload, self.tower.spec)
                items[i] = (rgb, image_tokens(rgb, self.tower.spec))
            else:
                if self.audio_tower is None:
                    raise ValueError("this server has no audio tower")
                from ..models.audio import audio_tokens, load_audio
                frames = load_audio(payload, self.audio_tower.spec)
                items[i] = (frames, audio_tokens(frames))
        counts = [n for _, n in items]
        img = (self.start_id, self.pad_id, self.end_id)
        triples = [img if kind == "image" else self.audio_ids for kind, _ in media]
        ids, positions = expand_prompt(render(msgs), counts, encode, [t[0] for t in triples], [t[1] for t in triples], [t[2] for t in triples])
        rows: list = [None] * len(media)
        with self._lock:
            for kind, tower in (("image", self.tower), ("audio", self.audio_tower)):
                sel = [i for i, (k, _) in enumerate(media) if k == kind]
                if not sel:
                    continue
                dev = getattr(tower, "device", None)
                if dev is not None and dev.type == "cuda":
                    torch.cuda.set_device(dev)                  # worker threads start on device 0
                for i, r in zip(sel, tower.encode([items[i][0] for i in sel])):       # all items of a kind in one batch
                    rows[i] = r
            out = torch.cat(rows)
            if out.is_cuda:
                torch.cuda.current_stream().synchronize()       # the scheduler thread reads the rows on its own stream
            for (kind, _), n in zip(media, counts):
                if kind == "image":
                    self.images, self.image_tokens = self.images + 1, self.image_tokens + n
                else:
                    self.clips, self.audio_tokens = self.clips + 1, self.audio_tokens + n
        return ids, {"positions": positions, "rows": out}

    def stats(self) -> dict:
        return {"images": self.images, "image_tokens": self.image_tokens, "clips": self.clips, "audio_tokens": self.audio_tokens,
                "encodes": getattr(self.tower, "encodes", 0) + getattr(self.audio_tower, "encodes", 0)}
