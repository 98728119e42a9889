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


def expand_prompt(text: str, counts: list[int], encode, start_id: int | None, pad_id: int, end_id: int | None) -> tuple[list[int], list[int]]:
    """Token ids of a rendered prompt whose images sit at `IMAGE_MARK`, and the prompt positions of the pad tokens."""
    pieces = text.split(IMAGE_MARK)
    if len(pieces) != len(counts) + 1:
        raise ValueError("the prompt text contains the image marker itself")
    ids, positions = [], []
    for i, piece in enumerate(pieces):
        if piece:
            ids += encode(piece)
        if i < len(counts):
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

    def __init__(self, tower, pad_id: int, start_id: int | None = None, end_id: int | None = None, max_images: int = 8):
        self.tower, self.pad_id, self.start_id, self.end_id, self.max_images = tower, pad_id, start_id, end_id, max_images
        self._lock = threading.Lock()           # one encode at a time: the tower's buffers are shared
        self.images = 0
        self.image_tokens = 0

    def prepare(self, messages: list, render, encode):
        """`render(messages) -> str`, `encode(str) -> ids`.  Returns (prompt ids, embeds dict or None)."""
        import torch
        from ..models.vision import image_tokens, load_image
        msgs, payloads = split_images(messages)
        if not payloads:
            return encode(render(messages)), None
        if len(payloads) > self.max_images:
            raise ValueError(f"{len(payloads)} images in one request (limit {self.max_images})")
        spec = self.tower.spec
        rgbs = [load_image(p, spec) for p in payloads]
        counts = [image_tokens(r, spec) for r in rgbs]
        ids, positions = expand_prompt(render(msgs), counts, encode, self.start_id, self.pad_id, self.end_id)
        with self._lock:
            dev = getattr(self.tower, "device", None)
            if dev is not None and dev.type == "cuda":
                torch.cuda.set_device(dev)                      # worker threads start on device 0
            rows = torch.cat(self.tower.encode(rgbs))
            if rows.is_cuda:
                torch.cuda.current_stream().synchronize()       # the scheduler thread reads the rows on its own stream
            self.images += len(rgbs)
            self.image_tokens += sum(counts)
        return ids, {"positions": positions, "rows": rows}

    def stats(self) -> dict:
        return {"images": self.images, "image_tokens": self.image_tokens, "encodes": getattr(self.tower, "encodes", 0)}
