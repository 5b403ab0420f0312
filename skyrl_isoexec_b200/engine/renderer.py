"""Rendering a multimodal conversation into what the engine and the trainer consume (reference: R/backends/renderer.py and
the ``/v1/chat/completions/render`` endpoint of its inference servers): token ids in which every image is a run of
placeholder tokens, where those runs are, and the images' patches.

    render_conversation(messages, tokenizer, cfg) ->
        {"token_ids": [...],
         "features": None, or {"mm_placeholders": {"image": [{"offset", "length"}, ...]},
                               "pixel_values": [patches, dim] float32, "image_grid_thw": [images, 3] int64,
                               "positions": [every placeholder position, ascending]}}

A message's ``content`` is a string or a list of parts: ``{"type": "text", "text": ...}``, ``{"type": "image", "image":
<tensor [3, H, W] | numpy [H, W, 3] | PIL image | encoded bytes>}``, ``{"type": "image_url", "image_url": {"url":
"data:image/png;base64,..."}}``. The conversation is rendered to text through the tokenizer's chat template with a
sentinel in place of every image, the text between sentinels is tokenized piece by piece (an image separates text
the way a special token does), and each sentinel becomes ``num_image_tokens`` copies of the model's ``image_token_id``.

Rendering is a pure function of the conversation, so a later turn's render extends an earlier turn's wherever the chat
template is prefix-stable; the vision-language generator relies on that to find the observation tokens of a turn.

``encode_features`` / ``decode_features`` turn the tensors of ``features`` into base64 text and back for the HTTP route.
"""

from __future__ import annotations

from ..utils.tokenizer import chat_ids

import base64
import io

import torch

from ..models.vision import patchify

_SENTINEL = "\x00<image>\x00"


def to_image_tensor(obj) -> torch.Tensor:
    """Anything an image part may hold -> uint8 / float tensor [3, H, W]."""
    if torch.is_tensor(obj):
        t = obj
        if t.dim() == 3 and t.shape[0] != 3 and t.shape[-1] == 3:
            t = t.permute(2, 0, 1)
        return t
    if isinstance(obj, (bytes, bytearray)):
        from PIL import Image

        obj = Image.open(io.BytesIO(bytes(obj)))
    if hasattr(obj, "convert"):                                  # a PIL image
        import numpy as np

        obj = np.asarray(obj.convert("RGB"))
    if hasattr(obj, "shape") and hasattr(obj, "dtype"):          # numpy, [H, W, 3]
        t = torch.from_numpy(obj.copy())
        return t.permute(2, 0, 1) if t.dim() == 3 and t.shape[-1] == 3 else t
    raise TypeError(f"cannot read an image from {type(obj).__name__}")


def _image_of_part(part: dict) -> torch.Tensor:
    if part.get("type") == "image":
        return to_image_tensor(part["image"])
    url = part["image_url"]["url"] if isinstance(part.get("image_url"), dict) else part.get("image_url")
    if not isinstance(url, str) or not url.startswith("data:"):
        raise ValueError("image_url parts must be data: URLs (base64); remote locations are not fetched")
    return to_image_tensor(base64.b64decode(url.split(",", 1)[1]))


def split_content(messages: list[dict]) -> tuple[list[dict], list[torch.Tensor]]:
    """Messages with string contents (a sentinel where an image was) and the images in order."""
    flat, images = [], []
    for m in messages:
        c = m.get("content")
        if isinstance(c, (list, tuple)):
            text = ""
            for part in c:
                if isinstance(part, str):
                    text += part
                elif part.get("type") == "text":
                    text += part.get("text", "")
                elif part.get("type") in ("image", "image_url"):
                    images.append(_image_of_part(part))
                    text += _SENTINEL
                else:
                    raise ValueError(f"unknown content part type {part.get('type')!r}")
            m = dict(m, content=text)
        flat.append(m)
    return flat, images


def render_conversation(messages: list[dict], tokenizer, cfg, add_generation_prompt: bool = True) -> dict:
    flat, images = split_content(messages)
    if not images:
        ids = chat_ids(tokenizer, flat, add_generation_prompt)
        return {"token_ids": ids, "features": None}
    if not getattr(cfg, "has_vision", False):
        raise ValueError(f"model {cfg.name!r} has no vision tower: the conversation must not contain images")
    text = tokenizer.apply_chat_template(flat, add_generation_prompt=add_generation_prompt, tokenize=False)
    pieces = text.split(_SENTINEL)
    if len(pieces) != len(images) + 1:
        raise ValueError("the chat template dropped or duplicated an image marker")
    ids: list[int] = []
    spans, pvs, grids = [], [], []
    for k, piece in enumerate(pieces):
        ids += _encode_text(tokenizer, piece)
        if k < len(images):
            pv, grid = patchify(images[k], cfg.vision_patch, cfg.vision_merge)
            n = int(grid[0, 1] * grid[0, 2]) // (cfg.vision_merge ** 2)
            spans.append({"offset": len(ids), "length": n})
            ids += [cfg.image_token_id] * n
            pvs.append(pv)
            grids.append(grid)
    positions = [p for s in spans for p in range(s["offset"], s["offset"] + s["length"])]
    return {"token_ids": ids, "features": {"mm_placeholders": {"image": spans}, "pixel_values": torch.cat(pvs, 0),
                                           "image_grid_thw": torch.cat(grids, 0), "positions": positions}}


def render_model_input(chunks: list[dict], cfg) -> dict:
    """A Tinker-style model input (reference: R/backends/renderer.py:76-176, R/tinker/types.py chunk types) -> the same
    ``{"token_ids", "features"}``. Chunks: ``{"type": "encoded_text", "tokens": [...]}`` and ``{"type": "image", "data":
    <base64 of an encoded image>, "format": "png", "expected_tokens": n?}``; an ``expected_tokens`` that differs from the
    number of placeholder tokens the image really takes is an error, as in Tinker."""
    ids: list[int] = []
    spans, pvs, grids = [], [], []
    for i, ch in enumerate(chunks):
        kind = ch.get("type", "encoded_text")
        if kind == "encoded_text":
            ids += [int(t) for t in ch["tokens"]]
        elif kind == "image":
            if not getattr(cfg, "has_vision", False):
                raise ValueError(f"model {cfg.name!r} has no vision tower: the input must not contain image chunks")
            data = ch["data"]
            img = to_image_tensor(base64.b64decode(data) if isinstance(data, str) else data)
            pv, grid = patchify(img, cfg.vision_patch, cfg.vision_merge)
            n = int(grid[0, 1] * grid[0, 2]) // (cfg.vision_merge ** 2)
            if ch.get("expected_tokens") is not None and int(ch["expected_tokens"]) != n:
                raise ValueError(f"chunk {i}: expected_tokens={ch['expected_tokens']} but the image takes {n} placeholder tokens")
            spans.append({"offset": len(ids), "length": n})
            ids += [cfg.image_token_id] * n
            pvs.append(pv)
            grids.append(grid)
        else:
            raise ValueError(f"chunk {i}: unknown type {kind!r} (image asset pointers are not fetched)")
    if not spans:
        return {"token_ids": ids, "features": None}
    positions = [p for s in spans for p in range(s["offset"], s["offset"] + s["length"])]
    return {"token_ids": ids, "features": {"mm_placeholders": {"image": spans}, "pixel_values": torch.cat(pvs, 0),
                                           "image_grid_thw": torch.cat(grids, 0), "positions": positions}}


def _encode_text(tokenizer, text: str) -> list[int]:
    """Tokenize rendered template text: special-token names in it become their ids again where the tokenizer can do that."""
    if not text:
        return []
    if hasattr(tokenizer, "encode_rendered"):
        return list(tokenizer.encode_rendered(text))
    try:
        return list(tokenizer.encode(text, add_special_tokens=False))
    except TypeError:
        return list(tokenizer.encode(text))


def encode_features(features: dict | None) -> dict | None:
    """Tensors -> base64 of their raw bytes plus shape and dtype (JSON-safe)."""
    if features is None:
        return None

    def enc(t):
        t = t.contiguous().cpu()
        return {"b64": base64.b64encode(t.view(torch.uint8).numpy().tobytes()).decode("ascii"), "shape": list(t.shape), "dtype": str(t.dtype).split(".")[-1]}

    return {"mm_placeholders": features["mm_placeholders"], "positions": list(features["positions"]),
            "kwargs_data": {"pixel_values": enc(features["pixel_values"]), "image_grid_thw": enc(features["image_grid_thw"])}}


def decode_features(features: dict | None) -> dict | None:
    """The inverse of ``encode_features``; passes already-decoded features through."""
    if features is None or "kwargs_data" not in features:
        return features

    def dec(d):
        dt = getattr(torch, d["dtype"])
        raw = torch.frombuffer(bytearray(base64.b64decode(d["b64"])), dtype=torch.uint8)
        return raw.view(dt).reshape(d["shape"]).clone()

    kd = features["kwargs_data"]
    return {"mm_placeholders": features["mm_placeholders"], "positions": list(features["positions"]),
            "pixel_values": dec(kd["pixel_values"]), "image_grid_thw": dec(kd["image_grid_thw"])}
