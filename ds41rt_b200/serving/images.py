"""Image preparation on the host: decode, resize to the patch grid, patch extraction, identity hash, prompt spans.

Policy: an image becomes a grid of `patch`-pixel patches whose sides are multiples of `downsample` (the tower merges
downsample x downsample patches into one language-model row); the image is scaled, keeping its aspect ratio as far as
the grid allows, so that it has at least `min_pixels` pixels and at most `max_image_tokens` merged rows.  The prompt
gets `image_start`, one `image_token` placeholder per merged row with a newline marker after every grid row, and
`image_end`; the placeholder rows are overwritten with the tower's output.
Reference: rust/crates/ds41rt-loader/src/v41_image.rs:7-70 and v41_image/resize.rs (decode JPEG/PNG/WebP/GIF, resize /
grid policy, content identity hash, prompt span expansion).
"""
from __future__ import annotations

import base64
import hashlib
import io
import math
from dataclasses import dataclass
from typing import List, Tuple

import numpy as np

from ..config import VisionConfig

MEAN = np.array([0.48145466, 0.4578275, 0.40821073], dtype=np.float32)
STD = np.array([0.26862954, 0.26130258, 0.27577711], dtype=np.float32)


class ImageError(ValueError):
    pass


@dataclass
class PreparedImage:
    patches: np.ndarray          # [gh * gw, 3 * patch * patch] float32, channel-major inside a patch
    grid: Tuple[int, int]        # (gh, gw) in patches
    rows: int                    # merged rows the language model sees
    identity: str                # content hash of the decoded pixels and the grid (prefix-reuse key)


def decode_image(data: bytes):
    try:
        from PIL import Image
        img = Image.open(io.BytesIO(data))
        img.load()
    except Exception as e:       # truncated, unsupported or hostile input
        raise ImageError(f"cannot decode image: {e}") from None
    if getattr(img, "n_frames", 1) > 1:
        img.seek(0)              # animated GIF / WebP: first frame
    if img.mode in ("RGBA", "LA", "P"):
        rgba = img.convert("RGBA")
        from PIL import Image as _I
        bg = _I.new("RGBA", rgba.size, (255, 255, 255, 255))
        img = _I.alpha_composite(bg, rgba)
    return img.convert("RGB")


def decode_data_url(url: str) -> bytes:
    if not url.startswith("data:") or ";base64," not in url:
        raise ImageError("image_url must be a base64 data URL")
    try:
        return base64.b64decode(url.split(";base64,", 1)[1], validate=True)
    except Exception:
        raise ImageError("image data is not valid base64") from None


def choose_grid(width: int, height: int, v: VisionConfig) -> Tuple[int, int]:
    """(gh, gw) in patches: multiples of `downsample`, >= min_pixels when possible, <= max_image_tokens merged rows."""
    if width <= 0 or height <= 0:
        raise ImageError("empty image")
    unit = v.patch * v.downsample
    area = width * height
    scale = 1.0
    if area < v.min_pixels:
        scale = math.sqrt(v.min_pixels / area)
    max_area = v.max_image_tokens * unit * unit
    if area * scale * scale > max_area:
        scale = math.sqrt(max_area / area)
    gh = max(1, round(height * scale / unit))
    gw = max(1, round(width * scale / unit))
    while gh * gw > v.max_image_tokens:          # rounding may overshoot by one row or column
        if gh >= gw:
            gh -= 1
        else:
            gw -= 1
    return gh * v.downsample, gw * v.downsample


def prepare_image(data: bytes, v: VisionConfig) -> PreparedImage:
    img = decode_image(data)
    gh, gw = choose_grid(img.width, img.height, v)
    from PIL import Image
    img = img.resize((gw * v.patch, gh * v.patch), Image.BICUBIC)
    px = np.asarray(img, dtype=np.float32) / 255.0
    px = (px - MEAN) / STD                                            # [H, W, 3]
    p = v.patch
    patches = px.reshape(gh, p, gw, p, 3).transpose(0, 2, 4, 1, 3).reshape(gh * gw, 3 * p * p)
    digest = hashlib.sha256()
    digest.update(np.asarray(img, dtype=np.uint8).tobytes())
    digest.update(f"{gh}x{gw}".encode())
    return PreparedImage(np.ascontiguousarray(patches), (gh, gw), (gh // v.downsample) * (gw // v.downsample),
                         digest.hexdigest())


def image_span(image: PreparedImage, v: VisionConfig, image_token: int, start: int, end: int, newline: int) -> List[int]:
    """Token ids standing for one image: start, the placeholders of each merged grid row followed by a newline, end."""
    rows, cols = image.grid[0] // v.downsample, image.grid[1] // v.downsample
    out = [start]
    for _ in range(rows):
        out.extend([image_token] * cols)
        out.append(newline)
    out.append(end)
    return out


def placeholder_positions(tokens: List[int], image_token: int) -> List[int]:
    return [i for i, t in enumerate(tokens) if t == image_token]
