"""Image preparation: grid policy, patch layout, identity hash, spans, hostile input."""
import io

import numpy as np
import pytest

from ds41rt_b200.config import VisionConfig
from ds41rt_b200.serving.images import (ImageError, choose_grid, decode_data_url, image_span, placeholder_positions,
                                        prepare_image)

V = VisionConfig()


def _png(w, h, seed=0):
    from PIL import Image
    rng = np.random.default_rng(seed)
    buf = io.BytesIO()
    Image.fromarray(rng.integers(0, 256, size=(h, w, 3), dtype=np.uint8)).save(buf, format="PNG")
    return buf.getvalue()


def test_grid_policy_bounds():
    for w, h in [(64, 64), (640, 480), (4000, 3000), (3000, 200), (14, 9000)]:
        gh, gw = choose_grid(w, h, V)
        assert gh % V.downsample == 0 and gw % V.downsample == 0 and gh > 0 and gw > 0
        assert (gh // 3) * (gw // 3) <= V.max_image_tokens
    gh, gw = choose_grid(64, 64, V)
    assert gh * gw * V.patch ** 2 >= 0.8 * V.min_pixels           # small images are scaled up to the minimum
    gh, gw = choose_grid(4000, 3000, V)
    assert abs(gw / gh - 4 / 3) < 0.15                              # aspect ratio survives the cap


def test_patches_and_identity():
    a = prepare_image(_png(320, 200, 1), V)
    b = prepare_image(_png(320, 200, 1), V)
    c = prepare_image(_png(320, 200, 2), V)
    gh, gw = a.grid
    assert a.patches.shape == (gh * gw, 3 * 14 * 14) and a.rows == (gh // 3) * (gw // 3)
    assert a.identity == b.identity != c.identity
    assert np.isfinite(a.patches).all() and abs(float(a.patches.mean())) < 3


def test_span_and_placeholders():
    img = prepare_image(_png(200, 120), V)
    span = image_span(img, V, image_token=9, start=1, end=2, newline=3)
    rows, cols = img.grid[0] // 3, img.grid[1] // 3
    assert span[0] == 1 and span[-1] == 2 and span.count(9) == img.rows and span.count(3) == rows
    assert len(placeholder_positions([5] + span + [6], 9)) == rows * cols


def test_bad_input_is_rejected():
    with pytest.raises(ImageError):
        prepare_image(b"not an image", V)
    with pytest.raises(ImageError):
        prepare_image(_png(50, 50)[:40], V)
    with pytest.raises(ImageError):
        decode_data_url("http://example.com/x.png")
    with pytest.raises(ImageError):
        decode_data_url("data:image/png;base64,@@@")
