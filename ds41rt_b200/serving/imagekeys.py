"""Image identity for the prefix banks: what the radix compares at the placeholder positions of an image.

Every row of an image enters the prompt as the same placeholder token, so two prompts with different pictures have the
same token sequence.  For cache matching only, the placeholders of an image are replaced by a key that stands for the
image's content (`PreparedImage.identity`, a hash of the decoded pixels and the grid); the model, the tokenizer-facing
counts and the Engram history keep seeing the real tokens.  Keys live above every vocabulary id (from 2^31 on), are
handed out once and never reused: when the bounded intern table forgets an image and the image comes back, it gets a new
key, so a stored snapshot can go unmatched but can never be matched by another picture.  When the key range is used up
image prompts stop being banked (`prepare` returns None) instead of wrapping around.

Counterpart of the reference's sparse image identities for its token radix
(rust/crates/ds41rt-daemon/src/v41_native_serve/prefix/images.rs:10-60: keys from 2^31, encode over the placeholder
spans); the reference recycles keys under pins held by requests and snapshots, here keys are single-use and need no pins.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import List, Optional, Sequence, Tuple

FIRST_IMAGE_KEY = 1 << 31
LAST_IMAGE_KEY = (1 << 32) - 1


class ImageKeys:
    """The (position -> key) bindings of one request."""

    def __init__(self, bindings: List[Tuple[int, int]]):
        self.bindings = bindings                                  # sorted by position

    def __bool__(self) -> bool:
        return bool(self.bindings)

    def encode(self, tokens: Sequence[int]) -> List[int]:
        """`tokens` (the prompt, or the prompt plus emitted tokens, possibly cut short) with every bound position that
        falls inside it replaced by its image key."""
        out = list(tokens)
        n = len(out)
        for pos, key in self.bindings:
            if pos >= n:
                break
            out[pos] = key
        return out


class ImageKeySpace:
    def __init__(self, capacity: int = 4096):
        self.capacity = max(1, capacity)
        self.keys: "OrderedDict[str, int]" = OrderedDict()        # identity -> key, least recently used first
        self.next = FIRST_IMAGE_KEY
        self.issued = self.forgotten = 0

    def _key(self, identity: str) -> Optional[int]:
        k = self.keys.get(identity)
        if k is not None:
            self.keys.move_to_end(identity)
            return k
        if self.next > LAST_IMAGE_KEY:
            return None
        k, self.next = self.next, self.next + 1
        self.keys[identity] = k
        self.issued += 1
        while len(self.keys) > self.capacity:
            self.keys.popitem(last=False)
            self.forgotten += 1
        return k

    def prepare(self, tokens: Sequence[int], images) -> Optional[ImageKeys]:
        """Bindings for a request whose `images` are (PreparedImage, [prompt positions of its rows]) pairs.  None when the
        prompt cannot be keyed (no identity, positions outside the prompt or shared by two images, placeholder tokens
        that differ inside one image, key range used up): such a prompt is computed in full and not banked."""
        bindings: List[Tuple[int, int]] = []
        seen = set()
        n = len(tokens)
        for image, positions in images:
            ident = getattr(image, "identity", None)
            if not ident or not positions:
                return None
            if any(p < 0 or p >= n or p in seen for p in positions):
                return None
            if len({tokens[p] for p in positions}) != 1:
                return None
            seen.update(positions)
            key = self._key(str(ident))
            if key is None:
                return None
            bindings += [(p, key) for p in positions]
        bindings.sort()
        return ImageKeys(bindings)

    def stats(self) -> dict:
        return {"live": len(self.keys), "issued": self.issued, "forgotten": self.forgotten}
