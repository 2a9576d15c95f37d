"""Identity of a page by its content and everything before it.

As in mercury/hashing.py:19-46: only full pages are hashed, and each hash chains on the one
before, so equal hashes mean equal prefixes. The reference hashes with Python's `hash`,
which differs between processes; here the default is 64-bit BLAKE2b over the parent hash
and the page's tokens as little-endian int32, and `cryptographic=True` gives the
reference's 128-bit SHA-256 variant (mercury/hashing.py:20-24).
"""

from __future__ import annotations

import hashlib
import struct
from typing import Sequence


def page_hash(parent: int, tokens: Sequence[int], cryptographic: bool = False) -> int:
    body = struct.pack(f"<{len(tokens)}i", *tokens)
    if cryptographic:
        digest = hashlib.sha256(parent.to_bytes(16, "big") + body).digest()[:16]
    else:
        digest = hashlib.blake2b(parent.to_bytes(16, "big") + body, digest_size=8).digest()
    return int.from_bytes(digest, "big")


def page_hashes(tokens: Sequence[int], page_size: int, parent: int = 0,
                cryptographic: bool = False) -> list[int]:
    """Chain hash of every FULL page of `tokens`."""
    out: list[int] = []
    for start in range(0, len(tokens) - page_size + 1, page_size):
        parent = page_hash(parent, tokens[start:start + page_size], cryptographic)
        out.append(parent)
    return out


def extend_hashes(hashes: list[int], tokens: Sequence[int], page_size: int,
                  cryptographic: bool = False) -> int:
    """Grow `hashes` in place to cover every full page of `tokens`; returns pages added."""
    full = len(tokens) // page_size
    parent = hashes[-1] if hashes else 0
    added = 0
    for index in range(len(hashes), full):
        parent = page_hash(parent, tokens[index * page_size:(index + 1) * page_size], cryptographic)
        hashes.append(parent)
        added += 1
    return added
