"""XXH64 in pure Python (test oracle).

The reference hashes KV blocks with ``xxhash.xxh64`` (engine/block_manager.py:51-57); xxhash is a
third-party dependency that the reference does not pin.  XXH64 is a frozen public algorithm; this
file restates it from its specification so the oracle does not depend on the package.
"""
from __future__ import annotations

_M = (1 << 64) - 1
_P1 = 0x9E3779B185EBCA87
_P2 = 0xC2B2AE3D27D4EB4F
_P3 = 0x165667B19E3779F9
_P4 = 0x85EBCA77C2B2AE63
_P5 = 0x27D4EB2F165667C5


def _rotl(x: int, r: int) -> int:
    return ((x << r) | (x >> (64 - r))) & _M


def _round(acc: int, lane: int) -> int:
    return (_rotl((acc + lane * _P2) & _M, 31) * _P1) & _M


def _merge(acc: int, val: int) -> int:
    return (((acc ^ _round(0, val)) * _P1) + _P4) & _M


def xxh64(data: bytes, seed: int = 0) -> int:
    n = len(data)
    pos = 0
    if n >= 32:
        v = [(seed + _P1 + _P2) & _M, (seed + _P2) & _M, seed & _M, (seed - _P1) & _M]
        while pos + 32 <= n:
            for i in range(4):
                v[i] = _round(v[i], int.from_bytes(data[pos + 8 * i:pos + 8 * i + 8], "little"))
            pos += 32
        h = (_rotl(v[0], 1) + _rotl(v[1], 7) + _rotl(v[2], 12) + _rotl(v[3], 18)) & _M
        for i in range(4):
            h = _merge(h, v[i])
    else:
        h = (seed + _P5) & _M
    h = (h + n) & _M
    while pos + 8 <= n:
        h ^= _round(0, int.from_bytes(data[pos:pos + 8], "little"))
        h = (_rotl(h, 27) * _P1 + _P4) & _M
        pos += 8
    if pos + 4 <= n:
        h ^= (int.from_bytes(data[pos:pos + 4], "little") * _P1) & _M
        h = (_rotl(h, 23) * _P2 + _P3) & _M
        pos += 4
    while pos < n:
        h ^= (data[pos] * _P5) & _M
        h = (_rotl(h, 11) * _P1) & _M
        pos += 1
    h ^= h >> 33
    h = (h * _P2) & _M
    h ^= h >> 29
    h = (h * _P3) & _M
    h ^= h >> 32
    return h


def block_hash(token_ids, prefix: int = -1) -> int:
    """BlockManager.compute_hash (engine/block_manager.py:45-57): optional 8-byte little-endian
    prefix hash followed by the token ids as little-endian int32."""
    data = b"" if prefix == -1 else int(prefix).to_bytes(8, "little")
    data += b"".join(int(t).to_bytes(4, "little", signed=True) for t in token_ids)
    return xxh64(data, 0)
