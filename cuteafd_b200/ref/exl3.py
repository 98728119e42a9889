"""EXL3 (trellis / "QTIP"-style) weight-format oracle, plus a matching encoder for synthetic tests.

Format, as shipped in checkpoints (reference: python/tools/lib/exl3_reference.py:13-96,
rust/crates/cuteafd-loader/src/formats/exl3_format.rs:1-36):
  * `trellis`  uint16 [K/16, N/16, 16*bits]: each 16x16 weight tile is 256 symbols of `bits` bits,
    stored big-endian inside 16-bit words whose pair order is swapped;
  * decoding walks a 16-bit shift register: state = (state << bits | symbol) & 0xffff, primed with the
    tile's final symbols (tail-biting); each state maps to a value through a multiplicative hash:
    r = state * 0xCBAC1FED; r = 0x3B603B60 ^ (r & 0x8FFF8FFF); value = fp16(lo16) + fp16(hi16);
  * the 256 values of a tile are in tensor-core fragment order (a fixed lane permutation);
  * `suh` [K] and `svh` [N] are sign/scale vectors around 128-wide Hadamard rotations on both axes:
    W = H128( (H128(inner^T)^T) * suh[:, None] ) * svh[None, :]  (input-major weight, y = x @ W).

`decode_tiles`/`dequantize` are the oracle for the dequant-GEMM kernel; `encode_tiles_greedy` produces
valid synthetic trellis tensors (greedy nearest-value walk; good enough for kernel tests, not a quantiser).
"""
from __future__ import annotations

import numpy as np

MULT = 0xCBAC1FED
MASK_AND = 0x8FFF8FFF
MASK_XOR = 0x3B603B60


def state_values() -> np.ndarray:
    """Value of each of the 65536 register states (float32)."""
    st = np.arange(65536, dtype=np.uint64)
    r = ((st * MULT) & 0xFFFFFFFF).astype(np.uint32)
    r = np.uint32(MASK_XOR) ^ (r & np.uint32(MASK_AND))
    lo = (r & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float32)
    hi = (r >> 16).astype(np.uint16).view(np.float16).astype(np.float32)
    return lo + hi


def fragment_permutation() -> np.ndarray:
    """perm[j] = row*16+col (within the 16x16 tile) held at storage slot j."""
    perm = []
    for lane in range(32):
        r, c = (lane % 4) * 2, lane // 4
        for dr, dc in ((0, 0), (1, 0), (8, 0), (9, 0), (0, 8), (1, 8), (8, 8), (9, 8)):
            perm.append((r + dr) * 16 + c + dc)
    return np.asarray(perm)


def unpack_symbols(words: np.ndarray, bits: int) -> np.ndarray:
    """[..., 16*bits] uint16 -> [..., 256] symbols."""
    w = np.asarray(words).astype(np.uint16)
    w = w.reshape(*w.shape[:-1], -1, 2)[..., ::-1].reshape(w.shape)       # swap word pairs
    # big-endian bit stream over the 16*bits words; symbol i occupies bits [i*bits, (i+1)*bits)
    bitsarr = ((w[..., :, None].astype(np.uint32) >> np.arange(15, -1, -1)) & 1).reshape(*w.shape[:-1], -1)
    sym = bitsarr.reshape(*w.shape[:-1], 256, bits)
    weights = (1 << np.arange(bits - 1, -1, -1)).astype(np.uint32)
    return (sym * weights).sum(-1).astype(np.uint32)


def pack_symbols(symbols: np.ndarray, bits: int) -> np.ndarray:
    s = np.asarray(symbols).astype(np.uint32)
    b = ((s[..., :, None] >> np.arange(bits - 1, -1, -1)) & 1).reshape(*s.shape[:-1], 16 * bits, 16)
    w = (b * (1 << np.arange(15, -1, -1))).sum(-1).astype(np.uint16)
    return w.reshape(*w.shape[:-1], -1, 2)[..., ::-1].reshape(w.shape)


def decode_symbols(symbols: np.ndarray, bits: int) -> np.ndarray:
    """[..., 256] symbols -> [..., 256] float32 values in storage (fragment) order."""
    vals = state_values()
    state = np.zeros(symbols.shape[:-1], dtype=np.uint32)
    warm = (16 + bits - 1) // bits - 1
    for p in range(256 - warm, 256):
        state = ((state << bits) | symbols[..., p]) & 0xFFFF
    out = np.empty(symbols.shape, dtype=np.float32)
    for p in range(256):
        state = ((state << bits) | symbols[..., p]) & 0xFFFF
        out[..., p] = vals[state]
    return out


def decode_tiles(trellis: np.ndarray) -> np.ndarray:
    """[K/16, N/16, 16*bits] uint16 -> inner weight [K, N] float32 (before rotations)."""
    t = np.asarray(trellis)
    bits = t.shape[-1] // 16
    stor = decode_symbols(unpack_symbols(t, bits), bits)
    tile = np.empty_like(stor)
    tile[..., fragment_permutation()] = stor
    kt, nt = tile.shape[:2]
    return tile.reshape(kt, nt, 16, 16).transpose(0, 2, 1, 3).reshape(kt * 16, nt * 16)


def hadamard128(x: np.ndarray) -> np.ndarray:
    """Normalised 128-wide Walsh-Hadamard transform over the last axis, block by block."""
    x = np.array(x, dtype=np.float64)
    shape = x.shape
    assert shape[-1] % 128 == 0
    y = x.reshape(-1, 128)
    h = 1
    while h < 128:
        y = y.reshape(-1, 128 // (2 * h), 2, h)
        y = np.stack([y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]], axis=2)
        h *= 2
    return y.reshape(shape) / np.sqrt(128.0)


def dequantize(trellis, suh, svh) -> np.ndarray:
    """Effective weight [K, N] float64 with y = x @ W."""
    inner = decode_tiles(trellis).astype(np.float64)
    w = hadamard128(inner.T).T * np.asarray(suh, dtype=np.float64)[:, None]
    return hadamard128(w) * np.asarray(svh, dtype=np.float64)[None, :]


def encode_tiles_greedy(inner: np.ndarray, bits: int, seed: int = 0) -> np.ndarray:
    """Greedy trellis walk producing a valid tail-biting encoding of `inner` [K, N].
    Symbol p is chosen to minimise |value(state') - target_p| given the running state; the warm-up
    symbols are the tile's own final symbols, found by two passes."""
    K, N = inner.shape
    vals = state_values()
    tiles = inner.reshape(K // 16, 16, N // 16, 16).transpose(0, 2, 1, 3).reshape(K // 16, N // 16, 256)
    target = tiles[..., fragment_permutation()]
    sym = np.random.default_rng(seed).integers(0, 1 << bits, size=target.shape).astype(np.uint32)
    warm = (16 + bits - 1) // bits - 1
    cand = np.arange(1 << bits, dtype=np.uint32)
    for _ in range(2):
        state = np.zeros(target.shape[:-1], dtype=np.uint32)
        for p in range(256 - warm, 256):
            state = ((state << bits) | sym[..., p]) & 0xFFFF
        for p in range(256):
            nxt = ((state[..., None] << bits) | cand) & 0xFFFF
            # the last `warm` symbols are frozen on the second pass so the tail-biting prefix stays valid
            best = np.abs(vals[nxt] - target[..., p, None]).argmin(-1).astype(np.uint32)
            if _ == 1 and p >= 256 - warm:
                best = sym[..., p]
            sym[..., p] = best
            state = ((state << bits) | best) & 0xFFFF
    return pack_symbols(sym, bits)
