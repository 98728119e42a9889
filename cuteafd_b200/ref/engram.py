"""N-gram memory ("engram") of the V4.1 line: at a few layers every token looks up rows of a very large hashed table by the
2-, 3- and 4-grams that end at it, and a learned gate mixes a projection of those rows into the residual stream(s).

Addressing (per engram layer): the token ids are first mapped to a compressed vocabulary; with c0 the current id and c1..c3 the three
before it (the pad id where the sequence has not started, or behind an image), a rolling value r = c0 * m0 is extended per order
o = 1..3 by r ^= c_o * m_o (64-bit wrap-around, odd multipliers drawn once per layer) and, for each of 8 heads per order, addresses
row (r mod p) + offset of that head's own table, p one of 24 consecutive primes - 24 rows of `row_dim` values per token and layer.
Rows are stored as FP8 E4M3 with one power-of-two scale per 32 values.  The 24 rows, concatenated, are projected to one key per
residual stream and one value; stream s takes  x_s + sigmoid(ssqrt(<x_s * wq_s * wk_s, k_s> / (rms(x_s) rms(k_s) sqrt(H)))) * v,
with ssqrt(d) = sign(d) sqrt(max(|d|, 1e-6)).  Image positions take nothing.

Only the last three ids matter for the next position, so a request's addressing state is three ids (`EngramHistory`): batches are
prepared against it without side effects and committed only for the tokens that were accepted (speculative decoding), it can be
forked and rebuilt from a stored lookback.

Reference: rust/crates/cuteafd-core/src/engram.rs (addressing and request-owned history), native/families/deepseek_v41/cuda/engram.cu
(row dequantisation and the gate), rust/crates/cuteafd-loader/src/families/deepseek_v41/engram_gather.rs (row gathers from mapped tables).
"""
from __future__ import annotations

import itertools
from dataclasses import dataclass, field

import numpy as np
import torch

ORDERS, HEADS = 3, 8
COLUMNS = ORDERS * HEADS


@dataclass(frozen=True)
class EngramSpec:
    layers: tuple = (1,)              # decoder layers whose input takes the memory
    vocab: int = 1024                 # compressed vocabulary (ids below this value; the pad id included)
    pad_id: int = 0
    row_dim: int = 256
    prime_floor: int = 500            # the tables' sizes are the primes that follow this value
    streams: int = 1                  # residual streams the gate serves (hyper-connection stacks: 4)
    hidden: int = 256

    @property
    def width(self) -> int:
        return COLUMNS * self.row_dim


def _primes_after(start: int, n: int) -> list[int]:
    out, c = [], start
    while len(out) < n:
        c += 1
        if c % 2 and all(c % d for d in range(3, int(c ** 0.5) + 1, 2)):
            out.append(c)
    return out


class EngramAddressing:
    """Multipliers, primes and table offsets of every engram layer."""

    def __init__(self, spec: EngramSpec):
        self.spec = spec
        primes = _primes_after(max(spec.prime_floor, 2), COLUMNS * len(spec.layers))
        self.primes = np.array(primes, dtype=np.uint64).reshape(len(spec.layers), COLUMNS)
        self.offsets = np.concatenate([np.zeros((len(spec.layers), 1), dtype=np.uint64), np.cumsum(self.primes, axis=1)[:, :-1]], axis=1)
        self.rows = [int(p.sum()) for p in self.primes]                 # table rows per layer
        hi = (np.iinfo(np.int64).max // spec.vocab) // 2
        self.mult = np.stack([np.random.default_rng(10007 * layer).integers(0, hi, 4).astype(np.uint64) * np.uint64(2) + np.uint64(1)
                              for layer in spec.layers])

    def hashes(self, ids: np.ndarray) -> np.ndarray:
        """ids: int64 [n + 3] compressed ids, the first three being the lookback of the first position (pad where there is none).
        Returns uint64 [layers, n, 24] table rows."""
        ids = np.asarray(ids, dtype=np.uint64)
        n = ids.shape[0] - 3
        out = np.zeros((len(self.spec.layers), n, COLUMNS), dtype=np.uint64)
        with np.errstate(over="ignore"):
            for l in range(len(self.spec.layers)):
                rolling = ids[3:] * self.mult[l, 0]
                for order in range(1, 4):
                    rolling = rolling ^ (ids[3 - order: 3 - order + n] * self.mult[l, order])
                    cols = slice((order - 1) * HEADS, order * HEADS)
                    out[l, :, cols] = rolling[:, None] % self.primes[l, cols][None, :] + self.offsets[l, cols][None, :]
        return out


_owner = itertools.count(1)


@dataclass
class EngramBatch:
    owner: int
    generation: int
    position: int
    ids: list                      # compressed ids of the batch (None: image position)
    hashes: np.ndarray             # uint64 [layers, n, 24]

    def is_image(self, row: int) -> bool:
        return self.ids[row] is None


@dataclass
class EngramHistory:
    """A request's addressing state: position and the last three compressed ids (None behind an image barrier)."""
    pad_id: int
    owner: int = field(default_factory=lambda: next(_owner))
    generation: int = 0
    position: int = 0
    recent: tuple = (None, None, None)          # most recent first

    def prepare(self, addr: EngramAddressing, ids: list) -> EngramBatch:
        """Addresses for the next len(ids) positions; the history itself does not move.  An image position (None) contributes nothing and
        hides everything before it from later positions."""
        look = list(self.recent)
        ctx = []
        for t in ids:
            ctx.append([t if t is not None else self.pad_id] + [x if x is not None else self.pad_id for x in look])
            look = [None, None, None] if t is None else [t] + look[:2]
        arr = np.array(ctx, dtype=np.int64).reshape(-1, 4)
        out = np.zeros((len(addr.spec.layers), len(ids), COLUMNS), dtype=np.uint64)
        for i in range(len(ids)):           # per row: barriers make the window irregular
            window = np.array([arr[i, 3], arr[i, 2], arr[i, 1], arr[i, 0]], dtype=np.int64)
            out[:, i] = addr.hashes(window)[:, 0]
        return EngramBatch(self.owner, self.generation, self.position, list(ids), out)

    def commit(self, batch: EngramBatch, accepted: int):
        """Accept the first `accepted` tokens of a batch prepared against this very state."""
        if batch.owner != self.owner or batch.generation != self.generation or batch.position != self.position:
            raise ValueError("engram batch was prepared against another state of the request")
        if not 0 <= accepted <= len(batch.ids):
            raise ValueError("accepted token count out of range")
        look = list(self.recent)
        for t in batch.ids[:accepted]:
            look = [None, None, None] if t is None else [t] + look[:2]
        self.recent, self.position, self.generation = tuple(look), self.position + accepted, self.generation + 1

    def fork(self) -> "EngramHistory":
        """Same lookback under a fresh identity: batches prepared for the original are refused by the fork."""
        return EngramHistory(self.pad_id, position=self.position, recent=self.recent)

    @staticmethod
    def from_recent(pad_id: int, position: int, recent: list) -> "EngramHistory":
        """Rebuild at an absolute position from the stored lookback (chronological, min(position, 3) entries)."""
        if len(recent) != min(position, 3):
            raise ValueError("engram resume needs the complete bounded lookback")
        look = [None, None, None]
        for t in recent:
            look = [t] + look[:2]
        return EngramHistory(pad_id, position=position, recent=tuple(look))


def context_hashes(addr: EngramAddressing, tokens_before: list, new_tokens: list, token_map=None) -> np.ndarray:
    """Addresses of `new_tokens` appended to a text-only sequence `tokens_before` (what a serving step needs: the scheduler knows the
    whole sequence, so no state has to be carried).  uint64 [layers, n, 24]."""
    look = list(tokens_before[-3:])
    seq = look + list(new_tokens)
    if token_map is not None:
        seq = [int(token_map[t]) for t in seq]
    return addr.hashes(np.array([addr.spec.pad_id] * (3 - len(look)) + seq, dtype=np.int64))


# ---------------------------------------------------------------------------------------------- table rows and the gate
def quantize_rows(rows: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """fp32 [n, row_dim] -> (E4M3 bytes uint8 [n, row_dim], UE8M0 exponents uint8 [n, row_dim / 32])."""
    n, d = rows.shape
    blocks = rows.reshape(n, d // 32, 32)
    amax = blocks.abs().amax(dim=-1).clamp(min=1e-12)
    exp = torch.ceil(torch.log2(amax / 448.0)).clamp(-127, 127)
    q = (blocks / torch.exp2(exp)[..., None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.reshape(n, d).view(torch.uint8), (exp + 127).to(torch.uint8)


def dequantize_rows(q: torch.Tensor, e: torch.Tensor) -> torch.Tensor:
    n, d = q.shape
    vals = q.view(torch.float8_e4m3fn).float().reshape(n, d // 32, 32)
    return (vals * torch.exp2(e.float() - 127)[..., None]).reshape(n, d)


def init_engram_weights(spec: EngramSpec, seed: int = 0) -> dict:
    g = torch.Generator().manual_seed(seed)
    addr = EngramAddressing(spec)
    S, H = spec.streams, spec.hidden
    layers = []
    for l in range(len(spec.layers)):
        q, e = quantize_rows(torch.randn(addr.rows[l], spec.row_dim, generator=g))
        layers.append({"table_q": q, "table_e": e, "proj": torch.randn((S + 1) * H, spec.width, generator=g) * spec.width ** -0.5,
                       "wq": 1 + 0.1 * torch.randn(S, H, generator=g), "wk": 1 + 0.1 * torch.randn(S, H, generator=g)})
    return {"layers": layers}


def gather_rows(lw: dict, hashes: np.ndarray) -> torch.Tensor:
    """uint64 [n, 24] -> fp32 [n, 24 * row_dim], rounded to bf16 as the device hands them to the projection."""
    idx = torch.from_numpy(hashes.astype(np.int64)).reshape(-1)
    rows = dequantize_rows(lw["table_q"][idx], lw["table_e"][idx])
    return rows.reshape(hashes.shape[0], -1).bfloat16().float()


def engram_gate(x: torch.Tensor, kv: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor, text_mask: torch.Tensor | None = None) -> torch.Tensor:
    """x [n, S, H], kv [n, S + 1, H] (keys per stream, then the value) -> x + gate * value."""
    S, H = x.shape[1], x.shape[2]
    k, v = kv[:, :S], kv[:, S]
    dot = (x * (wq * wk)[None] * k).sum(-1)
    rstd = torch.rsqrt(x.pow(2).mean(-1) + 1e-20) * torch.rsqrt(k.pow(2).mean(-1) + 1e-20)
    d = dot * rstd * H ** -0.5
    gate = torch.sigmoid(torch.sign(d) * torch.sqrt(d.abs().clamp(min=1e-6)))
    out = x + gate[..., None] * v[:, None, :]
    if text_mask is not None:
        out = torch.where(text_mask[:, None, None], out, x)
    return out


def engram_apply(spec: EngramSpec, lw: dict, x: torch.Tensor, hashes: np.ndarray, text_mask: torch.Tensor | None = None) -> torch.Tensor:
    """One engram layer on x [n, S, H] (fp32; bf16 roundings where the device stores bf16)."""
    rows = gather_rows(lw, hashes)
    kv = (rows @ lw["proj"].bfloat16().float().T).bfloat16().float().reshape(x.shape[0], spec.streams + 1, spec.hidden)
    return engram_gate(x, kv, lw["wq"], lw["wk"], text_mask)
