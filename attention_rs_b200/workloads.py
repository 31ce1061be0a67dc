"""Seeded synthetic workloads with the shapes of the benchmark configurations.

No dataset is involved: the model names attached to the configurations only supply
shapes.  Lengths, block tables and slot mappings come from a numpy Generator seeded
with ``20240 + configuration index``; tensor values are N(0,1).

Configuration index -> workload:
  1  decode, batch 4, 32 q / 32 kv heads, d128, block 16, context U{1..512}, 256-block pool
  2  decode, batch 64, 32 / 8, d128, block 16, context U{1024..8192}            (headline)
  3  reshape_and_cache, 16 x 2048 tokens, 8 heads, d128, block 16, 65536-slot pool, ~2% padding
  4  decode, FP8 cache, batch 128, 64 / 8, d128, block 16, context U{4096..32768}
  5  decode with ALiBi, batch 8, 32 / 8, d128, block 32, context U{65536..131072}
"""
from __future__ import annotations

import dataclasses
import math
from typing import Optional

import numpy as np

PARTITION_SIZE = 512


@dataclasses.dataclass
class DecodeWorkload:
    name: str
    num_seqs: int
    num_heads: int
    num_kv_heads: int
    head_size: int
    block_size: int
    dtype: str                 # "bf16" | "f16" | "f32"
    kv_dtype: str              # same as dtype, or "fp8"
    context_lens: np.ndarray   # uint32 [num_seqs]
    block_tables: np.ndarray   # uint32 [num_seqs, max_blocks]
    num_blocks: int
    scale: float
    alibi_slopes: Optional[np.ndarray] = None
    softcapping: float = 1.0
    seed: int = 0

    @property
    def max_context_len(self) -> int:
        return int(self.context_lens.max()) if self.context_lens.size else 0

    @property
    def kv_elem_size(self) -> int:
        return {"bf16": 2, "f16": 2, "f32": 4, "fp8": 1}[self.kv_dtype]

    def kv_bytes(self) -> int:
        """Algorithmic KV bytes of one decode step: every context token's K and V row,
        once per kv head, exact context length (no padding to the block size)."""
        return int(self.context_lens.astype(np.int64).sum()) * self.num_kv_heads * self.head_size * 2 * self.kv_elem_size

    def shard(self, rank: int, world: int) -> "DecodeWorkload":
        """The slice of this workload owned by ``rank`` when kv heads are split over ``world`` ranks.
        Block tables and context lengths are replicated; heads, slopes and the cache shrink."""
        if self.num_kv_heads % world != 0:
            raise ValueError(f"{self.num_kv_heads} kv heads do not split over {world} ranks")
        group = self.num_heads // self.num_kv_heads
        kvh = self.num_kv_heads // world
        slopes = None
        if self.alibi_slopes is not None:
            slopes = self.alibi_slopes[rank * kvh * group:(rank + 1) * kvh * group].copy()
        return dataclasses.replace(self, name=f"{self.name}/rank{rank}of{world}", num_heads=kvh * group,
                                   num_kv_heads=kvh, alibi_slopes=slopes)


def _tables(rng: np.random.Generator, lens: np.ndarray, block_size: int, num_blocks: Optional[int], disjoint: bool):
    need = (lens.astype(np.int64) + block_size - 1) // block_size
    max_blocks = max(int(need.max()) if need.size else 1, 1)
    if num_blocks is None:
        num_blocks = int(need.sum())
    tables = np.zeros((len(lens), max_blocks), dtype=np.uint32)
    if disjoint:
        perm = rng.permutation(num_blocks).astype(np.uint32)
        pos = 0
        for s, n in enumerate(need):
            tables[s, :n] = perm[pos:pos + n]
            pos += int(n)
    else:
        for s, n in enumerate(need):
            tables[s, :n] = rng.permutation(num_blocks).astype(np.uint32)[:n]
    return tables, num_blocks


def alibi_slopes(num_heads: int) -> np.ndarray:
    """The geometric sequence 2^(-8 i / n), i = 1..n."""
    return np.array([2.0 ** (-8.0 * i / num_heads) for i in range(1, num_heads + 1)], dtype=np.float32)


def decode_workload(cfg: int, *, num_seqs: Optional[int] = None, ctx_range: Optional[tuple] = None,
                    dtype: Optional[str] = None, seed: Optional[int] = None) -> DecodeWorkload:
    """Metadata (lengths, tables) of decode configuration ``cfg`` (1, 2, 4 or 5).  ``num_seqs`` and
    ``ctx_range`` shrink a configuration for tests without changing its structure."""
    seed = 20240 + cfg if seed is None else seed
    rng = np.random.default_rng(seed)
    if cfg == 1:
        ns, nh, nkv, hs, bs, lo, hi, dt, kv = 4, 32, 32, 128, 16, 1, 512, "bf16", None
    elif cfg == 2:
        ns, nh, nkv, hs, bs, lo, hi, dt, kv = 64, 32, 8, 128, 16, 1024, 8192, "bf16", None
    elif cfg == 4:
        ns, nh, nkv, hs, bs, lo, hi, dt, kv = 128, 64, 8, 128, 16, 4096, 32768, "bf16", "fp8"
    elif cfg == 5:
        ns, nh, nkv, hs, bs, lo, hi, dt, kv = 8, 32, 8, 128, 32, 65536, 131072, "bf16", None
    else:
        raise ValueError(f"configuration {cfg} is not a decode workload")
    ns = ns if num_seqs is None else num_seqs
    lo, hi = (lo, hi) if ctx_range is None else ctx_range
    dt = dt if dtype is None else dtype
    lens = rng.integers(lo, hi + 1, size=ns).astype(np.uint32)
    if cfg == 1:
        tables, nb = _tables(rng, lens, bs, 256, disjoint=False)   # each sequence: prefix of a permutation of the pool
    else:
        tables, nb = _tables(rng, lens, bs, None, disjoint=True)
    return DecodeWorkload(name=f"cfg{cfg}", num_seqs=ns, num_heads=nh, num_kv_heads=nkv, head_size=hs, block_size=bs,
                          dtype=dt, kv_dtype=kv or dt, context_lens=lens, block_tables=tables, num_blocks=nb,
                          scale=1.0 / math.sqrt(hs), alibi_slopes=alibi_slopes(nh) if cfg == 5 else None, seed=seed)


@dataclasses.dataclass
class ScatterWorkload:
    name: str
    num_tokens: int
    num_heads: int
    head_size: int
    block_size: int
    num_slots: int
    dtype: str
    slot_mapping: np.ndarray  # int64 [num_tokens]
    seed: int = 0

    @property
    def num_blocks(self) -> int:
        return self.num_slots // self.block_size

    def algorithmic_bytes(self, cache_elem_size: Optional[int] = None) -> int:
        es = {"bf16": 2, "f16": 2, "f32": 4}[self.dtype]
        ces = es if cache_elem_size is None else cache_elem_size
        valid = int((self.slot_mapping >= 0).sum())
        return valid * self.num_heads * self.head_size * 2 * (es + ces) + self.num_tokens * 8


def scatter_workload(*, num_tokens: int = 16 * 2048, num_heads: int = 8, head_size: int = 128, block_size: int = 16,
                     num_slots: int = 65536, pad_fraction: float = 0.02, dtype: str = "bf16",
                     contiguous: bool = False, seed: int = 20243) -> ScatterWorkload:
    """Configuration 3: tokens to seeded random free slots, ~2% padding (-1).  ``contiguous`` gives the
    slot pattern of a real prefill instead (runs of consecutive slots)."""
    rng = np.random.default_rng(seed)
    if contiguous:
        slots = np.arange(num_tokens, dtype=np.int64) + rng.integers(0, max(num_slots - num_tokens, 0) + 1)
    else:
        slots = rng.permutation(num_slots)[:num_tokens].astype(np.int64)
    pad = rng.random(num_tokens) < pad_fraction
    slots[pad] = -1
    return ScatterWorkload(name="cfg3" + ("-contiguous" if contiguous else ""), num_tokens=num_tokens,
                           num_heads=num_heads, head_size=head_size, block_size=block_size, num_slots=num_slots,
                           dtype=dtype, slot_mapping=slots, seed=seed)


# ---------------------------------------------------------------- device-side fills (torch)

def torch_dtype(name: str):
    import torch
    return {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32, "fp8": torch.uint8}[name]


def cache_shapes(num_blocks: int, num_kv_heads: int, head_size: int, block_size: int, kv_dtype: str):
    x = 16 // {"bf16": 2, "f16": 2, "f32": 4, "fp8": 1}[kv_dtype]
    return (num_blocks, num_kv_heads, head_size // x, block_size, x), (num_blocks, num_kv_heads, head_size, block_size)


def device_tensors(w: DecodeWorkload, device, seed: Optional[int] = None, chunk_blocks: int = 2048):
    """q, key_cache, value_cache, block_tables, context_lens (+ slopes, k_scale, v_scale) on ``device``.

    Cache values are drawn N(0,1) directly in the paged layout, which has the same
    distribution as scattering N(0,1) keys and values with reshape_and_cache.  For an FP8
    cache the scales are max|x| / 448 over the whole tensor, found in a first pass over
    the same seeded stream."""
    import torch
    g = torch.Generator(device=device)
    seed = w.seed if seed is None else seed
    qdt = torch_dtype(w.dtype)
    kshape, vshape = cache_shapes(w.num_blocks, w.num_kv_heads, w.head_size, w.block_size, w.kv_dtype)
    g.manual_seed(seed)
    q = torch.randn((w.num_seqs, w.num_heads, w.head_size), generator=g, device=device, dtype=torch.float32).to(qdt)
    k_scale = v_scale = 1.0
    per_block = w.num_kv_heads * w.head_size * w.block_size

    def stream(cb):
        g.manual_seed(seed + 1)
        for b0 in range(0, w.num_blocks, chunk_blocks):
            n = min(chunk_blocks, w.num_blocks - b0)
            kc = torch.randn((n, per_block), generator=g, device=device, dtype=torch.float32)
            vc = torch.randn((n, per_block), generator=g, device=device, dtype=torch.float32)
            cb(b0, n, kc, vc)

    if w.kv_dtype == "fp8":
        amax = [0.0, 0.0]

        def first(b0, n, kc, vc):
            amax[0] = max(amax[0], float(kc.to(qdt).float().abs().max()))
            amax[1] = max(amax[1], float(vc.to(qdt).float().abs().max()))
        stream(first)
        k_scale, v_scale = amax[0] / 448.0, amax[1] / 448.0
        key_cache = torch.empty(kshape, device=device, dtype=torch.uint8)
        value_cache = torch.empty(vshape, device=device, dtype=torch.uint8)

        def second(b0, n, kc, vc):
            kq = (kc.to(qdt).float() / k_scale).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
            vq = (vc.to(qdt).float() / v_scale).clamp_(-448.0, 448.0).to(torch.float8_e4m3fn).view(torch.uint8)
            key_cache[b0:b0 + n].view(n, per_block).copy_(kq)
            value_cache[b0:b0 + n].view(n, per_block).copy_(vq)
        stream(second)
    else:
        kvdt = torch_dtype(w.kv_dtype)
        key_cache = torch.empty(kshape, device=device, dtype=kvdt)
        value_cache = torch.empty(vshape, device=device, dtype=kvdt)

        def fill(b0, n, kc, vc):
            key_cache[b0:b0 + n].view(n, per_block).copy_(kc)
            value_cache[b0:b0 + n].view(n, per_block).copy_(vc)
        stream(fill)
    bt = torch.from_numpy(w.block_tables.astype(np.int32)).to(device)
    cl = torch.from_numpy(w.context_lens.astype(np.int32)).to(device)
    slopes = None if w.alibi_slopes is None else torch.from_numpy(w.alibi_slopes).to(device)
    return dict(q=q, key_cache=key_cache, value_cache=value_cache, block_tables=bt, context_lens=cl,
                alibi_slopes=slopes, k_scale=k_scale, v_scale=v_scale)
