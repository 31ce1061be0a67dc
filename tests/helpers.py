"""Small-case builders shared by the tests: inputs in numpy, expected values from the oracle."""
from __future__ import annotations

import dataclasses
import math
from typing import Optional, Sequence

import numpy as np

from oracle import oracle as O

DT = {"f16": O.F16, "bf16": O.BF16, "f32": O.F32, "fp8": O.FP8}


@dataclasses.dataclass
class Case:
    dtype: int
    kv_dtype: int
    q: np.ndarray              # storage array [ns, nh, hs]
    key_cache: np.ndarray      # storage, paged layout
    value_cache: np.ndarray
    block_tables: np.ndarray   # uint32 [ns, max_blocks]
    context_lens: np.ndarray   # uint32 [ns]
    scale: float
    softcapping: float = 1.0
    alibi_slopes: Optional[np.ndarray] = None
    k_scale: float = 1.0
    v_scale: float = 1.0
    key: Optional[np.ndarray] = None      # the rows that were scattered (storage arrays)
    value: Optional[np.ndarray] = None
    slot_mapping: Optional[np.ndarray] = None

    @property
    def max_context_len(self) -> int:
        return int(self.context_lens.max()) if self.context_lens.size else 0

    def expected(self, partition_size: int = 0) -> np.ndarray:
        return O.paged_attention(self.q, self.key_cache, self.value_cache, self.block_tables, self.context_lens,
                                 self.scale, self.dtype, self.kv_dtype, self.softcapping, self.alibi_slopes,
                                 self.k_scale, self.v_scale, partition_size, self.max_context_len)


def make_case(ctx: Sequence[int], num_heads: int, num_kv_heads: int, head_size: int, block_size: int,
              dtype: str = "bf16", kv_dtype: Optional[str] = None, seed: int = 0, softcapping: float = 1.0,
              alibi: bool = False, extra_blocks: int = 3, poison: bool = True, q_scale: float = 1.0) -> Case:
    """Random decode case whose cache is filled THROUGH the oracle's reshape_and_cache: tokens of every
    sequence are scattered to the slots its block table dictates.  Unwritten cache bytes are poisoned
    with NaN patterns so that reads past a context show up."""
    rng = np.random.default_rng(seed)
    dt, kvdt = DT[dtype], DT[kv_dtype or dtype]
    ctx = np.asarray(ctx, dtype=np.uint32)
    ns = len(ctx)
    need = (ctx.astype(np.int64) + block_size - 1) // block_size
    nb = int(need.sum()) + extra_blocks
    perm = rng.permutation(nb).astype(np.uint32)
    max_blocks = max(int(need.max()) if ns else 1, 1) + 1
    tables = np.full((ns, max_blocks), 0, dtype=np.uint32)
    pos = 0
    slots = []
    for s in range(ns):
        tables[s, :need[s]] = perm[pos:pos + need[s]]
        pos += int(need[s])
        t = np.arange(int(ctx[s]))
        slots.append(tables[s, t // block_size].astype(np.int64) * block_size + t % block_size)
    slot_mapping = np.concatenate(slots) if slots else np.zeros(0, dtype=np.int64)
    ntok = len(slot_mapping)
    q = O.to_storage(rng.standard_normal((ns, num_heads, head_size), dtype=np.float32) * q_scale, dt)
    key = O.to_storage(rng.standard_normal((ntok, num_kv_heads, head_size), dtype=np.float32), dt)
    value = O.to_storage(rng.standard_normal((ntok, num_kv_heads, head_size), dtype=np.float32), dt)
    kshape, vshape = O.cache_shapes(nb, num_kv_heads, head_size, block_size, kvdt)
    fill = {O.F16: 0x7E00, O.BF16: 0x7FC0, O.FP8: 0x7F}.get(kvdt) if poison else 0
    if kvdt == O.F32:
        kc = np.full(kshape, np.nan if poison else 0.0, dtype=np.float32)
        vc = np.full(vshape, np.nan if poison else 0.0, dtype=np.float32)
    else:
        kc = np.full(kshape, fill, dtype=O.NP_STORAGE[kvdt])
        vc = np.full(vshape, fill, dtype=O.NP_STORAGE[kvdt])
    k_scale = v_scale = 1.0
    if kvdt == O.FP8:
        k_scale = float(np.abs(O.from_storage(key, dt)).max()) / 448.0 if ntok else 1.0
        v_scale = float(np.abs(O.from_storage(value, dt)).max()) / 448.0 if ntok else 1.0
    if ntok:
        O.reshape_and_cache(key, value, kc, vc, slot_mapping, dt, kvdt, k_scale, v_scale)
    slopes = None
    if alibi:
        slopes = np.array([2.0 ** (-8.0 * (i + 1) / num_heads) for i in range(num_heads)], dtype=np.float32)
    return Case(dt, kvdt, q, kc, vc, tables, ctx, 1.0 / math.sqrt(head_size), softcapping, slopes, k_scale, v_scale,
                key, value, slot_mapping)


def tolerances(dtype: str, kv_dtype: Optional[str] = None):
    """(max-abs, mean-abs) bounds against the fp32 oracle: 2e-2 / 2e-3 for f16 / bf16 tensors, 6e-2 for an
    FP8 cache (mean bound scaled alike), 1e-4 / 1e-5 for f32."""
    if (kv_dtype or dtype) == "fp8":
        return 6e-2, 6e-3
    if dtype == "f32":
        return 1e-4, 1e-5
    return 2e-2, 2e-3


# ---------------------------------------------------------------- numpy <-> torch (GPU tests)

def to_torch(a: np.ndarray, dtype: int, device):
    import torch
    if dtype == O.F32:
        return torch.from_numpy(np.ascontiguousarray(a)).to(device)
    if dtype == O.FP8:
        return torch.from_numpy(np.ascontiguousarray(a)).to(device)          # uint8
    tdt = torch.float16 if dtype == O.F16 else torch.bfloat16
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16)).to(device).view(tdt)


def from_torch_f32(t) -> np.ndarray:
    return t.detach().float().cpu().numpy()


def torch_bits(t) -> np.ndarray:
    """Raw bytes of a tensor as a numpy uint8 array (for bit-exact comparisons)."""
    import torch
    return t.detach().contiguous().view(torch.uint8).cpu().numpy()


def case_to_device(c: Case, device):
    import torch
    d = dict(q=to_torch(c.q, c.dtype, device), key_cache=to_torch(c.key_cache, c.kv_dtype, device),
             value_cache=to_torch(c.value_cache, c.kv_dtype, device),
             block_tables=torch.from_numpy(c.block_tables.astype(np.int32)).to(device),
             context_lens=torch.from_numpy(c.context_lens.astype(np.int32)).to(device),
             alibi_slopes=None if c.alibi_slopes is None else torch.from_numpy(c.alibi_slopes).to(device))
    return d
