"""ctypes front-end of the CPU oracle (test infrastructure, never the product path).

Only the test-suite, the smoke check and the CPU-baseline / reference legs of the
benchmark import this module.  It loads ``oracle/liboracle.so`` (built from
``paged_oracle.c`` by ``make -C oracle``) and offers numpy-level helpers.

Array conventions: 16-bit floats travel as ``uint16`` bit patterns, FP8 as
``uint8``; fp32 as ``float32``.  dtype codes: 0 = f16, 1 = bf16, 2 = f32
(reference: src/kernels/src/pagedattention.cu:723), 3 = FP8 E4M3 (cache only,
no counterpart in the reference).
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "liboracle.so")

F16, BF16, F32, FP8 = 0, 1, 2, 3
ELEM_SIZE = {F16: 2, BF16: 2, F32: 4, FP8: 1}
NP_STORAGE = {F16: np.uint16, BF16: np.uint16, F32: np.float32, FP8: np.uint8}


def build(force: bool = False) -> str:
    src = os.path.join(HERE, "paged_oracle.c")
    if force or not os.path.exists(LIB_PATH) or os.path.getmtime(LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", HERE, "liboracle.so"], stdout=subprocess.DEVNULL)
    return LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = ctypes.CDLL(LIB_PATH)
        L.oracle_e4m3_decode.restype = ctypes.c_float
        L.oracle_e4m3_decode.argtypes = [ctypes.c_uint8]
        L.oracle_e4m3_encode.restype = ctypes.c_uint8
        L.oracle_e4m3_encode.argtypes = [ctypes.c_float]
        L.oracle_f16_decode.restype = ctypes.c_float
        L.oracle_f16_decode.argtypes = [ctypes.c_uint16]
        L.oracle_bf16_decode.restype = ctypes.c_float
        L.oracle_bf16_decode.argtypes = [ctypes.c_uint16]
        L.oracle_max_threads.restype = ctypes.c_int
        L.oracle_set_threads.restype = None
        L.oracle_set_threads.argtypes = [ctypes.c_int]
        vp, i32, u32, f32 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_uint32, ctypes.c_float
        L.oracle_reshape_and_cache.restype = ctypes.c_int
        L.oracle_reshape_and_cache.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, u32, u32, f32, f32]
        attn = [vp, vp, vp, vp, i32, f32, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, u32, u32, f32, vp, f32, f32]
        L.oracle_paged_attention.restype = ctypes.c_int
        L.oracle_paged_attention.argtypes = attn + [i32, i32]
        L.oracle_paged_attention_naive_f32.restype = ctypes.c_int
        L.oracle_paged_attention_naive_f32.argtypes = attn
        L.oracle_prefill_attention.restype = ctypes.c_int
        L.oracle_prefill_attention.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, ctypes.c_int64, ctypes.c_int64,
                                               ctypes.c_int64, u32, f32, f32, vp]
        _lib = L
    return _lib


def max_threads() -> int:
    return int(lib().oracle_max_threads())


def set_threads(n: int) -> None:
    """Thread count of the C routines' parallel regions (overrides an OMP_NUM_THREADS a launcher exported)."""
    lib().oracle_set_threads(int(n))


# ---------------------------------------------------------------- dtype helpers (numpy)

def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    rounded = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return rounded.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def to_storage(a_f32: np.ndarray, dtype: int) -> np.ndarray:
    """fp32 values -> storage array of the given dtype code (RN-even)."""
    if dtype == F32:
        return np.ascontiguousarray(a_f32, dtype=np.float32)
    if dtype == F16:
        return np.ascontiguousarray(a_f32, dtype=np.float32).astype(np.float16).view(np.uint16)
    if dtype == BF16:
        return f32_to_bf16_bits(a_f32)
    raise ValueError(dtype)


def from_storage(a: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == F32:
        return a.astype(np.float32)
    if dtype == F16:
        return a.view(np.float16).astype(np.float32)
    if dtype == BF16:
        return bf16_bits_to_f32(a)
    if dtype == FP8:
        table = np.array([lib().oracle_e4m3_decode(i) for i in range(256)], dtype=np.float32)
        return table[a]
    raise ValueError(dtype)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


# ---------------------------------------------------------------- ops

def cache_shapes(num_blocks, num_kv_heads, head_size, block_size, cache_dtype):
    x = 16 // ELEM_SIZE[cache_dtype]
    return (num_blocks, num_kv_heads, head_size // x, block_size, x), (num_blocks, num_kv_heads, head_size, block_size)


def reshape_and_cache(key, value, key_cache, value_cache, slot_mapping, dtype, cache_dtype=None,
                      k_scale=1.0, v_scale=1.0):
    """In-place scatter into ``key_cache`` / ``value_cache`` (numpy storage arrays)."""
    cache_dtype = dtype if cache_dtype is None else cache_dtype
    nt, nh, hs = key.shape
    if nt == 0:
        return
    assert key.strides[2] == key.itemsize and key.strides[1] == hs * key.itemsize
    assert value.strides[2] == value.itemsize and value.strides[1] == hs * value.itemsize
    nb, nh2, hsx, bs, x = key_cache.shape
    assert nh2 == nh and hsx * x == hs and key_cache.flags.c_contiguous and value_cache.flags.c_contiguous
    sm = np.ascontiguousarray(slot_mapping, dtype=np.int64)
    rc = lib().oracle_reshape_and_cache(_ptr(key), _ptr(value), _ptr(key_cache), _ptr(value_cache), _ptr(sm), nt, nh,
                                        hs, bs, x, key.strides[0] // key.itemsize, value.strides[0] // value.itemsize,
                                        dtype, cache_dtype, k_scale, v_scale)
    if rc != 0:
        raise RuntimeError(f"oracle_reshape_and_cache failed: {rc}")


def paged_attention(query, key_cache, value_cache, block_tables, context_lens, scale, dtype, kv_dtype=None,
                    softcapping=1.0, alibi_slopes=None, k_scale=1.0, v_scale=1.0, partition_size=0,
                    max_context_len=None, naive_f32=False, reference_literal_alibi=False):
    """fp32 output [num_seqs, num_heads, head_size] of the oracle's decode attention."""
    kv_dtype = dtype if kv_dtype is None else kv_dtype
    ns, nh, hs = query.shape
    nb, nkv, hsx, bs, x = key_cache.shape
    assert key_cache.flags.c_contiguous and value_cache.flags.c_contiguous
    assert query.strides[2] == query.itemsize and query.strides[1] == hs * query.itemsize
    bt = np.ascontiguousarray(block_tables, dtype=np.uint32)
    cl = np.ascontiguousarray(context_lens, dtype=np.uint32)
    if max_context_len is None:
        max_context_len = int(cl.max()) if cl.size else 0
    out = np.empty((ns, nh, hs), dtype=np.float32)
    sl = None if alibi_slopes is None else np.ascontiguousarray(alibi_slopes, dtype=np.float32)
    args = [_ptr(out), _ptr(query), _ptr(key_cache), _ptr(value_cache), nkv, scale, _ptr(bt), _ptr(cl), bs,
            max_context_len, ns, nh, hs, bt.shape[1], query.strides[0] // query.itemsize, nkv * hs * bs, hs * bs,
            dtype, kv_dtype, softcapping, _ptr(sl), k_scale, v_scale]
    if naive_f32:
        rc = lib().oracle_paged_attention_naive_f32(*args)
    else:
        rc = lib().oracle_paged_attention(*args, partition_size, 1 if reference_literal_alibi else 0)
    if rc != 0:
        raise RuntimeError(f"oracle_paged_attention failed: {rc}")
    return out


def prefill_attention(q, k, v, cu_seqlens, scale, dtype, softcapping=1.0, alibi_slopes=None):
    """fp32 [tokens, heads, head_size]: causal self-attention over packed prompts (storage arrays in)."""
    nt, nh, hs = q.shape
    nkv = k.shape[1]
    cu = np.ascontiguousarray(cu_seqlens, dtype=np.uint32)
    out = np.zeros((nt, nh, hs), dtype=np.float32)
    sl = None if alibi_slopes is None else np.ascontiguousarray(alibi_slopes, dtype=np.float32)
    rc = lib().oracle_prefill_attention(_ptr(out), _ptr(q), _ptr(k), _ptr(v), _ptr(cu), len(cu) - 1, nh, nkv, hs,
                                        q.strides[0] // q.itemsize, k.strides[0] // k.itemsize,
                                        v.strides[0] // v.itemsize, dtype, scale, softcapping, _ptr(sl))
    if rc != 0:
        raise RuntimeError(f"oracle_prefill_attention failed: {rc}")
    return out


def numpy_prefill_attention(q, k, v, cu_seqlens, scale, softcapping=1.0):
    """fp64 twin of prefill_attention on fp32-decoded inputs; tiny shapes only."""
    nt, nh, hs = q.shape
    group = nh // k.shape[1]
    out = np.zeros((nt, nh, hs), dtype=np.float64)
    for s in range(len(cu_seqlens) - 1):
        lo, hi = int(cu_seqlens[s]), int(cu_seqlens[s + 1])
        n = hi - lo
        mask = np.tril(np.ones((n, n), dtype=bool))
        for h in range(nh):
            logits = (q[lo:hi, h].astype(np.float64) @ k[lo:hi, h // group].astype(np.float64).T) * scale
            if softcapping != 1.0:
                logits = np.tanh(logits / softcapping) * softcapping
            logits = np.where(mask, logits, -np.inf)
            p = np.exp(logits - logits.max(axis=1, keepdims=True))
            out[lo:hi, h] = (p / p.sum(axis=1, keepdims=True)) @ v[lo:hi, h // group].astype(np.float64)
    return out


# ---------------------------------------------------------------- pure-numpy twin (small cases only)

def numpy_reshape_and_cache(key, value, key_cache, value_cache, slot_mapping):
    """Index-by-index restatement of src/kernels/src/reshape_and_cache_kernel.cu:27-58."""
    nt, nh, hs = key.shape
    bs, x = key_cache.shape[3], key_cache.shape[4]
    for t in range(nt):
        slot = int(slot_mapping[t])
        if slot < 0:
            continue
        blk, off = divmod(slot, bs)
        key_cache[blk, :, :, off, :] = key[t].reshape(nh, hs // x, x)
        value_cache[blk, :, :, off] = value[t]


def numpy_paged_attention(q, key_cache, value_cache, block_tables, context_lens, scale, softcapping=1.0,
                          alibi_slopes=None):
    """fp64 attention over fp32-decoded caches; loops in Python, for tiny shapes."""
    ns, nh, hs = q.shape
    nb, nkv, hsx, bs, x = key_cache.shape
    group = nh // nkv
    out = np.zeros((ns, nh, hs), dtype=np.float64)
    for s in range(ns):
        ctx = int(context_lens[s])
        if ctx == 0:
            continue
        nblk = (ctx + bs - 1) // bs
        blocks = block_tables[s, :nblk].astype(np.int64)
        k = key_cache[blocks].transpose(1, 0, 3, 2, 4).reshape(nkv, nblk * bs, hs)[:, :ctx].astype(np.float64)
        v = value_cache[blocks].transpose(1, 0, 3, 2).reshape(nkv, nblk * bs, hs)[:, :ctx].astype(np.float64)
        for h in range(nh):
            logits = (k[h // group] @ q[s, h].astype(np.float64)) * scale
            if softcapping != 1.0:
                logits = np.tanh(logits / softcapping) * softcapping
            if alibi_slopes is not None:
                logits = logits + float(alibi_slopes[h]) * (np.arange(ctx) - ctx + 1)
            p = np.exp(logits - logits.max())
            out[s, h] = (p / p.sum()) @ v[h // group]
    return out
