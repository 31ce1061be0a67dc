"""Generates the golden fixtures of tests/golden/ by running the REFERENCE's own CUDA kernels.

The reference ships no tests or golden vectors, and it cannot run on a machine without a GPU, so
the fixtures are made on a B200: this script builds small seeded inputs, runs the reference kernels
compiled unchanged (oracle/_ref/libref_pa.so, plus the ALiBi harness oracle/_ref/libref_alibi.so;
both built by `make -C oracle ref` where the reference checkout is present) and stores inputs and
reference outputs.  The CPU tests then check the oracle against these files.

    python tests/golden/make_golden.py --out <dir>

Each fixture holds: the scattered key/value rows, slot mapping, block tables, context lengths, query
(all as raw storage arrays), the reference's attention outputs (v1 and v2 entry points) as raw
storage arrays, and the SHA-256 of the key / value cache bytes its reshape_and_cache wrote into a
zero-initialised cache.
"""
from __future__ import annotations

import argparse
import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

CASES = [
    # name, ctx, heads, kv heads, head size, block size, dtype, softcap, alibi, pad slots
    ("bf16_gqa_d64_bs16", [1, 17, 100, 530], 4, 2, 64, 16, "bf16", 1.0, False),
    ("f16_mha_d128_bs32", [33, 600], 2, 2, 128, 32, "f16", 1.0, False),
    ("f32_mqa_d64_bs8", [5, 260], 4, 1, 64, 8, "f32", 1.0, False),
    ("bf16_softcap_d64_bs16", [20, 520], 4, 2, 64, 16, "bf16", 30.0, False),
    ("bf16_alibi_d128_bs16", [40, 700], 4, 2, 128, 16, "bf16", 1.0, True),
    ("f16_alibi_d64_bs32", [70, 1100], 8, 2, 64, 32, "f16", 1.0, True),
]


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).view(np.uint8).tobytes()).hexdigest()


def main() -> None:
    import torch

    from oracle import oracle as O
    from oracle import ref_gpu
    from tests.helpers import DT, make_case, to_torch

    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    args = ap.parse_args()
    os.makedirs(args.out, exist_ok=True)
    assert ref_gpu.available(), "oracle/_ref/libref_pa.so is missing: run `make -C oracle ref` where the reference is"
    dev = torch.device("cuda:0")

    def storage(t, dt):
        if dt == O.F32:
            return t.cpu().numpy()
        return t.view(torch.int16).cpu().numpy().view(np.uint16)

    for i, (name, ctx, nh, nkv, hs, bs, dtype, softcap, alibi) in enumerate(CASES):
        c = make_case(ctx, nh, nkv, hs, bs, dtype, seed=1000 + i, softcapping=softcap, alibi=alibi, poison=False)
        dt = DT[dtype]
        # a few padding tokens appended to the scatter input: they must leave the cache untouched
        rng = np.random.default_rng(2000 + i)
        npad = 3
        key = np.concatenate([c.key, O.to_storage(rng.standard_normal((npad, nkv, hs), dtype=np.float32), dt)])
        value = np.concatenate([c.value, O.to_storage(rng.standard_normal((npad, nkv, hs), dtype=np.float32), dt)])
        slots = np.concatenate([c.slot_mapping, np.full(npad, -1, dtype=np.int64)])
        order = rng.permutation(len(slots))
        key, value, slots = key[order], value[order], slots[order]

        tkey, tvalue = to_torch(key, dt, dev), to_torch(value, dt, dev)
        kc = torch.zeros(c.key_cache.shape, dtype=tkey.dtype, device=dev)
        vc = torch.zeros(c.value_cache.shape, dtype=tkey.dtype, device=dev)
        ref_gpu.reshape_and_cache(tkey, tvalue, kc, vc, torch.from_numpy(slots).to(dev))
        torch.cuda.synchronize()
        q = to_torch(c.q, dt, dev)
        bt = torch.from_numpy(c.block_tables.astype(np.int32)).to(dev)
        cl = torch.from_numpy(c.context_lens.astype(np.int32)).to(dev)
        slopes = None if c.alibi_slopes is None else torch.from_numpy(c.alibi_slopes).to(dev)
        out = {}
        if slopes is None:
            o1 = torch.zeros_like(q)
            ref_gpu.paged_attention_v1(o1, q, kc, vc, bt, cl, c.max_context_len, c.scale, softcap)
            out["ref_out_v1"] = storage(o1, dt)
        o2 = torch.zeros_like(q)
        ref_gpu.paged_attention_v2(o2, q, kc, vc, bt, cl, c.max_context_len, c.scale, softcap, alibi_slopes=slopes)
        torch.cuda.synchronize()
        out["ref_out_v2"] = storage(o2, dt)
        path = os.path.join(args.out, name + ".npz")
        np.savez_compressed(
            path, dtype=np.int32(dt), num_kv_heads=np.int32(nkv), block_size=np.int32(bs), scale=np.float32(c.scale),
            softcapping=np.float32(softcap), key=key, value=value, slot_mapping=slots, q=c.q,
            block_tables=c.block_tables, context_lens=c.context_lens, num_blocks=np.int32(c.key_cache.shape[0]),
            alibi_slopes=c.alibi_slopes if c.alibi_slopes is not None else np.zeros(0, dtype=np.float32),
            ref_key_cache_sha256=np.array(sha(storage(kc, dt))), ref_value_cache_sha256=np.array(sha(storage(vc, dt))),
            **out)
        print(f"wrote {path} ({os.path.getsize(path)} bytes)")


if __name__ == "__main__":
    main()
