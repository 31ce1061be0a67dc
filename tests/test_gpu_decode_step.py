"""The fused decode step (scatter of the step's token folded into the attention kernel) must reproduce
reshape_and_cache followed by paged_attention exactly: same output bits, same cache bytes."""
import numpy as np
import pytest

from tests.helpers import case_to_device, from_torch_f32, make_case, to_torch, tolerances, torch_bits

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    import torch
    return torch.device("cuda:0")


def run(dev, ctx, nh, nkv, hs, bs, dtype, kv=None, alibi=False, softcap=1.0, seed=0, stride_pad=0):
    import torch
    import attention_rs_b200 as pa
    c = make_case(ctx, nh, nkv, hs, bs, dtype, kv, seed=seed, alibi=alibi, softcapping=softcap, poison=False)
    d = case_to_device(c, dev)
    ns = len(ctx)
    # the newest token of every sequence: its rows, and the slot the block table gives it
    last = [int(sum(ctx[:i + 1])) - 1 for i in range(ns)]
    rows = [l for l, n in zip(last, ctx) if n > 0]
    key_all, value_all = to_torch(c.key, c.dtype, dev), to_torch(c.value, c.dtype, dev)
    new_k = torch.zeros((ns, nkv + stride_pad, hs), dtype=key_all.dtype, device=dev)
    new_v = torch.zeros_like(new_k)
    live = torch.tensor([i for i, n in enumerate(ctx) if n > 0], device=dev, dtype=torch.long)
    if len(rows):
        new_k[live, :nkv] = key_all[torch.tensor(rows, device=dev)]
        new_v[live, :nkv] = value_all[torch.tensor(rows, device=dev)]
    new_k, new_v = new_k[:, :nkv], new_v[:, :nkv]
    slots = torch.full((ns,), -1, dtype=torch.int64, device=dev)
    if len(rows):
        slots[live] = torch.from_numpy(c.slot_mapping[rows]).to(dev)
    # caches as they were BEFORE the step: the newest token's slot holds garbage
    kc0, vc0 = d["key_cache"].clone(), d["value_cache"].clone()
    junk_k, junk_v = torch.zeros_like(new_k), torch.zeros_like(new_v)
    junk_k += 3.0
    junk_v -= 2.0
    pa.reshape_and_cache(junk_k, junk_v, kc0, vc0, slots, c.k_scale, c.v_scale)
    args = (d["block_tables"], d["context_lens"], d["alibi_slopes"], c.max_context_len, c.scale, c.softcapping,
            c.k_scale, c.v_scale)
    # reference sequence: two calls
    kc_a, vc_a = kc0.clone(), vc0.clone()
    pa.reshape_and_cache(new_k, new_v, kc_a, vc_a, slots, c.k_scale, c.v_scale)
    out_a = pa.paged_attention(d["q"], kc_a, vc_a, *args)
    # fused
    kc_b, vc_b = kc0.clone(), vc0.clone()
    out_b = pa.decode_step(d["q"], new_k, new_v, kc_b, vc_b, *args)
    torch.cuda.synchronize()
    assert np.array_equal(torch_bits(kc_a), torch_bits(kc_b)), "key cache bytes differ"
    assert np.array_equal(torch_bits(vc_a), torch_bits(vc_b)), "value cache bytes differ"
    assert np.array_equal(torch_bits(out_a), torch_bits(out_b)), "outputs differ"
    assert np.array_equal(torch_bits(kc_b), torch_bits(d["key_cache"]))          # and equal to the oracle-built cache
    mx, mean = tolerances(dtype, kv)
    err = np.abs(from_torch_f32(out_b) - c.expected())
    assert err.max() <= mx and err.mean() <= mean


@pytest.mark.parametrize("dtype,kv", [("bf16", None), ("f16", None), ("bf16", "fp8"), ("f16", "fp8")])
@pytest.mark.parametrize("bs", [16, 32])
def test_fused_step_matches_two_calls(dev, dtype, kv, bs):
    run(dev, [1, 16, 17, 33, 512, 513, 1500, 0, 700], 8, 2, 128, bs, dtype, kv, seed=bs)


def test_fused_step_variants(dev):
    run(dev, [5, 1030, 64], 8, 2, 128, 8, "bf16", seed=1)                    # block size 8: two blocks per stage
    run(dev, [9, 2000], 4, 4, 64, 16, "f16", seed=2, alibi=True, softcap=25.0)
    run(dev, [300, 31], 12, 1, 128, 16, "bf16", seed=3)                      # two n-tiles of heads
    run(dev, [300, 31], 40, 2, 128, 16, "bf16", seed=4)                      # several CTAs per kv head
    run(dev, [100, 900], 8, 2, 128, 16, "bf16", seed=5, stride_pad=2)        # rows sliced out of a fused tensor
    run(dev, [77, 600], 4, 2, 80, 16, "bf16", seed=6)
    run(dev, [77, 600], 4, 2, 128, 16, "f32", seed=7)                        # generic route (scatter + attention)
    run(dev, [77, 600], 4, 2, 80, 16, "bf16", "fp8", seed=8)                 # generic route, FP8
