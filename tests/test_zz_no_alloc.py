"""paged_attention_v2_static: the partitioned decode path with its scratch inside the library.

Who needs it: hosts that cannot give the library scratch memory - an engine that handed all free
device memory to its KV-cache pool at start-up, or a serving loop that bans cudaMalloc because the
call synchronises the device.  The test calls the entry point through the C ABI twice in a row (the
second call on different inputs, so stale scratch from the first would show) and checks each result
against paged_attention_v2_ex fed with caller-allocated scratch, and against the CPU oracle.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import numpy as np
import pytest

from tests.helpers import case_to_device, from_torch_f32, make_case, tolerances

pytestmark = pytest.mark.gpu


def _tail(q, kc, bt, cl, scale, mcl):
    from attention_rs_b200 import ops
    ns, nh, hs = q.shape
    return [kc.shape[1], float(scale), bt.data_ptr(), cl.data_ptr(), kc.shape[3], int(mcl), ns, nh, hs, bt.shape[1],
            q.stride(0), kc.stride(0), kc.stride(1), ops.dtype_code(q), 1.0]


def _run_both(L, c, dev):
    import torch
    d = case_to_device(c, dev)
    q, kc, vc, bt, cl = d["q"], d["key_cache"], d["value_cache"], d["block_tables"], d["context_lens"]
    mcl = c.max_context_len
    ns, nh, hs = q.shape
    parts = max((mcl + 511) // 512, 1)
    stream = torch.cuda.current_stream().cuda_stream
    slopes = None if d["alibi_slopes"] is None else d["alibi_slopes"].data_ptr()
    from attention_rs_b200 import ops
    kvcode = ops.dtype_code(kc)

    out_static = torch.full(q.shape, float("nan"), dtype=q.dtype, device=dev)
    rc = L.paged_attention_v2_static(out_static.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                                     *_tail(q, kc, bt, cl, c.scale, mcl), slopes, kvcode, c.k_scale, c.v_scale, stream)
    assert rc == 0, L.pa_last_error().decode()

    out_ex = torch.full(q.shape, float("nan"), dtype=q.dtype, device=dev)
    exp_sums = torch.empty((ns, nh, parts), dtype=torch.float32, device=dev)
    max_logits = torch.empty_like(exp_sums)
    tmp_out = torch.empty((ns, nh, parts, hs), dtype=q.dtype, device=dev)
    rc = L.paged_attention_v2_ex(out_ex.data_ptr(), exp_sums.data_ptr(), max_logits.data_ptr(), tmp_out.data_ptr(),
                                 q.data_ptr(), kc.data_ptr(), vc.data_ptr(), *_tail(q, kc, bt, cl, c.scale, mcl), slopes,
                                 kvcode, c.k_scale, c.v_scale, stream)
    assert rc == 0, L.pa_last_error().decode()
    torch.cuda.synchronize()
    return from_torch_f32(out_static), from_torch_f32(out_ex)


def test_static_scratch_entry_point_matches_caller_scratch_twice_in_a_row():
    import torch
    from attention_rs_b200 import ops
    L = ops.load_library()
    dev = torch.device("cuda:0")
    max_tol, mean_tol = tolerances("bf16")
    cases = [make_case([700, 33, 1500, 0, 512], 8, 2, 128, 16, "bf16", seed=101),
             make_case([90, 2100, 513], 16, 4, 128, 16, "bf16", seed=202, alibi=True)]   # other shapes, other data
    for c in cases:
        got, ref = _run_both(L, c, dev)
        assert not np.isnan(got).any()
        err = np.abs(got - ref)
        assert err.max() <= max_tol and err.mean() <= mean_tol, f"static vs caller scratch: max {err.max():.3e}"
        err = np.abs(got - c.expected())
        assert err.max() <= max_tol and err.mean() <= mean_tol, f"static vs oracle: max {err.max():.3e}"
    assert ops.device_status() == 0


def test_static_scratch_refuses_problems_beyond_its_size():
    import torch
    from attention_rs_b200 import ops
    L = ops.load_library()
    dev = torch.device("cuda:0")
    cap = 16 * 1024 * 1024
    # 64 sequences x 32 heads x 64 partitions x (128 x 2 + 8) bytes is well past the 16 MiB array
    assert L.pa_static_scratch_needed(64, 32, 128, 32768, 1) > cap
    assert 0 < L.pa_static_scratch_needed(64, 32, 128, 8192, 1) <= cap
    c = make_case([40], 32, 8, 128, 16, "bf16", seed=303)
    d = case_to_device(c, dev)
    q, kc, vc, bt, cl = d["q"], d["key_cache"], d["value_cache"], d["block_tables"], d["context_lens"]
    out = torch.zeros_like(q)
    tail = _tail(q, kc, bt, cl, c.scale, 32768)
    tail[6] = 64            # claim 64 sequences: rejected on size before anything is launched
    rc = L.paged_attention_v2_static(out.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), *tail, None, 1, 1.0,
                                     1.0, torch.cuda.current_stream().cuda_stream)
    assert rc == 4 and b"built-in array holds" in L.pa_last_error()
    torch.cuda.synchronize()
