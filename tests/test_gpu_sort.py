"""asort_*: row-wise argsort through the C ABI against numpy's stable argsort (the oracle for this row:
a restatement of what src/kernels/src/sort.cu computes, with ties resolved by original position)."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TYPES = {"f32": ("float32", np.float32), "f16": ("float16", np.float16), "bf16": ("bfloat16", None),
         "f64": ("float64", np.float64), "u8": ("uint8", np.uint8), "u32": ("uint32", np.uint32), "i64": ("int64", np.int64)}


def reference_order(vals: np.ndarray, asc: bool) -> np.ndarray:
    """Indices that sort each row; equal keys keep their original order, in both directions."""
    out = np.empty(vals.shape, dtype=np.uint32)
    for r in range(vals.shape[0]):
        row = vals[r]
        if asc:
            out[r] = np.argsort(row, kind="stable")
        else:
            # descending with ties by ascending index: sort by (-rank) stably
            order = np.argsort(row, kind="stable")[::-1]            # descending, ties by DEscending index
            # re-stabilise runs of equal keys
            sorted_vals = row[order]
            start = 0
            order = order.copy()
            for i in range(1, len(order) + 1):
                if i == len(order) or sorted_vals[i] != sorted_vals[start]:
                    order[start:i] = np.sort(order[start:i])
                    start = i
            out[r] = order
    return out


@pytest.mark.parametrize("tname", sorted(TYPES))
@pytest.mark.parametrize("asc", [True, False])
@pytest.mark.parametrize("shape", [(3, 1), (4, 37), (2, 4096), (3, 5000), (2, 33000)])
def test_asort_matches_stable_argsort(tname, asc, shape):
    import torch
    from attention_rs_b200 import ops
    L = ops.load_library()
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(shape[1] + len(tname))
    tdt = getattr(torch, TYPES[tname][0])
    if tname in ("f32", "f64", "f16", "bf16"):
        host = torch.from_numpy(rng.standard_normal(shape).astype(np.float32) * 50).to(tdt)
        if tname in ("f16", "bf16"):                                  # few distinct values: many ties
            host = ((host / 8).round() + 0.0).to(tdt)        # + 0.0: no negative zeros (they order before +0 here)
    elif tname == "u8":
        host = torch.from_numpy(rng.integers(0, 256, shape).astype(np.uint8))
    elif tname == "u32":
        host = torch.from_numpy(rng.integers(0, 2**32, shape, dtype=np.uint64).astype(np.uint32).view(np.int32)).view(torch.uint32)
    else:
        host = torch.from_numpy(rng.integers(-2**62, 2**62, shape, dtype=np.int64))
    vals = host.float().numpy().astype(np.float64) if tname in ("f16", "bf16") else (
        host.view(torch.int32).numpy().view(np.uint32) if tname == "u32" else host.numpy())
    want = reference_order(vals, asc)
    fn = getattr(L, f"asort_{'asc' if asc else 'desc'}_{tname}")
    fn.restype = None
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_bool, ctypes.c_int64]
    for inplace in (False, True):
        x = host.to(dev)
        dst = torch.full(shape, 0x7fffffff, dtype=torch.int32, device=dev)
        fn(x.data_ptr(), dst.data_ptr(), shape[0], shape[1], inplace, torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        got = dst.cpu().numpy().view(np.uint32)
        assert np.array_equal(got, want), f"{tname} asc={asc} shape={shape}"
        back = x.cpu()
        if inplace:
            sorted_host = torch.gather(host.view(torch.int32) if tname == "u32" else host, 1, torch.from_numpy(want.astype(np.int64)))
            assert torch.equal(back.view(torch.int32) if tname == "u32" else back, sorted_host)
        else:
            assert torch.equal(back.view(torch.uint8), host.view(torch.uint8))
