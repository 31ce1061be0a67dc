"""CPU tests of the oracle: codecs, layouts, the attention restatement against an independent
numpy twin, and - the pin - against outputs of the reference's own CUDA kernels (tests/golden/)."""
import glob
import hashlib
import os

import numpy as np
import pytest

from oracle import oracle as O
from tests.helpers import make_case

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def test_e4m3_decode_table_matches_torch():
    torch = pytest.importorskip("torch")
    if not hasattr(torch, "float8_e4m3fn"):
        pytest.skip("torch without float8_e4m3fn")
    codes = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    want = codes.view(torch.float8_e4m3fn).float().numpy()
    got = O.from_storage(np.arange(256, dtype=np.uint8), O.FP8)
    assert np.array_equal(np.isnan(got), np.isnan(want))
    ok = ~np.isnan(want)
    assert np.array_equal(got[ok], want[ok])
    assert np.array_equal(np.signbit(got[ok]), np.signbit(want[ok]))


def test_e4m3_encode_round_trips_and_rounds_to_nearest_even():
    L = O.lib()
    table = O.from_storage(np.arange(256, dtype=np.uint8), O.FP8)
    for code in range(256):
        if np.isnan(table[code]):
            continue
        assert L.oracle_e4m3_encode(float(table[code])) == code
    finite = np.sort(table[:0x7f])          # positive codes
    for lo, hi in zip(finite[:-1], finite[1:]):
        mid = (np.float64(lo) + np.float64(hi)) / 2
        lo_code, hi_code = L.oracle_e4m3_encode(float(lo)), L.oracle_e4m3_encode(float(hi))
        even = lo_code if lo_code % 2 == 0 else hi_code
        assert L.oracle_e4m3_encode(float(mid)) == even                         # tie -> even mantissa
        assert L.oracle_e4m3_encode(float(np.nextafter(np.float32(mid), np.float32(0)))) == lo_code
        assert L.oracle_e4m3_encode(float(np.nextafter(np.float32(mid), np.float32(1e9)))) == hi_code
    assert L.oracle_e4m3_encode(1e9) == 0x7e and L.oracle_e4m3_encode(-1e9) == 0xfe      # saturate to +-448
    assert L.oracle_e4m3_encode(463.9) == 0x7e and L.oracle_e4m3_encode(float("nan")) & 0x7f == 0x7f


def test_e4m3_encode_matches_torch_on_random_values():
    torch = pytest.importorskip("torch")
    if not hasattr(torch, "float8_e4m3fn"):
        pytest.skip("torch without float8_e4m3fn")
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(20000) * s for s in (1e-3, 0.05, 1.0, 30.0, 200.0)]).astype(np.float32)
    x = x[np.abs(x) < 448]
    want = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = np.array([O.lib().oracle_e4m3_encode(float(v)) for v in x], dtype=np.uint8)
    assert np.array_equal(got, want)


def test_f16_bf16_decode():
    rng = np.random.default_rng(1)
    bits = rng.integers(0, 65536, size=5000).astype(np.uint16)
    want16 = bits.view(np.float16).astype(np.float32)
    got16 = np.array([O.lib().oracle_f16_decode(int(b)) for b in bits], dtype=np.float32)
    assert np.array_equal(np.isnan(got16), np.isnan(want16)) and np.array_equal(got16[~np.isnan(want16)], want16[~np.isnan(want16)])
    wantb = O.bf16_bits_to_f32(bits)
    gotb = np.array([O.lib().oracle_bf16_decode(int(b)) for b in bits], dtype=np.float32)
    okb = ~np.isnan(wantb)      # signalling-NaN payloads may be quieted on their way through a C float return
    assert np.array_equal(np.isnan(gotb), np.isnan(wantb))
    assert np.array_equal(gotb[okb].view(np.uint32), wantb[okb].view(np.uint32))


@pytest.mark.parametrize("dtype", [O.F16, O.BF16, O.F32])
@pytest.mark.parametrize("block_size", [8, 16, 32])
def test_reshape_and_cache_matches_numpy_twin(dtype, block_size):
    rng = np.random.default_rng(block_size + dtype)
    nt, nh, hs = 50, 3, 64
    key = O.to_storage(rng.standard_normal((nt, nh, hs), dtype=np.float32), dtype)
    value = O.to_storage(rng.standard_normal((nt, nh, hs), dtype=np.float32), dtype)
    slots = rng.permutation(12 * block_size)[:nt].astype(np.int64)
    slots[rng.random(nt) < 0.2] = -1
    kshape, vshape = O.cache_shapes(12, nh, hs, block_size, dtype)
    kc = rng.integers(0, 60000, size=kshape).astype(O.NP_STORAGE[dtype])
    vc = rng.integers(0, 60000, size=vshape).astype(O.NP_STORAGE[dtype])
    kc2, vc2 = kc.copy(), vc.copy()
    O.reshape_and_cache(key, value, kc, vc, slots, dtype)
    O.numpy_reshape_and_cache(key, value, kc2, vc2, slots)
    assert np.array_equal(kc.view(np.uint8), kc2.view(np.uint8)) and np.array_equal(vc.view(np.uint8), vc2.view(np.uint8))


def test_reshape_and_cache_strided_rows_and_fp8():
    rng = np.random.default_rng(3)
    nt, nh, hs, bs = 20, 2, 32, 16
    fused = O.to_storage(rng.standard_normal((nt, nh + 3, hs), dtype=np.float32), O.BF16)
    key = fused[:, 1:1 + nh]
    slots = np.arange(nt, dtype=np.int64) + 7
    kshape, vshape = O.cache_shapes(3, nh, hs, bs, O.FP8)
    kc, vc = np.zeros(kshape, dtype=np.uint8), np.zeros(vshape, dtype=np.uint8)
    O.reshape_and_cache(key, key, kc, vc, slots, O.BF16, O.FP8, 0.02, 0.03)
    vals = O.from_storage(np.ascontiguousarray(key), O.BF16)
    want_v = np.array([O.lib().oracle_e4m3_encode(float(np.float32(v) / np.float32(0.03))) for v in vals.reshape(-1)],
                      dtype=np.uint8).reshape(nt, nh, hs)
    for t in range(nt):
        blk, off = divmod(int(slots[t]), bs)
        assert np.array_equal(vc[blk, :, :, off], want_v[t])
        got_k = kc[blk, :, :, off, :].reshape(nh, hs)
        want_k = np.array([O.lib().oracle_e4m3_encode(float(np.float32(v) / np.float32(0.02))) for v in vals[t].reshape(-1)],
                          dtype=np.uint8).reshape(nh, hs)
        assert np.array_equal(got_k, want_k)


@pytest.mark.parametrize("dtype,kv", [("bf16", None), ("f16", None), ("f32", None), ("bf16", "fp8")])
@pytest.mark.parametrize("block_size", [8, 16, 32])
def test_attention_matches_numpy_twin(dtype, kv, block_size):
    c = make_case([0, 1, 15, 16, 17, 130], 6, 2, 32, block_size, dtype, kv, seed=block_size, softcapping=20.0, alibi=True)
    want = O.numpy_paged_attention(O.from_storage(c.q, c.dtype), O.from_storage(c.key_cache, c.kv_dtype) * c.k_scale,
                                   O.from_storage(c.value_cache, c.kv_dtype) * c.v_scale, c.block_tables, c.context_lens,
                                   c.scale, c.softcapping, c.alibi_slopes)
    got = c.expected()
    assert np.abs(got - want).max() < 2e-6
    assert (got[0] == 0).all()                                    # empty context -> zeros


def test_partitioned_equals_single_pass():
    c = make_case([5, 511, 512, 513, 1700], 4, 2, 64, 16, "bf16", seed=9, alibi=True)
    a, b, d = c.expected(0), c.expected(512), c.expected(64)
    assert np.abs(a - b).max() < 1e-6 and np.abs(a - d).max() < 1e-6


def test_naive_fp32_variant_agrees():
    c = make_case([3, 200, 900], 8, 2, 128, 16, "bf16", seed=10, softcapping=15.0, alibi=True)
    a = c.expected()
    b = O.paged_attention(c.q, c.key_cache, c.value_cache, c.block_tables, c.context_lens, c.scale, c.dtype,
                          c.kv_dtype, c.softcapping, c.alibi_slopes, naive_f32=True)
    assert np.abs(a - b).max() < 1e-5


def test_poisoned_cache_never_read_past_context():
    c = make_case([1, 17, 40], 4, 2, 32, 16, "f16", seed=11, poison=True)
    assert not np.isnan(c.expected()).any()


# ---------------------------------------------------------------- the pin: reference kernel outputs

def _sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).view(np.uint8).tobytes()).hexdigest()


def test_golden_fixtures_present():
    assert len(GOLDEN) >= 5, "golden fixtures (outputs of the reference's CUDA kernels) are missing"


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_oracle_against_reference_kernel_outputs(path):
    g = np.load(path)
    dt = int(g["dtype"])
    nkv, bs = int(g["num_kv_heads"]), int(g["block_size"])
    key, value, slots, q = g["key"], g["value"], g["slot_mapping"], g["q"]
    hs = q.shape[2]
    kshape, vshape = O.cache_shapes(int(g["num_blocks"]), nkv, hs, bs, dt)
    kc, vc = np.zeros(kshape, dtype=O.NP_STORAGE[dt]), np.zeros(vshape, dtype=O.NP_STORAGE[dt])
    O.reshape_and_cache(key, value, kc, vc, slots, dt)
    # cache bytes: bit-exact with what the reference's reshape_and_cache kernel wrote
    assert _sha(kc) == str(g["ref_key_cache_sha256"])
    assert _sha(vc) == str(g["ref_value_cache_sha256"])
    slopes = g["alibi_slopes"] if g["alibi_slopes"].size else None
    # With slopes the reference's kernel evaluates its bias in unsigned arithmetic (see the header of
    # oracle/paged_oracle.c); the oracle reproduces that literal expression for this comparison only.
    got = O.paged_attention(q, kc, vc, g["block_tables"], g["context_lens"], float(g["scale"]), dt,
                            softcapping=float(g["softcapping"]), alibi_slopes=slopes,
                            reference_literal_alibi=slopes is not None)
    max_tol, mean_tol = (1e-4, 1e-5) if dt == O.F32 else (2e-2, 2e-3)
    for name in ("ref_out_v1", "ref_out_v2"):
        if name not in g.files:
            continue
        ref = O.from_storage(g[name], dt)
        err = np.abs(got - ref)
        assert err.max() <= max_tol and err.mean() <= mean_tol, f"{name}: max {err.max():.3e} mean {err.mean():.3e}"


def test_prefill_oracle_matches_numpy_twin():
    rng = np.random.default_rng(21)
    lens = [1, 17, 40]
    nt = sum(lens)
    cu = np.concatenate([[0], np.cumsum(lens)]).astype(np.uint32)
    q = O.to_storage(rng.standard_normal((nt, 4, 32), dtype=np.float32), O.BF16)
    k = O.to_storage(rng.standard_normal((nt, 2, 32), dtype=np.float32), O.BF16)
    v = O.to_storage(rng.standard_normal((nt, 2, 32), dtype=np.float32), O.BF16)
    got = O.prefill_attention(q, k, v, cu, 0.2, O.BF16, softcapping=15.0)
    want = O.numpy_prefill_attention(O.from_storage(q, O.BF16), O.from_storage(k, O.BF16), O.from_storage(v, O.BF16), cu,
                                     0.2, softcapping=15.0)
    assert np.abs(got - want).max() < 2e-6
    # the last row of a sequence attends over the whole sequence; the first only over itself
    assert np.allclose(got[0], np.repeat(O.from_storage(v, O.BF16)[0], 2, axis=0), atol=1e-6)


def test_thread_count_can_be_set():
    """The timed CPU legs ask for every host core even when a launcher exported OMP_NUM_THREADS=1."""
    before = O.max_threads()
    O.set_threads(3)
    assert O.max_threads() == 3
    O.set_threads(before)
    assert O.max_threads() == before
