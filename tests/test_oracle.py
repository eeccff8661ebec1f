"""The CPU oracle against independent implementations: storage codecs vs numpy / ml_dtypes /
torch, and the C loop vs a numpy float64 product.  (The reference has no GEMM arithmetic of its
own, so these pins are what stands behind the oracle: numerics parity is otherwise unpinned.)"""
import numpy as np
import pytest

from frisk_b200 import workloads as W
from oracle import ref


def test_e4m3_decode_all_codes_match_ml_dtypes():
    ml_dtypes = pytest.importorskip("ml_dtypes")
    codes = np.arange(256, dtype=np.uint8)
    want = codes.view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    got_c = np.array([ref.lib().frisk_ref_decode_e4m3(int(c)) for c in codes], dtype=np.float32)
    got_np = W.e4m3_decode(codes)
    for got in (got_c, got_np):
        assert np.array_equal(np.isnan(got), np.isnan(want))
        assert np.array_equal(got[~np.isnan(want)], want[~np.isnan(want)])


def test_e4m3_encode_matches_torch_and_saturates():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(0)
    x = np.concatenate([
        (rng.standard_normal(100000) * 50).astype(np.float32),
        np.array([0.0, -0.0, 448, 449, 464, 465, 480, 1e9, -1e9, 2.0 ** -9, 2.0 ** -10,
                  1.5 * 2.0 ** -9, 2.0 ** -10 * 1.0001, 0.0009765625], dtype=np.float32)])
    mine = W.e4m3_encode(x)
    want = torch.from_numpy(np.clip(x, -448, 448)).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(mine, want)
    assert np.all(np.abs(W.e4m3_decode(mine)) <= 448.0)
    assert not np.any(np.isnan(W.e4m3_decode(mine)))


def test_e5m2_codecs_match_torch_and_saturate():
    """e5m2 is the top byte of an IEEE half: all 256 codes decode as torch's float8_e5m2 does (C
    oracle and numpy alike); the encoder rounds to nearest even and saturates at +-57344."""
    torch = pytest.importorskip("torch")
    codes = np.arange(256, dtype=np.uint8)
    want = torch.from_numpy(codes).view(torch.float8_e5m2).to(torch.float32).numpy()
    got_c = np.array([ref.lib().frisk_ref_decode_e5m2(int(c)) for c in codes], dtype=np.float32)
    for got in (got_c, W.e5m2_decode(codes)):
        assert np.array_equal(np.isnan(got), np.isnan(want))
        assert np.array_equal(got[~np.isnan(want)], want[~np.isnan(want)])
    rng = np.random.default_rng(2)
    x = np.concatenate([
        (rng.standard_normal(100000) * 10.0 ** rng.integers(-6, 5, 100000)).astype(np.float32),
        np.array([0.0, -0.0, 57344, 57345, 61439, 61440, 65536, 1e9, -1e9, 2.0 ** -16, 2.0 ** -17,
                  1.5 * 2.0 ** -16, 2.0 ** -17 * 1.0001, 2.0 ** -14, 1.25, 1.375, 1.125], dtype=np.float32)])
    mine = W.e5m2_encode(x)
    want = torch.from_numpy(np.clip(x, -57344, 57344)).to(torch.float8_e5m2).view(torch.uint8).numpy()
    assert np.array_equal(mine, want)
    dec = W.e5m2_decode(mine)
    assert np.all(np.abs(dec) <= 57344.0) and not np.any(np.isnan(dec))


def test_bf16_and_f16_codecs_match_torch():
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(1)
    x = np.concatenate([(rng.standard_normal(200000) * 10).astype(np.float32),
                        np.array([0, -0.0, 65504, 65519.9, 65520, 1e-8, 5.96e-8, 2.98e-8, 2.9803e-8,
                                  6.1e-5, 6.0975e-5, 1e30, -1e30, np.inf, -np.inf], dtype=np.float32)])
    t = torch.from_numpy(x)
    bf_want = t.to(torch.bfloat16).view(torch.uint16).numpy()
    assert np.array_equal(W.bf16_encode(x), bf_want)
    L = ref.lib()
    bf_c = np.array([L.frisk_ref_encode_bf16(float(v)) for v in x[:5000]], dtype=np.uint16)
    assert np.array_equal(bf_c, bf_want[:5000])
    h_want = t.to(torch.float16).view(torch.uint16).numpy()
    sel = np.concatenate([np.arange(5000), np.arange(len(x) - 15, len(x))])
    h_c = np.array([L.frisk_ref_encode_f16(float(x[i])) for i in sel], dtype=np.uint16)
    assert np.array_equal(h_c, h_want[sel])
    # decoders: every bf16 code via the table identity, a sweep of fp16 codes
    codes = np.arange(0, 65536, 7, dtype=np.uint16)
    h_dec = np.array([L.frisk_ref_decode_f16(int(c)) for c in codes], dtype=np.float32)
    want = codes.view(np.float16).astype(np.float32)
    assert np.array_equal(np.isnan(h_dec), np.isnan(want))
    assert np.array_equal(h_dec[~np.isnan(want)], want[~np.isnan(want)])


@pytest.mark.parametrize("name,dims", [
    ("cfg1", (64, 48, 80)), ("cfg1", (1, 1, 1)), ("cfg1", (7, 513, 3)),
    ("cfg2", (40, 56, 64)), ("cfg3", (16, 256, 128)), ("cfg4", (32, 64, 128)),
    ("cfg5", (70, 64, 96)), ("bf16_8192", (33, 17, 65)),
])
def test_c_loop_matches_numpy_float64(name, dims):
    w = W.make_workload(name, *dims)
    got = W.decode(ref.ref_gemm(w), w.c_type)
    want = ref.ref_gemm_f64(w)
    ok, err, metric = W.check(got, want, w.ab_type, absdot=ref.abs_dot(w))
    assert ok, f"{metric} = {err}"
    # the float64-accumulate variant differs from numpy only by the final cast
    got64 = W.decode(ref.ref_gemm(w, acc64=True), w.c_type)
    tol = {W.F32: 1e-6, W.F16: 1e-3, W.BF16: 8e-3}[w.c_type]
    assert np.all(np.abs(got64 - want) <= tol * np.abs(want) + 1e-30)


def test_c_loop_takes_e5m2_inputs():
    """cfg4's form with the other 8-bit float: the C loop against numpy float64 on the decoded bits."""
    w = W.make_workload("cfg4", 32, 64, 128)
    w.A, w.B, w.ab_type = W.encode(W.decode(w.A, W.E4M3), W.E5M2), W.encode(W.decode(w.B, W.E4M3), W.E5M2), W.E5M2
    got = W.decode(ref.ref_gemm(w), w.c_type)
    want = ref.ref_gemm_f64(w)
    ok, err, metric = W.check(got, want, W.E5M2, absdot=ref.abs_dot(w))
    assert ok, f"{metric} = {err}"
    got64 = W.decode(ref.ref_gemm(w, acc64=True), w.c_type)
    assert np.all(np.abs(got64 - want) <= 8e-3 * np.abs(want) + 1e-30)


def test_transposed_storage_and_accumulate():
    rng = np.random.default_rng(3)
    M, N, K = 19, 23, 31
    a = rng.standard_normal((M, K)).astype(np.float32)
    b = rng.standard_normal((K, N)).astype(np.float32)
    c0 = rng.standard_normal((M, N)).astype(np.float32)
    want = (a.astype(np.float64) @ b.astype(np.float64)) + c0
    for ta in (False, True):
        for tb in (False, True):
            w = W.GemmWorkload("t", M, N, K, W.F32, W.F32, transA=ta, transB=tb, clear_accum=False,
                               A=np.ascontiguousarray(a.T if ta else a),
                               B=np.ascontiguousarray(b.T if tb else b), C0=c0)
            got = ref.ref_gemm(w)
            assert W.rel_frobenius(got, want) < 1e-6


def test_row_range_and_bad_arguments():
    w = W.make_workload("cfg5", 20, 16, 24)
    full = ref.ref_gemm(w)
    part = ref.ref_gemm(w, rows=(5, 9))
    assert np.array_equal(part[5:9], full[5:9])
    assert not part[:5].any() and not part[9:].any()
    with pytest.raises(ValueError):
        ref.ref_gemm(w, rows=(9, 5))


def test_workload_generators_are_deterministic_and_shaped():
    for name in W.WORKLOADS:
        w1 = W.make_workload(name, 24, 32, 128)
        w2 = W.make_workload(name, 24, 32, 128)
        assert np.array_equal(w1.A, w2.A) and np.array_equal(w1.B, w2.B)
        assert w1.A.shape == ((128, 24) if w1.transA else (24, 128))
        assert w1.B.shape == ((32, 128) if w1.transB else (128, 32))
    w = W.make_workload("cfg4", 24, 32, 128)
    assert w.scale_a.shape == (24,) and w.scale_b.shape == (32,)
    assert (w.scale_a >= 0.5 / 448).all() and (w.scale_a <= 2.0 / 448).all()
    assert np.abs(W.e4m3_decode(w.A)).max() <= 448
