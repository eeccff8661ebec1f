"""GPU parity of frisk.reduce on whole buffers: the CUDA kernels, called through the C ABI,
against the float64 restatement in oracle/ref.py on the same seeded inputs.

Tolerances: min and max are exact -- the stored bits must equal the oracle's.  add and mul
accumulate in fp32 and round once: |got - want| <= 1e-5 * (sum of the magnitudes folded; for a
product of n factors max(1e-5, n * 2^-24) * |product|) + one unit in the last place of the
stored type at the result (the fp32 accumulation order differs
from the oracle's float64, so the last rounding may fall either way).  Full-size inputs are
checked on sampled lines plus a size-independent property: folding the two halves of the reduced
dimension and then the two results gives the same bits for min / max."""
import numpy as np
import pytest

from frisk_b200 import runtime as R
from frisk_b200 import workloads as W
from oracle import ref

pytestmark = pytest.mark.gpu

ULP = {W.F32: 2.0 ** -23, W.F16: 2.0 ** -10, W.BF16: 2.0 ** -7}


def make_src(shape, dtype, kind, seed):
    rng = np.random.default_rng(seed)
    n = int(np.prod(shape))
    if kind == "mul":  # factors near 1 so that long products stay in range
        ext = max(shape) if shape else 1
        x = 1.0 + rng.uniform(-1.0, 1.0, size=n) / max(ext, 1) ** 0.5
        x *= rng.choice([-1.0, 1.0], size=n, p=[0.1, 0.9])
    else:
        x = rng.standard_normal(n)
    return W.encode(x.astype(np.float32).reshape(shape), dtype)


def check(got_bits, want64, mag, dtype, kind, count=1):
    got = W.decode(got_bits, dtype).astype(np.float64).reshape(want64.shape)
    if kind in ("min", "max"):
        want_bits = W.encode(want64.astype(np.float32), dtype).reshape(got_bits.shape)
        assert np.array_equal(got_bits, want_bits)
        return
    if kind == "mul":  # a chain of n roundings: n * 2^-24 relative, at worst
        mag = mag * max(1.0, count * 2.0 ** -24 / 1e-5)
    tol = 1e-5 * mag + ULP[dtype] * np.maximum(np.abs(want64), 1e-30) * 1.01 + 1e-38
    bad = np.abs(got - want64) > tol
    assert not bad.any(), f"{int(bad.sum())} of {bad.size} off; worst {np.abs(got - want64).max():.3e}"


CASES = [
    # shape, dim
    ((64, 8192), 1),          # lines, a warp per line
    ((3, 1000), 1),           # line length not a multiple of the vector
    ((5, 1003), 1),           # odd length: every line starts at a different alignment
    ((7, 1), 1),              # a single element per line
    ((1, 300000), 1),         # one long line: cut into pieces, two launches
    ((2, 70001), 1),          # pieces with a ragged last one
    ((4096, 64), 0),          # columns, 8 vectors per row
    ((1000, 8), 0),           # one vector per row
    ((777, 5), 0),            # scalar columns
    ((50000, 16), 0),         # few columns, long extent: pieces through the workspace
    ((33, 4096), 0),          # wide rows: several CTAs along the contiguous dimension
    ((300, 2500), 0),         # inner not a power of two
    ((4, 8, 16), 1),          # the reference's own test shape (test_pass/attr_test.cpp:299-300)
    ((4, 8, 16), 0),
    ((4, 8, 16), 2),
    ((6, 5000, 3), 1),
    ((128,), 0),              # rank 1 to a single value
]


@pytest.mark.parametrize("dtype", [W.F32, W.F16, W.BF16], ids=["f32", "f16", "bf16"])
@pytest.mark.parametrize("kind", ["add", "mul", "min", "max"])
@pytest.mark.parametrize("shape,dim", CASES, ids=[f"{'x'.join(map(str, s))}-d{d}" for s, d in CASES])
def test_reduce_matches_the_oracle(shape, dim, kind, dtype):
    src = make_src(shape, dtype, kind, seed=len(shape) * 1000 + dim)
    dst_shape = tuple(d for k, d in enumerate(shape) if k != dim) or (1,)
    dst = np.zeros(dst_shape, dtype=src.dtype)
    R.reduce_host(src, dst, dim, dtype, kind, clear=True)
    want, mag = ref.ref_reduce(src, dim, dtype, kind)
    check(dst, want.reshape(dst_shape), mag.reshape(dst_shape), dtype, kind, count=shape[dim])


@pytest.mark.parametrize("kind", ["add", "mul", "min", "max"])
@pytest.mark.parametrize("shape,dim", [((16, 4096), 1), ((1, 200000), 1), ((4096, 24), 0), ((60000, 8), 0)])
def test_reduce_without_clear_folds_the_old_destination_in(shape, dim, kind):
    dtype = W.BF16
    src = make_src(shape, dtype, kind, seed=7)
    dst_shape = tuple(d for k, d in enumerate(shape) if k != dim)
    dst0 = W.encode((np.random.default_rng(8).standard_normal(dst_shape) * 3).astype(np.float32), dtype)
    dst = dst0.copy()
    R.reduce_host(src, dst, dim, dtype, kind, clear=False)
    want, mag = ref.ref_reduce(src, dim, dtype, kind, clear=False, dst0=dst0)
    check(dst, want, mag, dtype, kind, count=shape[dim])


def test_reduce_edge_shapes():
    # nothing to write
    R.reduce_host(np.zeros((0, 8), np.float32), np.zeros((0,), np.float32), 1, W.F32, "add")
    R.reduce_host(np.zeros((4, 8, 0), np.float32), np.zeros((4, 0), np.float32), 1, W.F32, "add")
    # an empty reduced dimension gives the identity of the kind, or leaves dst alone
    for kind, ident in (("add", 0.0), ("mul", 1.0), ("min", np.inf), ("max", -np.inf)):
        dst = np.full((4,), 7.0, np.float32)
        R.reduce_host(np.zeros((4, 0), np.float32), dst, 1, W.F32, kind)
        assert np.array_equal(dst, np.full((4,), ident, np.float32))
        dst = np.full((2, 3), 7.0, np.float32)
        R.reduce_host(np.zeros((2, 0, 3), np.float32), dst, 1, W.F32, kind, clear=False)
        assert np.array_equal(dst, np.full((2, 3), 7.0, np.float32))
    # min / max skip NaN (a line of nothing else gives the identity); infinities pass through
    vals = np.array([[np.nan, 1.0, -2.0, np.inf], [np.nan] * 4, [-np.inf, 0.0, np.nan, 5.0]], np.float32)
    for dtype in (W.F32, W.F16, W.BF16):
        src = W.encode(vals, dtype)
        for kind, want in (("max", [np.inf, -np.inf, 5.0]), ("min", [-2.0, np.inf, -np.inf])):
            dst = np.zeros((3,), src.dtype)
            R.reduce_host(src, dst, 1, dtype, kind)
            assert np.array_equal(W.decode(dst, dtype), np.array(want, np.float32))
            assert np.array_equal(ref.ref_reduce(src, 1, dtype, kind)[0], np.array(want, np.float64))
    with pytest.raises(ValueError):
        R.reduce_desc((4, 4), 2, W.F32, "add")
    with pytest.raises(ValueError):
        R.reduce_desc((4, 4), 1, W.F32, "xor")
    with pytest.raises(R.FriskError) as e:
        R.reduce_host(np.zeros((4, 4), np.uint8), np.zeros((4,), np.uint8), 1, W.E4M3, "add")
    assert e.value.code == -2


def test_reduce_on_device_buffers_at_any_alignment_and_with_a_workspace():
    import torch
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(3)
    for shape, dim, kind in (((37, 4099), 1, "max"), ((37, 4099), 1, "add"), ((2, 100000), 1, "add"),
                             ((2049, 40), 0, "min"), ((30000, 24), 0, "add")):
        host = W.encode(rng.standard_normal(shape).astype(np.float32), W.F16)
        desc = R.reduce_desc(shape, dim, W.F16, kind)
        ws_bytes = R.reduce_workspace_bytes(desc)
        ws = torch.empty(max(ws_bytes, 16), dtype=torch.uint8, device=dev)
        want, mag = ref.ref_reduce(host, dim, W.F16, kind)
        for shift in (0, 1, 3, 8):  # elements past a 256-byte aligned allocation
            pad = torch.zeros(host.size + 16, dtype=torch.int16, device=dev)
            flat = pad[shift:shift + host.size]
            flat.copy_(torch.from_numpy(host.view(np.int16).reshape(-1)))
            out = torch.full((want.size + 2,), 0x7c01, dtype=torch.int16, device=dev)  # guards around dst
            R.reduce_run(desc, flat.data_ptr(), out[1:].data_ptr(), ws if ws_bytes else None)
            torch.cuda.synchronize()
            got = out.cpu().numpy()
            assert got[0] == 0x7c01 and got[-1] == 0x7c01
            check(got[1:-1].view(np.float16).reshape(want.shape), want, mag, W.F16, kind)
        if ws_bytes:
            with pytest.raises(R.FriskError) as e:
                R.reduce_run(desc, flat.data_ptr(), out[1:].data_ptr(), None)
            assert e.value.code == -4


def test_online_softmax_row_statistics_at_full_size():
    """The two reduces of the reference's online-softmax sketch (tmp/ir.mlir:21-78) at its size:
    the row maximum of an 8192 x 8192 fp16 matrix and row sums in fp32.  Seeded normal values
    stand in for the activations."""
    import torch
    dev = torch.device("cuda:0")
    g = torch.Generator(device=dev).manual_seed(11)
    x = torch.randn((8192, 8192), generator=g, device=dev, dtype=torch.float32).to(torch.float16)
    rows = np.random.default_rng(12).choice(8192, 48, replace=False)
    host_rows = x[torch.from_numpy(rows).to(dev)].cpu().numpy()

    desc = R.reduce_desc((8192, 8192), 1, W.F16, "max")
    assert R.reduce_info(desc) == dict(lines=1, vector=8, chunks=1, launches=1, chunk_len=8192, ctas=1024,
                                       workspace_bytes=0)
    out = torch.empty(8192, dtype=torch.float16, device=dev)
    R.reduce_run(desc, x, out)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    want, mag = ref.ref_reduce(host_rows, 1, W.F16, "max")
    check(got[rows], want, mag, W.F16, "max")
    # max over a line = max of the maxima of its halves, bit for bit
    halves = torch.empty((8192, 2), dtype=torch.float16, device=dev)
    R.reduce_run(R.reduce_desc((8192 * 2, 4096), 1, W.F16, "max"), x, halves)
    again = torch.empty(8192, dtype=torch.float16, device=dev)
    R.reduce_run(R.reduce_desc((8192, 2), 1, W.F16, "max"), halves, again)
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int16), again.view(torch.int16))
    # the column direction of the same matrix, and the same property there
    cols = torch.empty(8192, dtype=torch.float16, device=dev)
    cdesc = R.reduce_desc((8192, 8192), 0, W.F16, "min")
    ws = torch.empty(max(R.reduce_workspace_bytes(cdesc), 16), dtype=torch.uint8, device=dev)
    R.reduce_run(cdesc, x, cols, ws)
    torch.cuda.synchronize()
    pick = np.random.default_rng(13).choice(8192, 32, replace=False)
    host_cols = np.ascontiguousarray(x[:, torch.from_numpy(pick).to(dev)].cpu().numpy())
    want, mag = ref.ref_reduce(host_cols, 0, W.F16, "min")
    check(cols.cpu().numpy()[pick], want, mag, W.F16, "min")

    # row sums in fp32 of the same values
    xf = x.to(torch.float32)
    sums = torch.empty(8192, dtype=torch.float32, device=dev)
    R.reduce_run(R.reduce_desc((8192, 8192), 1, W.F32, "add"), xf, sums)
    torch.cuda.synchronize()
    want, mag = ref.ref_reduce(xf[torch.from_numpy(rows).to(dev)].cpu().numpy(), 1, W.F32, "add")
    check(sums.cpu().numpy()[rows], want, mag, W.F32, "add")
    # run-to-run bit equality: the order of the fold is fixed by the shape
    sums2 = torch.empty_like(sums)
    R.reduce_run(R.reduce_desc((8192, 8192), 1, W.F32, "add"), xf, sums2)
    torch.cuda.synchronize()
    assert torch.equal(sums.view(torch.int32), sums2.view(torch.int32))
