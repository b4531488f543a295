"""Stand-alone operators of the expert path (Q8_K quantise, weighted clamp + SwiGLU, vector add, gather)
against the CPU oracle, bit for bit, through the C ABI."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _q8k_inputs():
    rng = np.random.default_rng(41)
    x = rng.standard_normal((37, 256)).astype(np.float32)
    x[3] = 0.0                                   # an all-zero block: an all-zero record
    x[5] *= 1.0e4
    x[6] *= 1.0e-6
    x[7, :] = 0.25; x[7, 1] = 2.0; x[7, 128] = -2.0      # equal |x| of both signs: the tree prefers index 128
    x[8, :] = 0.0; x[8, 255] = -3.0                      # the last element alone
    x[9] = np.round(x[9] * 4) / 4                        # many exact ties of rint(iscale * x) at .5
    return x


def test_q8_k_quantize_bitexact(torch_cuda, moe, oracle):
    torch = torch_cuda
    x = _q8k_inputs()
    want = oracle.q8_k_quantize(x)
    got = moe.Q8KQuantize.launch(torch.from_numpy(x).cuda()).cpu().numpy()
    assert np.array_equal(got, want)
    blocks = got.reshape(-1, 292)
    assert blocks[7, :4].view(np.float32)[0] > 0 and blocks[7, 4 + 128:4 + 129].view(np.int8)[0] == -127
    # offset form of the reference (launch_with_offsets): blocks 10.. written at record 2 of a larger buffer
    buf = torch.full((40 * 292,), 0xEE, dtype=torch.uint8, device="cuda")
    moe.Q8KQuantize.launch(torch.from_numpy(x[10:]).cuda(), out=buf[2 * 292:])
    b = buf.cpu().numpy()
    assert np.array_equal(b[2 * 292:(2 + 27) * 292], want[10 * 292:]) and (b[:2 * 292] == 0xEE).all() and (b[29 * 292:] == 0xEE).all()
    # many blocks: every warp of a full grid takes several
    big = np.random.default_rng(42).standard_normal((20000, 256)).astype(np.float32)
    assert np.array_equal(moe.Q8KQuantize.launch(torch.from_numpy(big).cuda()).cpu().numpy(), oracle.q8_k_quantize(big))


@pytest.mark.parametrize("n,ff,clamp", [(6, 2048, 10.0), (1, 4, 0.0), (257, 2304, 7.0)])
def test_swiglu_clamp_weighted_bitexact(torch_cuda, moe, oracle, n, ff, clamp):
    torch = torch_cuda
    rng = np.random.default_rng(n)
    gate = (rng.standard_normal((n, ff)) * 6).astype(np.float32)
    up = (rng.standard_normal((n, ff)) * 6).astype(np.float32)
    gate.flat[:4] = [100.0, -100.0, 0.0, -0.0]
    w = rng.random(n).astype(np.float32)
    got = moe.SwigluClampWeighted.launch(torch.from_numpy(gate).cuda(), torch.from_numpy(up).cuda(), torch.from_numpy(w).cuda(), clamp).cpu().numpy()
    want = oracle.swiglu_clamp_weighted(gate, up, w, clamp)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    libm = oracle.swiglu_clamp_weighted(gate, up, w, clamp, use_det=False)     # expf as the reference source reads
    assert np.allclose(got, libm, rtol=1e-6, atol=1e-30)


@pytest.mark.parametrize("n,offset", [(1, 0), (4099, 0), (1 << 20, 0), (1001, 1)])
def test_vec_add_inplace_and_gather(torch_cuda, moe, n, offset):
    torch = torch_cuda
    rng = np.random.default_rng(n)
    a = rng.standard_normal(n + offset).astype(np.float32)
    b = rng.standard_normal(n + offset).astype(np.float32)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    moe.VecAddInplace.launch(da[offset:], db[offset:])            # offset 1: rows off the 16-byte boundary
    got = da.cpu().numpy()
    assert np.array_equal(got[offset:], a[offset:] + b[offset:]) and np.array_equal(got[:offset], a[:offset])
    idx = rng.integers(-3, n, size=777).astype(np.int32)
    g = moe.VecAddInplace.launch_gather(db[offset:], torch.from_numpy(idx).cuda()).cpu().numpy()
    want = np.where(idx >= 0, b[offset:][np.maximum(idx, 0)], -np.inf).astype(np.float32)
    assert np.array_equal(g, want)
