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


@pytest.mark.parametrize("T,k,H", [(5, 6, 1032), (33, 8, 2048), (3, 16, 264)])
def test_reduce_partials_owner_filter_and_row_table(torch_cuda, moe, T, k, H):
    """The slot-order reduction with the owner filter (picks outside [lo, lo + n) were never computed: skipped), for
    widths where a warp lies inside one token's row (multiples of 256) and where it does not; and the same through a
    table of row pointers with some rows wanted nowhere."""
    torch = torch_cuda
    import ctypes as C
    rng = np.random.default_rng(T * H)
    partial = rng.standard_normal((T * k + T, H)).astype(np.float32)
    sel = rng.integers(0, 32, size=(T, k)).astype(np.int32)
    sel[0, :] = 31                                          # a token with no pick in the range
    lo, n = 4, 12
    want = np.zeros((T, H), np.float32)
    for t in range(T):
        acc = np.zeros(H, np.float32)
        for s in range(k):
            if lo <= sel[t, s] < lo + n:
                acc = (acc + partial[t * k + s]).astype(np.float32)
        want[t] = (acc + partial[T * k + t]).astype(np.float32)
    want_bf16 = torch.from_numpy(want).to(torch.bfloat16)
    dp, ds = torch.from_numpy(partial).cuda(), torch.from_numpy(sel).cuda()
    got = moe.reduce_partials(dp, T, k, with_shared=True, selected=ds, expert_lo=lo, n_local=n)
    assert torch.equal(got.cpu(), want_bf16)
    # through a row table: even tokens into a scattered buffer, odd tokens nowhere
    buf = torch.full((2 * T, H), float("nan"), dtype=torch.bfloat16, device="cuda")
    table = torch.zeros((T,), dtype=torch.int64, device="cuda")
    for t in range(0, T, 2):
        table[t] = buf[2 * T - 1 - t].data_ptr()
    moe._check(moe.lib().dsx_reduce_partials_to(C.c_void_p(dp.data_ptr()), C.c_int64(T), k, C.c_int64(H), 1, C.c_void_p(ds.data_ptr()), lo, n,
                                               C.c_void_p(table.data_ptr()), moe._stream()))
    out = buf.cpu()
    for t in range(T):
        row = out[2 * T - 1 - t]
        if t % 2 == 0:
            assert torch.equal(row, want_bf16[t])
        else:
            assert torch.isnan(row.float()).all()
