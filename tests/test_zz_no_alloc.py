"""The allocation-free group builder against the regular one.

Collected last on purpose: a run that stops at the first failure has then
already exercised every other test.  The entry point under test keeps its
temporary in a fixed array inside the library (for engines that own all device
memory themselves, or that cannot tolerate an allocation on their serving path),
so the check is that two calls in a row -- the second smaller than the first, so
that it finds the first call's leftovers in the shared array -- give exactly
the outputs of the allocating entry point.  All outputs are integers: the
comparison is bit for bit, like the other group-builder tests.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _picks(rng, T, k, E):
    sel = np.stack([rng.choice(E, k, replace=False) for _ in range(T)]).astype(np.int32)
    sel[1, 0] = -1          # dropped, as NO_PICK is
    sel[2, k - 1] = E + 7   # past the bound: dropped
    return sel


def test_static_scratch_matches_allocating_entry_point_twice_in_a_row(oracle):
    import torch
    from deepstrix_b200 import moe
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    rng = np.random.default_rng(2024)
    E, k, chunk = 256, 8, 32
    for T in (6000, 700):   # 24 chunks of scratch, then 3: the second call sees stale entries
        sel = torch.from_numpy(_picks(rng, T, k, E)).cuda()
        got = moe.MoeGroupBuilder.launch_static(sel, E, chunk)
        want = moe.MoeGroupBuilder.launch(sel, E, chunk)
        torch.cuda.synchronize()
        n = int(want[1][-1].item())
        assert int(got[4].item()) == int(want[4].item())
        ni = int(want[4].item())
        for name, g, w, m in (("hist", got[0], want[0], E), ("offsets", got[1], want[1], E + 1),
                              ("perm", got[2], want[2], n), ("work_items", got[3], want[3], ni)):
            assert torch.equal(g[:m], w[:m]), name
        # and against the CPU oracle's group inversion and work items
        oh, oo, op = oracle.group_build(sel.cpu().numpy(), E)
        assert np.array_equal(got[0].cpu().numpy(), oh) and np.array_equal(got[1].cpu().numpy(), oo)
        assert np.array_equal(got[2].cpu().numpy()[: op.size], op)
        oi, on = oracle.work_items(oh, chunk)
        assert on == ni and np.array_equal(got[3].cpu().numpy()[:on], oi)


def test_static_scratch_refuses_oversized_input():
    import torch
    from deepstrix_b200 import moe
    torch.cuda.set_device(0)
    sel = torch.zeros((16385, 8), dtype=torch.int32, device="cuda")   # 131080 picks > 131072
    with pytest.raises(moe.DsxError) as e:
        moe.MoeGroupBuilder.launch_static(sel, 256, 32)
    assert e.value.code == -2 and "131072" in str(e.value)
    sel = torch.zeros((4, 8), dtype=torch.int32, device="cuda")
    with pytest.raises(moe.DsxError) as e:
        moe.MoeGroupBuilder.launch_static(sel, 544, 32)               # more experts than the scratch has columns for
    assert e.value.code == -2
