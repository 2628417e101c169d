"""The launch that allocates nothing (wg_launch_noalloc), for callers that cannot call
cudaMalloc at the point of use -- code living inside another framework's memory pool or under
a fixed memory budget, or a latency-critical loop that must not hit cudaMalloc's implicit
synchronisation.  Its hand-off flags live in a device array built into the library, shared by
every call, so the test makes two calls in a row (the second sees the first's leftovers) and
switches shapes in between; each result must equal what the planned entry point gives.
Collected last on purpose: a failure here stops nothing else."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")
import warpc_public_release_b200 as w  # noqa: E402
from warpc_public_release_b200 import plan as wplan  # noqa: E402
from warpc_public_release_b200 import _lib  # noqa: E402
from oracle import gemm_ref  # noqa: E402


def planned(variant, m, n, k, da, db):
    dc = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    p = w.Plan(variant, m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr())
    p.launch()
    p.status()
    p.close()
    return dc


def test_noalloc_matches_planned_entry_on_two_calls_in_a_row():
    cases = [((512, 1024, 1024), lambda s: w.swapped(*s, 256, 256, 4, split_grid=4, split_add=True)),     # split-K: 32 flags
             ((1024, 512, 1024), lambda s: w.swapped(*s, 256, 128, 6, streamk=True, split_add=True, bufs=2)),  # stream-K: 148 + 16 flags
             ((512, 1024, 1024), lambda s: w.swapped(*s, 256, 256, 4, split_grid=3, split_add=True))]     # fewer flags than the call before
    for shape, build in cases:
        m, n, k = shape
        a, bt = gemm_ref.inputs_integers(m, n, k)
        da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
        v = build(shape)
        want = planned(v, m, n, k, da, db)
        for call in range(2):
            dc = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
            torch.cuda.synchronize()
            free_before = torch.cuda.mem_get_info()[0]     # the driver's count of free device memory
            wplan.launch_noalloc(v, m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr())
            assert wplan.noalloc_status()[0] == 0
            assert torch.cuda.mem_get_info()[0] == free_before, "the call changed the device's free memory"
            # integer inputs: exact, whatever order the L2 adds land in (the tolerance the other tests use: 1e-3)
            assert torch.equal(dc, want), "call %d at %s" % (call, shape)
            assert gemm_ref.count_wrong(dc.cpu().numpy(), gemm_ref.gemm_ref(a, bt), 1e-3) == 0


def test_noalloc_uses_the_rule_when_no_variant_is_given_and_rejects_oversize():
    m, n, k = 512, 768, 512
    a, bt = gemm_ref.inputs_hash(m, n, k)
    da, db = torch.from_numpy(a).cuda(), torch.from_numpy(bt).cuda()
    dc = torch.zeros((m, n), dtype=torch.float32, device="cuda")
    wplan.launch_noalloc(None, m, n, k, da.data_ptr(), db.data_ptr(), dc.data_ptr())
    wplan.noalloc_status()
    assert np.array_equal(dc.cpu().numpy(), gemm_ref.gemm_ref(a, bt))
    # stream-K keeps a word per CTA tile: 148 + (8192/256)*(8192/128) = 2196 fits, 148 + 64*128 does not
    assert wplan.noalloc_max_flags() == 4096
    big = w.swapped(16384, 16384, 64, 256, 128, 6, streamk=True, split_add=True, bufs=2)
    with pytest.raises(_lib.WarpcError) as e:
        wplan.launch_noalloc(big, 16384, 16384, 64, da.data_ptr(), db.data_ptr(), dc.data_ptr())
    assert e.value.code == _lib.WG_E_LIMIT
