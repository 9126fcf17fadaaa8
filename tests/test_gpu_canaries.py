"""No kernel stores outside the destination block or the scratchpad it was given.

Every case of tests/cases.py runs with its destination placed inside a larger buffer -- guard
rows above and below, guard columns at the end of every row (the destination's row pitch is
larger than N) -- and with a user scratchpad placed between two guard areas.  Afterwards the
guards must still hold the byte they were filled with, and the block must hold, bit for bit,
what the same primitive writes into an ordinary dense destination.  Two row pitches: one that
keeps every row 16-byte aligned (the vector stores of the fast kernels stay in use) and an odd
one (their element-wise fallbacks).  The ragged cases of the catalogue are the ones that matter:
tiles, chunks and strips that reach past M or N must not store there.
"""
import numpy as np
import pytest

import cases
from parity import assert_close
from onednn_b200 import api, dtypes as dt

pytestmark = pytest.mark.gpu

GUARD = 0xA5
GUARD_ROWS = 2
SCRATCH_GUARD = 512


@pytest.fixture(scope="module")
def ctx():
    eng = api.Engine()
    return eng, api.Stream(eng)


@pytest.mark.parametrize("name", list(cases.CASES))
@pytest.mark.parametrize("weights", ["any", "plain"])
@pytest.mark.parametrize("pad", [16, 3])
def test_stores_stay_inside_dst_and_scratchpad(ctx, name, weights, pad):
    import torch
    eng, strm = ctx
    c = cases.build(name)
    elem = np.dtype(dt.RAW[c.dst_dt]).itemsize
    # what the primitive writes into a dense destination of its own
    ref_plan = api.CasePlan(c, eng, strm, weights=weights)
    ref_plan.execute()
    want = np.ascontiguousarray(ref_plan.result()).view(np.uint8).reshape(c.M, c.N * elem)

    pitch = c.N + pad
    plan = api.CasePlan(c, eng, strm, weights=weights, dst_strides=(pitch, 1), scratchpad="user")
    assert plan.impl == ref_plan.impl, "the padded destination changed the dispatch"
    rows = c.M + 2 * GUARD_ROWS
    buf = torch.full((rows, pitch * elem), GUARD, dtype=torch.uint8, device="cuda")
    block = buf[GUARD_ROWS:GUARD_ROWS + c.M, :c.N * elem]
    if c.dst_init is not None:
        block.copy_(torch.from_numpy(np.ascontiguousarray(c.dst_init).view(np.uint8).reshape(c.M, c.N * elem)))
    args = dict(plan.args)
    args[api.ARG_DST] = api.Memory(plan.mds["dst"], eng, handle=buf.data_ptr() + GUARD_ROWS * pitch * elem)
    scratch_bytes = plan.pd.scratchpad_desc().get_size()
    sbuf = None
    if scratch_bytes:
        sbuf = torch.full((scratch_bytes + 2 * SCRATCH_GUARD,), GUARD, dtype=torch.uint8, device="cuda")
        sbuf[SCRATCH_GUARD:SCRATCH_GUARD + scratch_bytes].zero_()
        args[api.ARG_SCRATCHPAD] = api.Memory(plan.pd.scratchpad_desc(), eng, handle=sbuf.data_ptr() + SCRATCH_GUARD)
    torch.cuda.synchronize()
    plan.prim.execute(strm, args)
    strm.wait()

    got = buf.cpu().numpy()
    assert (got[:GUARD_ROWS] == GUARD).all(), "%s via %s stored above the destination" % (name, plan.impl)
    assert (got[GUARD_ROWS + c.M:] == GUARD).all(), "%s via %s stored below the destination" % (name, plan.impl)
    assert (got[:, c.N * elem:] == GUARD).all(), "%s via %s stored past the end of a row" % (name, plan.impl)
    inner = np.ascontiguousarray(got[GUARD_ROWS:GUARD_ROWS + c.M, :c.N * elem])
    if "wc_" in plan.impl:
        # the decode kernels add partial sums with atomics: the order, and with it the last bits, vary
        raw = dt.RAW[c.dst_dt]
        assert_close(c, inner.view(raw).reshape(c.M, c.N), want.view(raw).reshape(c.M, c.N), name)
    else:
        assert np.array_equal(inner, want), "%s via %s: the padded destination holds other bytes" % (name, plan.impl)
    if sbuf is not None:
        s = sbuf.cpu().numpy()
        assert (s[:SCRATCH_GUARD] == GUARD).all() and (s[SCRATCH_GUARD + scratch_bytes:] == GUARD).all(), \
            "%s via %s stored outside its scratchpad" % (name, plan.impl)
