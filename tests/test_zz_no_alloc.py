"""msx_sum_rows_static, the entry point for hosts that cannot allocate device memory after they
start (their memory is already committed to a pool of their own, or their loop may not call the
driver's allocator): its scratch is a device array inside the library. Called through the C ABI on
the caller's own device buffers and compared with the plan's SumRows on the same inputs, twice in
a row with different shapes so that what the first call left in the shared scratch cannot leak
into the second. Collected last, so a failure here stops nothing else."""
import ctypes as C

import numpy as np
import pytest

import modelspec_b200 as M
from helpers import ProgramText, assert_kernel_close

pytestmark = pytest.mark.gpu


def plan_sum_rows(device, g):
    rows, h = g.shape
    p = ProgramText()
    x = p.input("g", "f32", [rows, h])
    out = p.op("SumRows", [h], [x])
    p.output(out)
    plan = M.Plan(device, p.text(), flags=M.PLAN_NO_GRAPH)
    try:
        plan.set_input("g", g)
        plan.run()
        return plan.value(out, h)
    finally:
        plan.destroy()


def test_static_sum_rows_matches_the_plan_twice_in_a_row(device):
    import torch

    L = M.lib()
    r = np.random.default_rng(21)
    for rows, h in [(4096, 128), (833, 30)]:
        g = r.standard_normal((rows, h)).astype(np.float32)
        expected = plan_sum_rows(device, g)
        # The caller's buffers: this test may allocate, the entry point does not.
        d_g = torch.from_numpy(g).to("cuda:0")
        d_out = torch.full((h,), float("nan"), dtype=torch.float32, device="cuda:0")
        torch.cuda.synchronize()
        rc = L.msx_sum_rows_static(C.c_void_p(d_g.data_ptr()), rows, h, C.c_void_p(d_out.data_ptr()), None)
        assert rc == M.OK, L.msx_static_last_error().decode()
        torch.cuda.synchronize()
        got = d_out.cpu().numpy()
        assert_kernel_close(got, expected, scale=np.abs(g).sum(axis=0), what="static sum_rows %dx%d" % (rows, h))
        assert np.array_equal(got, expected), "the same kernels give the same bits"


@pytest.mark.parametrize("rows,h", [(833, 1024), (100, 2048), (4096, 4096), (7, 12)])
def test_static_sum_rows_wide_rows_and_a_stream_of_the_callers(device, rows, h):
    """Rows of 1,024 or more columns take the wide first stage; 4,096 columns is the most the
    scratch holds; 7 rows are one chunk. The call is made on a stream of the caller's, not the
    default one, and still has the plan's bits."""
    import torch

    L = M.lib()
    g = np.random.default_rng(rows + h).standard_normal((rows, h)).astype(np.float32)
    expected = plan_sum_rows(device, g)
    d_g = torch.from_numpy(g).to("cuda:0")
    d_out = torch.full((h,), float("nan"), dtype=torch.float32, device="cuda:0")
    torch.cuda.synchronize()
    stream = torch.cuda.Stream(device="cuda:0")
    rc = L.msx_sum_rows_static(C.c_void_p(d_g.data_ptr()), rows, h, C.c_void_p(d_out.data_ptr()), C.c_void_p(stream.cuda_stream))
    assert rc == M.OK, L.msx_static_last_error().decode()
    stream.synchronize()
    got = d_out.cpu().numpy()
    assert np.array_equal(got, expected), "the chunk sums are added in the same order"


def test_static_sum_rows_refuses_what_its_scratch_cannot_hold(device):
    import torch

    L = M.lib()
    buf = torch.zeros(8, dtype=torch.float32, device="cuda:0")
    ptr = C.c_void_p(buf.data_ptr())
    assert L.msx_sum_rows_static(ptr, 1, 4097, ptr, None) == M.BAD_ARGUMENT
    assert "4096" in L.msx_static_last_error().decode()
    assert L.msx_sum_rows_static(ptr, 1, 0, ptr, None) == M.BAD_ARGUMENT
    assert L.msx_sum_rows_static(None, 1, 8, ptr, None) == M.BAD_ARGUMENT
