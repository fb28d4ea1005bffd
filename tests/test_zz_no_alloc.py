"""The allocation-free MSE entry point (fg_mse_loss_grad_noalloc), called through the C ABI.

Some hosts cannot let the library allocate device memory: their own pool already owns the
GPU, or an allocation's device-wide synchronisation breaks a latency bound, or the job is
sized to a fixed memory budget.  For them the reduction scratch is a fixed array inside the
library.  This test checks the variant against the regular entry point on two calls in a
row (the second call reuses the same array with different, larger data), and that an input
beyond the stated maximum is refused.  It lives in a file that pytest collects last, so a
run that stops at the first failure has already run every other test.
"""
import numpy as np
import pytest

from conftest import rel_err_ok

pytestmark = pytest.mark.gpu


def test_noalloc_matches_regular_entry_point_twice():
    from ferrograd_b200 import FgError, GpuContext
    ctx = GpuContext(0)
    try:
        r = np.random.Generator(np.random.Philox(2024))
        # calls in a row on the shared array; sizes around the 65,536-element chunk edge, then ones that need
        # several partial sums
        for n in (65_536, 65_537, 70_001, 1_300_000):
            p, t = r.standard_normal(n, np.float32), r.standard_normal(n, np.float32)
            dp_, dt_ = ctx.init_tensor_f32((n,), p), ctx.init_tensor_f32((n,), t)
            ref = [ctx.new_tensor((n,)), ctx.new_tensor((1,)), ctx.new_tensor((n,))]
            got = [ctx.new_tensor((n,)), ctx.new_tensor((1,)), ctx.new_tensor((n,))]
            ctx.mse_loss_grad(dp_, dt_, n, grad_scale=0.25, loss_elem=ref[0], loss_sum=ref[1], grad=ref[2])
            ws = ctx.workspace_bytes()
            ctx.mse_loss_grad_noalloc(dp_, dt_, n, grad_scale=0.25, loss_elem=got[0], loss_sum=got[1], grad=got[2])
            ctx.sync()
            assert ctx.workspace_bytes() == ws                      # the scratch arena was not touched
            assert np.array_equal(ctx.to_numpy(got[0]), ctx.to_numpy(ref[0]))
            assert np.array_equal(ctx.to_numpy(got[2]), ctx.to_numpy(ref[2]))
            ok, worst = rel_err_ok(ctx.to_numpy(got[1]), ctx.to_numpy(ref[1]), 1e-5)
            assert ok, f"loss sum differs: {worst:.3g} x 1e-5"
            # and both agree with a float64 sum on the host
            exact = float(np.sum((p.astype(np.float64) - t) ** 2))
            assert abs(float(ctx.to_numpy(got[1])[0]) - exact) <= 1e-5 * exact
        # nothing to sum: the result is zero and nothing is launched
        z = ctx.init_tensor_f32((1,), np.array([7.0], np.float32))
        ctx.mse_loss_grad_noalloc(dp_, dt_, 0, loss_sum=z)
        ctx.sync()
        assert float(ctx.to_numpy(z)[0]) == 0.0
        # sum only (no per-element outputs), then a size beyond the maximum
        s = ctx.new_tensor((1,))
        ctx.mse_loss_grad_noalloc(dp_, dt_, n, loss_sum=s)
        ctx.sync()
        assert abs(float(ctx.to_numpy(s)[0]) - exact) <= 1e-5 * exact
        with pytest.raises(FgError) as e:
            ctx.mse_loss_grad_noalloc(dp_, dt_, 268_435_456 + 1, loss_sum=s)
        assert e.value.kind == "FG_ERR_INVALID_ARGUMENT" and "268,435,456" in str(e.value)
    finally:
        ctx.sync()
        ctx.destroy()
