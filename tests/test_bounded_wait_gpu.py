"""The failure path of the tensor-core scan: every device-side wait is bounded, and a wait that runs out makes
the kernels unwind (status word set, tensor memory freed, context usable) instead of hanging.  The tests make
waits run out on purpose in the only allowed way: a barrier that nothing signals and a short limit."""
import numpy as np
import pytest
import torch

from test_scan_gpu import oracle_scan, run_fused
from util import BF16_TOL, rel_err, to_np

pytestmark = pytest.mark.gpu


def test_wait_primitive_gives_up_after_its_limit(ops):
    assert ops.selftest_bounded_wait(1_000_000) == 1      # 1 ms: gave up, reported it, returned
    assert ops.selftest_bounded_wait(200_000) == 1
    torch.cuda.synchronize()


@pytest.mark.parametrize("D", [128, 64])
def test_scan_waits_run_out_and_the_next_call_is_correct(ops, orc, D):
    B, H, L, N = 1, 4, 2 * D + 5, 2
    inp = orc.make_inputs(B, H, L, D, N=N, seed=41, bf16=True)
    old = ops.set_wait_limit_ns(2_000_000)                # 2 ms instead of 400 ms
    try:
        run_fused(ops, inp, torch.bfloat16, N, D, flags=ops.TENSOR_CORE_WA | ops.TEST_WITHHOLD)
        code = ops.scan_fused_status()
        assert 200 <= code < 400, code                    # a compute warp (2xx) or the producer (3xx) gave up
        with pytest.raises(ops.CdssmError):
            run_fused(ops, inp, torch.bfloat16, N, D, flags=ops.TENSOR_CORE_WA | ops.TEST_WITHHOLD, strict=True)
    finally:
        ops.set_wait_limit_ns(old)
    # the context is intact and tensor memory was released: the same scan now runs and is right
    y, fin = run_fused(ops, inp, torch.bfloat16, N, D, flags=ops.TENSOR_CORE_WA, strict=True)
    assert ops.scan_fused_status() == 0
    wy, _ = oracle_scan(orc, inp, N, D, orc.ROUND_REFERENCE)
    assert rel_err(to_np(y), wy) <= BF16_TOL
