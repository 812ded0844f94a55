"""A bounded wait that runs out leaves cleanly: the kernel records who gave up, every role of
the CTA drains and exits, tensor memory is freed, the host reads CKL_ERR_DEVICE, and the next
launch on the same device is correct.  Nothing faults, traps or waits beyond the short limit
set here: the two cases are a pipeline stage whose barrier never completes (the producer
announces 16 bytes it never loads) and a stream-K flag value that no CTA publishes.  The
reference has no counterpart (its launchers do not even check the launch,
src/gemm/gemm_mma_opt.cu:223-225)."""

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu

LIMIT_NS = 2_000_000          # 2 ms instead of the 2 s default
ROLE_PRODUCER, ROLE_MMA, ROLE_EPILOGUE, ROLE_DRAIN = 1, 2, 3, 4


def _healthy_gemm(ckl, orc, m, n, k, algo):
    abits = orc.narrow(orc.random_matrix(m, k, 5), ckl.BF16)
    bbits = orc.narrow(orc.random_matrix(k, n, 6), ckl.BF16)
    a = torch.from_numpy(abits.view(np.int16)).view(torch.bfloat16).cuda()
    b = torch.from_numpy(bbits.view(np.int16)).view(torch.bfloat16).cuda()
    c = torch.zeros(m, n, device="cuda")
    ckl.gemm_ex(ckl.BF16, a, b, c, ckl.F32, m, n, k, k, n, n, 1.0, 0.0, algo)
    torch.cuda.synchronize()
    assert ckl.device_status() == [0, 0, 0, 0]
    ref, _ = orc.gemm_reference_mt(orc.widen(abits, ckl.BF16), orc.widen(bbits, ckl.BF16), None, 1.0, 0.0)
    assert orc.relative_frobenius_error(c.cpu().numpy(), ref) <= 1e-3
    return a, b


def test_a_stage_that_never_completes_is_given_up(ckl, orc):
    if not torch.cuda.is_available():
        pytest.fail("tests marked gpu need a CUDA device")
    m, n, k = 128, 256, 256                      # one tile, four k blocks = the four ring stages
    a, b = _healthy_gemm(ckl, orc, m, n, k, ckl.ALGO_UMMA_1CTA)
    c = torch.zeros(m, n, device="cuda")
    ckl.arm_wait_fault(1, LIMIT_NS)
    ckl.gemm_ex(ckl.BF16, a, b, c, ckl.F32, m, n, k, k, n, n, 1.0, 0.0, ckl.ALGO_UMMA_1CTA)
    with pytest.raises(ckl.CklError) as e:
        ckl.device_status()
    assert e.value.status == ckl.ERR_DEVICE and "gave up a bounded wait" in str(e.value)
    info = (ckl_status_words(str(e.value)))
    assert info["code"] == 1 and info["block"] == 0
    # Every role waits, directly or not, for the 16 bytes that never arrive (the MMA thread for
    # the stage, the epilogue warps for the accumulator behind it, the producer for the ring
    # slot), all with the same limit: whoever started its wait first reports.
    assert info["role"] in (ROLE_MMA, ROLE_DRAIN, ROLE_PRODUCER, ROLE_EPILOGUE)
    assert ckl.device_status() == [0, 0, 0, 0]   # reading clears the word
    _healthy_gemm(ckl, orc, m, n, k, ckl.ALGO_UMMA_1CTA)             # the device is fine


def test_a_stream_k_flag_nobody_sets_is_given_up(ckl, orc):
    if not torch.cuda.is_available():
        pytest.fail("tests marked gpu need a CUDA device")
    m, n, k = 2048, 2816, 2048                   # one whole wave and a split remainder: fused form
    plan = ckl.plan_gemm(m, n, k, algo=ckl.ALGO_UMMA_SK)
    assert plan.sk_tiles > 0 and plan.dp_tiles >= plan.units
    a, b = _healthy_gemm(ckl, orc, m, n, k, ckl.ALGO_UMMA_SK)
    c = torch.zeros(m, n, device="cuda")
    ckl.arm_wait_fault(2, LIMIT_NS)
    ckl.gemm_ex(ckl.BF16, a, b, c, ckl.F32, m, n, k, k, n, n, 1.0, 0.0, ckl.ALGO_UMMA_SK)
    with pytest.raises(ckl.CklError) as e:
        ckl.device_status()
    assert e.value.status == ckl.ERR_DEVICE
    info = ckl_status_words(str(e.value))
    assert info["code"] == 1 and info["role"] == ROLE_EPILOGUE
    assert info["detail"] >> 28 == 0x5           # a flag wait, low bits = the unit waited for
    _healthy_gemm(ckl, orc, m, n, k, ckl.ALGO_UMMA_SK)
    # the hook is one-shot: nothing is armed any more
    _healthy_gemm(ckl, orc, 128, 256, 256, ckl.ALGO_UMMA_1CTA)


def ckl_status_words(message: str) -> dict:
    """code=.. block=.. role=.. detail=0x.. out of the library's error text."""
    import re
    mt = re.search(r"code=(\d+) block=(\d+) role=(\d+) detail=0x([0-9a-fA-F]+)", message)
    assert mt, message
    return {"code": int(mt.group(1)), "block": int(mt.group(2)), "role": int(mt.group(3)),
            "detail": int(mt.group(4), 16)}
