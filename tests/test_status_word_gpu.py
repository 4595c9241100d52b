"""The device-side status word: a kernel that cannot go on says so there and ends; the host turns it into
BMXK_ERR_DEVICE.  Two routes are exercised without faulting or hanging anything:
  * a full fp16 window (the host skipped a flush) -> status 2, nothing written;
  * a bounded wait that runs out (a barrier nothing arrives on, limit ~1 ms) -> status 1 with block and site.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu
D = 128


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def test_full_window_is_reported_and_nothing_is_written():
    from bmx_b200 import kernels as K
    from bmx_b200._lib import BmxkError

    dev = _dev()
    B, h_kv, cap = 2, 2, 8
    gen = torch.Generator().manual_seed(3)
    win = [torch.zeros(B, h_kv, cap, D, dtype=torch.float16, device=dev) for _ in range(3)]
    tail_len = torch.tensor([cap - 1, cap], dtype=torch.int32, device=dev)  # sequence 1 is already full
    counters = torch.zeros(B, dtype=torch.int32, device=dev)
    status = torch.zeros(64, dtype=torch.int32, device=dev)
    src = [torch.randn(B, h_kv, 1, D, generator=gen).half().to(dev) for _ in range(3)]
    K.window_append_devpos(src[0], src[1], src[2], win[0], win[1], win[2], tail_len, counters, status)
    torch.cuda.synchronize()
    assert tail_len.tolist() == [cap, cap] and counters.tolist() == [0, 0]
    assert torch.equal(win[0][0, :, cap - 1], src[0][0, :, 0])           # sequence 0 took its token
    assert float(win[0][1].abs().max()) == 0.0 and float(win[1][1].abs().max()) == 0.0  # sequence 1: untouched
    with pytest.raises(BmxkError) as ei:
        K.check_status(status.view(torch.uint8))
    assert ei.value.code == 3 and "window" in str(ei.value)
    # the word is sticky until the owner clears it; once cleared the same buffers work again
    status.zero_()
    tail_len.fill_(0)
    K.window_append_devpos(src[0], src[1], src[2], win[0], win[1], win[2], tail_len, counters, status)
    K.check_status(status.view(torch.uint8))
    assert tail_len.tolist() == [1, 1]


def test_bounded_wait_runs_out_and_reports_block_and_site():
    from bmx_b200 import kernels as K
    from bmx_b200._lib import BmxkError

    dev = _dev()
    status = torch.zeros(64, dtype=torch.int32, device=dev)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    K.selftest_bounded_wait(status, 2_000_000)  # ~1 ms at 2 GHz
    t1.record()
    torch.cuda.synchronize()
    assert t0.elapsed_time(t1) < 5000.0, "the wait did not end near its limit"  # the clock is read every 256 polls
    assert status[:4].tolist() == [1, 0, 77, 2], status[:4].tolist()
    with pytest.raises(BmxkError) as ei:
        K.check_status(status.view(torch.uint8))
    assert ei.value.code == 3 and "site 77" in str(ei.value)
    # the context is still usable and a limit outside the allowed range is refused on the host
    assert int((torch.ones(8, device=dev) * 2).sum()) == 16
    with pytest.raises(BmxkError):
        K.selftest_bounded_wait(status, 10**12)


def test_exchange_kernel_alone_on_one_gpu():
    """bmxk_xchg_merge with a world of one: the rank stores its state into its own buffer, flags, finds its flag and
    normalises; two steps use both buffer parities, a third takes the step number from the buffer's own count.  (Several
    ranks are exercised by tests/multi_gpu_seqsplit.py on boxes with more than one GPU; kernels of two ranks that wait for
    each other are never launched on one GPU.)"""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    import ctypes

    from bmx_b200._lib import DTYPE_F32, call, lib

    dev = torch.device("cuda:0")
    rows = 48
    lib()
    buf, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
    call("bmxk_xchg_alloc", rows, 1, ctypes.byref(buf), handle)
    try:
        ptrs = (ctypes.c_void_p * 1)(buf.value)
        status = torch.zeros(4, dtype=torch.int32, device=dev)
        g = torch.Generator().manual_seed(3)
        stream = torch.cuda.current_stream().cuda_stream
        for step in (1, 2, 0):  # 0: "the step after the last completed one" (3)
            part = torch.rand(rows, 130, generator=g).to(dev)
            part[:, 1] += 0.5
            out = torch.empty(rows, 128, dtype=torch.float32, device=dev)
            call("bmxk_xchg_merge", part.data_ptr(), rows, 0, 1, ptrs, step, 2_000_000_000, status.data_ptr(), out.data_ptr(), DTYPE_F32, stream)
            torch.cuda.synchronize()
            assert status.cpu().tolist() == [0, 0, 0, 0]
            torch.testing.assert_close(out, part[:, 2:] / part[:, 1:2], rtol=1e-6, atol=0)
    finally:
        call("bmxk_xchg_free", buf)
