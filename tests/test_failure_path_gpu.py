"""The path a kernel takes when one of its bounded device-side waits gives up: the wait
returns, the kernel records a status word and exits normally, the host reads B200K_ETIMEOUT and
the context stays usable.  The expiry is produced without any fault: one warp waits 1 ms on a
barrier that nothing arrives on."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_expired_wait_is_reported_and_context_survives(cuda_device):
    from b200k import _lib, gemm
    L = _lib.lib()
    assert _lib.device_status() == (0, 0)
    rc = L.b200k_debug_wait_timeout(1_000_000, torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    code, detail = _lib.device_status()          # synchronises, reads and clears
    assert code == -7 and (detail >> 24) == 15
    assert _lib.strerror(code) == "a bounded device-side wait expired"
    assert _lib.device_status() == (0, 0)        # cleared
    # the context is intact: a real kernel runs and is correct afterwards
    a = torch.eye(256, dtype=torch.float16, device=cuda_device)
    b = torch.arange(256 * 256, dtype=torch.float32, device=cuda_device).remainder(17).reshape(256, 256).half()
    assert torch.equal(gemm.gemm(a, b), b)
    assert L.b200k_debug_wait_timeout(0, None) == -9   # limit out of range is refused
