"""The abort path of the kernels' bounded waits (expiry -> status word -> exception -> next call
works) and the one documented deviation from the reference's numbers.  No test here makes a GPU
fault, trap or hang: the wait that expires belongs to a hook that has nothing in flight.
Needs a B200."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.fail("a CUDA device is required for -m gpu tests")
    return torch.device("cuda:0")


def test_expired_wait_reaches_the_caller_and_the_next_call_works():
    """A wait on a barrier nobody arrives at runs out after 20 microseconds: the kernel ends
    normally, the status word reads SPSATTN_STATUS_WAIT_EXPIRED, check_device_status() raises and
    clears it, and the attention call after that gives the right numbers again."""
    import sps_b200
    from sps_b200 import _lib
    from sps_b200.attention import _status
    from oracle import sps_oracle as orc
    dev = _dev()
    lib = _lib.load()
    sps_b200.check_device_status(dev)                 # clean start
    word = _status(dev)
    result = torch.zeros(1, dtype=torch.int32, device=dev)
    rc = lib.spsattn_debug_wait_expiry(word.data_ptr(), 20_000, result.data_ptr(),
                                       torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert int(result.item()) == 1                    # the wait gave up, the block ended
    assert int(word.item()) == 1                      # SPSATTN_STATUS_WAIT_EXPIRED
    with pytest.raises(_lib.SpsAttnError, match="bounded wait"):
        sps_b200.check_device_status(dev)
    assert int(word.item()) == 0                      # cleared by the check
    g = torch.Generator().manual_seed(3)
    q, k, v = (torch.randn(1, 2, 256, 64, generator=g).bfloat16() for _ in range(3))
    out = sps_b200.sps_sliding_attention(q.to(dev), k.to(dev), v.to(dev), 0.125, 8)
    sps_b200.check_device_status(dev)
    ref = orc.prefill_attention(q, k, v, 0.125, temporary_window=8)
    assert float((out.float().cpu() - ref).abs().max()) <= 2e-2
    assert lib.spsattn_debug_wait_expiry(None, 20_000, None, None) != 0      # argument errors
    assert lib.spsattn_debug_wait_expiry(word.data_ptr(), 2_000_000_000, None, None) != 0


@pytest.mark.parametrize("d", [64, 128, 32])
def test_row_without_a_visible_key_returns_zero(d):
    """Deliberate difference from the reference: a query row that sees no key at all gives 0 (and
    log-sum-exp -inf) instead of the softmax over masked keys that the reference's finite -1e6
    biases produce.  No caller of the reference has such a row (every row sees itself); here it
    is made with a temporary window of -1 and a persistent window of -1, which leaves the
    temporary-parity rows without any key.  If this ever changes it must be on purpose."""
    import sps_b200
    from oracle import sps_oracle as orc
    dev = _dev()
    g = torch.Generator().manual_seed(11)
    q, k, v = (torch.randn(1, 2, 384, d, generator=g).bfloat16().to(dev) for _ in range(3))
    out, lse = sps_b200.prefill_attention(q, k, v, 1 / math.sqrt(d), persistent_parity=0, temporary_window=-1,
                                          persistent_window=-1, return_lse=True)
    sps_b200.check_device_status(dev)
    vis = orc.visible_mask(384, persistent_parity=0, temporary_window=-1, persistent_window=-1)
    empty = torch.from_numpy(~vis.any(axis=-1).reshape(-1))
    assert bool(empty[1::2].all()) and not bool(empty[0::2].any())
    assert float(out[:, :, empty.to(dev)].float().abs().max()) == 0.0
    assert bool(torch.isinf(lse[:, :, empty.to(dev)]).all())
    # the rows that do see a key (only themselves) return their own value row
    seen = ~empty
    assert float((out[:, :, seen.to(dev)].float() - v[:, :, seen.to(dev)].float()).abs().max()) <= 1e-2
