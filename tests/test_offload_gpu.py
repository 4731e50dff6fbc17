"""VMM-backed offloadable buffers: contents and address survive an offload / onload cycle and
the physical memory is really returned in between."""
import pytest
import torch

from areal_b200.utils.offload import OffloadableBuffer

pytestmark = pytest.mark.gpu


def test_offload_roundtrip_keeps_address_and_contents():
    n = 256 << 20
    buf = OffloadableBuffer(n)
    t = buf.tensor(torch.int32)
    t.copy_(torch.arange(t.numel(), device="cuda", dtype=torch.int32))
    ptr = t.data_ptr()
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    buf.offload(preserve=True)
    free1, _ = torch.cuda.mem_get_info()
    assert free1 - free0 >= n * 0.9
    buf.onload()
    free2, _ = torch.cuda.mem_get_info()
    assert free1 - free2 >= n * 0.9
    assert t.data_ptr() == ptr
    assert torch.equal(t[:1000].cpu(), torch.arange(1000, dtype=torch.int32))
    assert int(t[-1]) == t.numel() - 1
    buf.offload(preserve=False)
    buf.onload()
    assert int(t.abs().max()) == 0
    buf.free()
