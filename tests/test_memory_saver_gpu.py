"""Tagged virtual-memory arena: pause releases physical memory, resume restores it at the same address."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_pause_resume_keeps_addresses_and_contents():
    from miles_b200.utils.memory_saver import MemorySaver

    ms = MemorySaver()
    if not ms.available:
        pytest.skip("CUDA virtual memory management is not available")
    n = 256 << 20  # 256 MiB
    with ms.region("kv"):
        x = torch.arange(n // 4, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    ptr = x.data_ptr()
    free0, _ = torch.cuda.mem_get_info()
    released = ms.pause("kv", keep_contents=True)
    free1, _ = torch.cuda.mem_get_info()
    assert released >= n and free1 - free0 >= n // 2
    # nothing touches x while it is paused
    mapped = ms.resume("kv")
    assert mapped == released and x.data_ptr() == ptr
    assert int(x[12345].item()) == 12345 and int(x[-1].item()) == n // 4 - 1
    st = ms.stats()
    assert st["kv"][0] >= n and st["kv"][1] == 0
    del x
