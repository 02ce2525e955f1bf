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


def test_engine_releases_its_kv_cache_and_keeps_its_graphs():
    """An engine whose KV cache lives in the tagged arena: release gives the memory back, resume maps it again at the same
    addresses, the captured decode graphs are still valid and the same requests produce the same tokens."""
    from miles_b200.engine import Engine, SamplingParams
    from miles_b200.models import ParamStore, build_model, get_config
    from miles_b200.utils.memory_saver import MemorySaver

    if not MemorySaver().available:
        pytest.skip("CUDA virtual memory management is not available")
    dev = torch.device("cuda")
    cfg = get_config("qwen3-smoke")
    m = build_model(cfg, ParamStore(cfg, dev, torch.bfloat16, init_std=0.02), "b200")
    eng = Engine(m, max_running=4, page_size=64, max_seq_len=2048, num_pages=4096, use_cuda_graph=True, memory_saver=True)
    assert eng._saver is not None
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (70, 130, 20)]
    sps = [SamplingParams(temperature=1.0, max_new_tokens=24, sampling_seed=i) for i in range(3)]
    first = [r["output_ids"] for r in eng.generate(prompts, sps)]
    graphs, ptr = dict(eng._graphs), eng.kv_cache[0][0].data_ptr()
    kv_bytes = 2 * cfg.num_layers * 4096 * 64 * cfg.num_kv_heads * cfg.head_dim * 2
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    eng.release_memory_occupation(("kv_cache",))
    free1, _ = torch.cuda.mem_get_info()
    assert free1 - free0 >= kv_bytes // 2, (free1 - free0, kv_bytes)
    eng.resume_memory_occupation(("kv_cache",))
    assert eng.kv_cache[0][0].data_ptr() == ptr and eng._graphs == graphs and graphs
    again = [r["output_ids"] for r in eng.generate(prompts, sps)]
    assert again == first
    m.check_status()
