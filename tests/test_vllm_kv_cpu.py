"""vLLM-independent parts of the KV backend, on CPU: page spec, split contract, pool watch, prefill page tables."""
import pytest
import torch


def test_page_spec_and_split_contract():
    from statetree_b200 import vllm_kv as V
    assert V.BYTES_PER_TOKEN_PER_HEAD == 400 and V.PAGE * V.BYTES_PER_TOKEN_PER_HEAD == 4 * V.RKV
    for B in (1, 2, 7, 8, 33, 64, 256):
        s = V.decode_splits(B, 8)
        assert 1 <= s <= V.MAX_SPLITS and s & (s - 1) == 0                   # a power of two
        assert s == 1 or B * 8 * s <= 3 * 148                                # never more CTAs than three per SM
        assert V.decode_splits(B, 8) == s                                    # a function of the batch size only
    assert V.decode_splits(0, 8) == 1 and V.decode_splits(1, 8) == 32 and V.decode_splits(64, 8) == 1
    cache = torch.zeros(5, 8, 16, 400, dtype=torch.uint8)
    assert V.page_view(cache, 8).shape == (5, 8, 2, 2, 1600)
    assert V.page_view(cache.view(torch.int16), 8).shape == (5, 8, 2, 2, 1600)
    with pytest.raises(RuntimeError, match="unexpected layer cache"):
        V.page_view(cache, 4)


def test_pool_watch_raises_one_step_late():
    from statetree_b200.vllm_kv import SharedPool
    sh = SharedPool("cpu", 32, 8, pool_mb=1)
    assert sh.pool.shape == (16384, 16)
    assert sh.poll() is None and sh.steps == 1
    sh.cnt[0] = 9000                                                         # more than half the blocks in use
    assert sh.poll() is None                                                 # this step still sees the old copy
    note = sh.poll()
    assert note is not None and "extension pool" in note
    sh.cnt[1] = 1                                                            # the kernel flagged exhaustion
    sh.poll()
    with pytest.raises(RuntimeError, match="exhausted"):
        sh.poll()


def test_one_pool_per_process_and_device(monkeypatch):
    import statetree_b200.vllm_kv as V
    monkeypatch.setenv("STATETREE_KV_POOL_MB", "1")
    monkeypatch.setattr(V, "_POOLS", {})
    a = V.shared_pool("cpu", 32, 8)
    assert V.shared_pool(torch.device("cpu"), 32, 8) is a                    # every layer of a model shares it
    with pytest.raises(NotImplementedError, match="different head counts"):
        V.shared_pool("cpu", 16, 8)
    a.cnt[0] = 7
    assert V.pool_usage() == {("cpu", None): (7, 16384, False)}


def test_prefill_page_tables():
    from statetree_b200.vllm_kv import prefill_page_tables
    bt = torch.arange(40, dtype=torch.int32).view(4, 10) + 100               # 4 requests, the first is a decode
    blocks, table = prefill_page_tables(torch.tensor([17, 48, 1]), bt, first_request=1)
    assert blocks.tolist() == [110, 111, 120, 121, 122, 130]                 # 2 + 3 + 1 pages
    assert table.tolist() == [[0, 1, 0], [2, 3, 4], [5, 0, 0]]


def test_register_reports_why_nothing_is_installed():
    from statetree_b200.vllm_kv import register
    ok, why = register()
    assert ok is False and isinstance(why, str) and why
