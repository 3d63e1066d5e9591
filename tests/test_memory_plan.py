"""How large the cache pools are made, and what is refused before anything is allocated
(the reference's failsafe: src/context.c:395-429,479-491)."""
import pytest

from kappai_b200.engine.memory import CacheMemoryError, GroupNeed, pages_of_group, plan_cache

GIB = 1 << 30
KV_1P2B = [GroupNeed("kv", 12288)]            # six attention layers x K,V x 8 heads x 64 x 2 bytes
STATE_1P2B = 10 * 2 * 2048 * 4                # ten conv layers x (K-1) x hidden x 4 bytes


def test_an_asked_size_is_taken_as_it_is_or_refused_with_the_figures():
    p = plan_cache(KV_1P2B, STATE_1P2B, 64, 64, 4096, 64 * 4096, 170 * GIB)
    assert p.tokens == 64 * 4096 and p.pages == {"kv": 4096}
    assert p.cache_bytes == 64 * 4096 * 12288 + 64 * STATE_1P2B
    with pytest.raises(CacheMemoryError) as e:
        plan_cache(KV_1P2B, STATE_1P2B, 64, 64, 128000, 1 << 24, 100 * GIB)
    msg = str(e.value)
    assert "196618.0 MB" in msg and "refusing to run" in msg and "kv_tokens" in msg          # 2^24 tokens x 12 KiB and 10 MB of state
    # a count that is no multiple of the page is rounded up
    assert plan_cache(KV_1P2B, 0, 2, 64, 4096, 100, None).tokens == 128


def test_an_open_size_takes_what_the_requests_could_use_or_what_fits():
    # room for everything: max_batch x ctx_size
    p = plan_cache(KV_1P2B, STATE_1P2B, 8, 64, 4096, 0, 170 * GIB)
    assert p.tokens == 8 * 4096
    # the default command line (64 requests, the model's 128000 positions) wants 100 GB; with 40 GB free it gets less
    p = plan_cache(KV_1P2B, STATE_1P2B, 64, 64, 128000, 0, 40 * GIB)
    assert 128000 <= p.tokens < 64 * 128000 and p.tokens % 64 == 0
    assert p.cache_bytes <= 40 * GIB * 0.92 < p.cache_bytes + 64 * 12288 * 2
    # not even one request of the asked context fits: refused, with a sentence
    with pytest.raises(CacheMemoryError, match="not even one request of 128000 tokens"):
        plan_cache(KV_1P2B, STATE_1P2B, 64, 64, 128000, 0, 1 * GIB)


def test_float32_and_a_larger_model_cost_more():
    kv_2p6b_f32 = [GroupNeed("kv", 8 * 2 * 8 * 64 * 4)]
    with pytest.raises(CacheMemoryError):
        plan_cache(kv_2p6b_f32, 22 * 2 * 2048 * 4, 64, 64, 32768, 64 * 32768, 60 * GIB)
    assert plan_cache(kv_2p6b_f32, 22 * 2 * 2048 * 4, 16, 64, 32768, 16 * 32768, 120 * GIB).tokens == 16 * 32768


def test_a_windowed_group_gets_pages_for_its_windows_only():
    full, win = GroupNeed("full", 4096), GroupNeed("win", 4096, window=512)
    assert pages_of_group(win, 10000, 64, 4, 256) == 4 * (12 + 1)          # (512 + 256) / 64 pages and one more
    assert pages_of_group(win, 10, 64, 4, 256) == 10                       # never more than the full pool
    assert pages_of_group(win, 10000, 64, 4, None) == 10000                # no limit on a step known: a full pool
    assert pages_of_group(full, 10000, 64, 4, 256) == 10000
    p = plan_cache([full, win], 0, 4, 64, 8192, 0, None, max_step_tokens=256)
    assert p.pages == {"full": 4 * 8192 // 64, "win": 52}
    assert p.cache_bytes == (512 + 52) * 64 * 4096
