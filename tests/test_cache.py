"""The cache's bookkeeping on the CPU: no slot or page is ever lost, held twice or freed twice;
lengths, reservations and windows; per-sequence state starts at zero on a reused slot."""

import random

import pytest
import torch

from dryft_b200.cache import CacheError, FreeList, KVNeed, PageLedger, SequenceCache, StateNeed, pages_for


def test_free_list_invariants():
    f = FreeList(5, "slot")
    a = f.take(3)
    assert a == [0, 1, 2] and f.n_free == 2 and f.n_held == 3
    f.check()
    with pytest.raises(CacheError):
        f.take(3)  # only 2 left; nothing is taken on failure
    assert f.n_free == 2
    f.give_back([1])
    with pytest.raises(CacheError):
        f.give_back([1])  # freed twice
    with pytest.raises(CacheError):
        f.give_back([4])  # never taken
    with pytest.raises(CacheError):
        f.give_back([0, 0])
    with pytest.raises(CacheError):
        f.give_back([9])
    assert f.take(1) == [1]  # the freed id is handed out again first
    f.check()


def test_free_list_random_walk():
    rng = random.Random(0)
    f = FreeList(17, "page")
    held = set()
    for _ in range(2000):
        if held and rng.random() < 0.5:
            ids = rng.sample(sorted(held), rng.randint(1, len(held)))
            f.give_back(ids)
            held -= set(ids)
        else:
            n = rng.randint(0, 4)
            if n <= f.n_free:
                got = f.take(n)
                assert not (set(got) & held)
                held |= set(got)
            else:
                with pytest.raises(CacheError):
                    f.take(n)
        f.check()
        assert f.n_held == len(held) and f.n_free == 17 - len(held)


def test_page_ledger_growth_close_and_window():
    led = PageLedger(n_pages=6, page_size=64, max_pages_per_slot=4)
    led.open(0)
    assert led.grow(0, 0, 65) == {0: 0, 1: 1}
    assert led.grow(0, 65, 128) == {}          # still inside page 1
    assert list(led.grow(0, 128, 129)) == [2]
    with pytest.raises(CacheError):
        led.grow(0, 129, 64 * 4 + 1)           # beyond the longest sequence
    led.open(1)
    with pytest.raises(CacheError):
        led.grow(1, 0, 64 * 4)                 # 4 pages wanted, 3 free
    led.check()
    with pytest.raises(CacheError):
        led.open(1)
    led.close(0)
    with pytest.raises(CacheError):
        led.close(0)
    assert led.pool.n_free == 6
    led.check()
    # a windowed group gives pages back once every position in them is out of sight
    w = PageLedger(n_pages=4, page_size=64, max_pages_per_slot=100, window=40)
    w.open(3)
    w.grow(3, 0, 130)
    assert w.trim(3, 130) == [0]               # next query at 130 sees keys 91.. -> page 0 is dead
    assert w.trim(3, 130) == []
    w.grow(3, 130, 300)                        # needs pages 3,4: only possible because page 0 came back...
    assert sorted(w.held(3)) == [1, 2, 3, 4]
    held = w.held(3)
    dead = w.trim(3, 300)                      # next query at 300 sees keys 261.. -> pages 1..3 are dead
    assert sorted(dead) == sorted(held[lp] for lp in (1, 2, 3)) and sorted(w.held(3)) == [4]
    w.check()
    w.close(3)
    assert w.pool.n_free == 4


def _cache(window=None, max_tokens=512, slots=3, state=False, device="cpu"):
    needs = [(KVNeed(2, 16, None), None), (KVNeed(2, 16, window), StateNeed((4,), torch.float32) if state else None),
             (KVNeed(2, 16, None), None)]
    return SequenceCache(needs, [None, None, 0], max_tokens=max_tokens, max_slots=slots, max_seq_len=256, page_size=64,
                         dtype=torch.float32, device=torch.device(device))


def test_groups_have_storage_of_their_own_and_borrowers_share():
    c = _cache(window=40)
    assert c.n_groups() == 2  # all keys / a window of them
    e0, e1, e2 = c.entry(0), c.entry(1), c.entry(2)
    assert e0.k.data_ptr() != e1.k.data_ptr() and e0.page_table.data_ptr() != e1.page_table.data_ptr()
    assert e2.k.data_ptr() == e0.k.data_ptr() and e1.window == 40 and e0.window is None
    assert e0.k.shape == (8, 2, 64, 16) and float(e0.k.abs().max()) == 0.0  # zero-initialised
    same = _cache(window=None)
    assert same.n_groups() == 1 and same.entry(0).k.shape == same.entry(1).k.shape
    assert same.entry(0).k.data_ptr() != same.entry(1).k.data_ptr()  # same group, entries of their own


def test_sequences_reserve_advance_and_give_back():
    c = _cache()
    a, b = c.open_sequences(2)
    c.reserve(a, 70)
    c.reserve(b, 1)
    c.flush()
    for g in c._groups:  # the device page table shows what the ledger holds
        held = g.ledger.held(a)
        assert sorted(held) == [0, 1] and [int(g.page_table[a, lp]) for lp in (0, 1)] == [held[0], held[1]]
    c.advanced(a, 70)
    c.advanced(b, 1)
    assert c.len_host[a] == 70 and c.len_host[b] == 1
    c.reserve(a, 58)      # to 128: still two pages
    c.advanced(a, 58)
    c.reserve(a, 1)       # 129: a third page
    c.advanced(a, 1)
    c.check()
    assert c.free_tokens() == 512 - 64 * 4
    with pytest.raises(CacheError):
        c.reserve(a, 200)  # beyond max_seq_len
    with pytest.raises(CacheError):
        c.reserve(2, 1)    # slot not held
    assert c.can_hold([64]) and not c.can_hold([64, 64]) and not c.can_hold([300])
    c.close_sequences([a])
    with pytest.raises(CacheError):
        c.close_sequences([a])
    assert c.open_sequences(1) == [a] and c.len_host[a] == 0  # the slot is used again, from length zero
    with pytest.raises(CacheError):
        c.open_sequences(2)  # one slot left
    c.check()
    c.close_sequences([a, b])
    assert c.slots.n_held == 0 and c.free_tokens() == 512
    c.check()


def test_cache_full_takes_nothing():
    c = _cache(max_tokens=128, slots=3)
    a, b = c.open_sequences(2)
    c.reserve(a, 64)
    c.advanced(a, 64)
    c.reserve(b, 64)
    c.advanced(b, 64)
    with pytest.raises(CacheError) as e:
        c.reserve(a, 1)
    assert "cache full" in str(e.value)
    c.check()
    c.close_sequences([b])
    c.reserve(a, 1)
    c.check()


def test_state_is_zeroed_when_a_slot_is_reused():
    c = _cache(state=True)
    (s,) = c.open_sequences(1)
    st = c.state(1)
    assert st.shape == (3, 4) and c.state(0) is None
    st[s] = 7.0
    c.seq_len[s] = 9
    c.last_token[s] = 5
    c.close_sequences([s])
    (s2,) = c.open_sequences(1)
    assert s2 == s and float(st[s].abs().max()) == 0.0 and int(c.seq_len[s]) == 0 and int(c.last_token[s]) == 0


def test_a_mixer_may_ask_for_several_named_states():
    """A mapping of names to ``StateNeed`` gives a mapping of tensors of their own shapes and dtypes, all zeroed
    when the slot is taken again; a borrower shares them; anything else is refused."""
    import pytest

    from dryft_b200.cache.slots import CacheError

    two = {"tail": StateNeed((3, 5), torch.bfloat16), "h": StateNeed((4,), torch.float32)}
    c = SequenceCache([(None, two), (KVNeed(2, 16, None), None), (None, None)], [None, None, 0], max_tokens=256, max_slots=2,
                      max_seq_len=128, page_size=64, dtype=torch.float32, device=torch.device("cpu"))
    st = c.state(0)
    assert set(st) == {"tail", "h"} and st["tail"].shape == (2, 3, 5) and st["tail"].dtype == torch.bfloat16
    assert st["h"].shape == (2, 4) and st["h"].dtype == torch.float32
    assert c.state(2) is st and c.state(1) is None
    a, b = c.open_sequences(2)
    st["tail"][a] = 1.0
    st["h"][a] = 2.0
    st["h"][b] = 3.0
    c.close_sequences([a])
    (a2,) = c.open_sequences(1)
    assert a2 == a and float(st["tail"][a].abs().max()) == 0.0 and float(st["h"][a].abs().max()) == 0.0
    assert float(st["h"][b].min()) == 3.0          # the other sequence's state is untouched
    with pytest.raises(CacheError):
        SequenceCache([(None, {"x": 3})], [None], max_tokens=64, max_slots=1, max_seq_len=64, page_size=64,
                      dtype=torch.float32, device=torch.device("cpu"))


def _random_traffic(device):
    rng = random.Random(1)
    c = _cache(window=40, max_tokens=1024, slots=3, device=device)
    live = {}
    for _ in range(400):
        r = rng.random()
        if r < 0.25 and c.slots.n_free:
            (s,) = c.open_sequences(1)
            live[s] = 0
        elif r < 0.45 and live:
            s = rng.choice(sorted(live))
            c.close_sequences([s])
            del live[s]
        elif live:
            s = rng.choice(sorted(live))
            n = rng.choice([1, 1, 1, 5, 64, 100])
            try:
                c.reserve(s, n)
            except CacheError:
                continue
            c.flush()
            for g in c._groups:   # after a flush the device's page tables are the host's, row for row
                assert torch.equal(g.page_table.cpu(), g.page_table_host)
            c.advanced(s, n)
            live[s] += n
            assert c.len_host[s] == live[s]
        c.check()
    c.close_sequences(sorted(live))
    c.check()
    assert c.free_tokens() == 1024


def test_random_traffic_never_loses_a_page():
    _random_traffic("cpu")


@pytest.mark.gpu
def test_random_traffic_on_the_device_keeps_the_page_tables_equal():
    """The same traffic with the tables on the GPU: changed rows travel as one pinned asynchronous copy."""
    _random_traffic("cuda:0")
