"""The cache's bookkeeping on the CPU: no slot or page lost, held twice or freed twice."""
import random

import pytest
import torch

from gogguf_b200.cache import CacheError, CacheFull, FreeList, KVRequest, SequenceCache, StateRequest


def test_free_list():
    f = FreeList(3)
    a, b, c = f.take(), f.take(), f.take()
    assert sorted([a, b, c]) == [0, 1, 2] and f.free_count == 0
    with pytest.raises(CacheFull):
        f.take()
    f.give(b)
    with pytest.raises(CacheError):
        f.give(b)                      # freed twice
    with pytest.raises(CacheError):
        f.give(7)                      # never existed
    assert f.take() == b               # last freed is first reused
    f.check()


def make_cache(max_tokens=640, window=None, state=False, max_slots=None):
    reqs = [KVRequest(2, 8), KVRequest(2, 8, window=window) if window else KVRequest(2, 8), None]
    cache_of = [None, None, None]
    if state:
        reqs.append(StateRequest((3,), torch.float32))
        cache_of.append(None)
    return SequenceCache(reqs, cache_of, max_tokens, dtype=torch.float32, device="cpu", max_slots=max_slots)


def test_groups_by_need():
    c = make_cache(window=16)
    assert len(c.groups) == 2 and c.groups[0].k.shape == (1, 10, 2, 64, 8)
    same = make_cache()
    assert len(same.groups) == 1 and same.groups[0].k.shape[0] == 2
    assert same.view(0).k.data_ptr() != same.view(1).k.data_ptr()
    assert same.view(2) is None


def test_plan_commit_lengths_and_capacity():
    c = make_cache(max_tokens=256)          # 4 pages
    a, b = c.open(), c.open()
    c.plan([a, b], [65, 3])                 # 2 + 1 pages
    assert c.length(a) == 0                 # lengths move only at commit (cache.go:37-45)
    c.commit([a, b], [65, 3])
    assert (c.length(a), c.length(b)) == (65, 3)
    c.plan([b], [61])                       # still in b's first page
    c.commit([b], [61])
    with pytest.raises(CacheFull):
        c.plan([a, b], [64, 64])            # needs 2 more pages, 1 free; nothing may be reserved
    assert c.groups[0].pages.free_count == 1
    c.plan([b], [1])
    c.commit([b], [1])
    assert c.groups[0].pages.free_count == 0
    c.check()
    c.close(a)
    assert c.groups[0].pages.free_count == 2
    with pytest.raises(CacheError):
        c.close(a)                          # closed twice
    with pytest.raises(CacheError):
        c.plan([a], [1])                    # not open
    with pytest.raises(CacheError):
        c.plan([b, b], [1, 1])
    c.check()


def test_slots_and_pages_are_reused():
    c = make_cache(max_tokens=128, max_slots=2)
    s1 = c.open()
    c.plan([s1], [100]); c.commit([s1], [100])
    pages1 = list(c.groups[0].seq_pages[s1])
    c.close(s1)
    s2 = c.open()
    assert s2 == s1 and c.length(s2) == 0
    c.plan([s2], [70]); c.commit([s2], [70])
    assert set(c.groups[0].seq_pages[s2]) == set(pages1)
    c.check()


def test_window_group_gives_pages_back():
    c = make_cache(max_tokens=64 * 8, window=70)
    s = c.open()
    c.plan([s], [64 * 4]); c.commit([s], [64 * 4])
    full, win = c.groups
    assert full.pages.held_count == 4
    # length 256, window 70: positions below 187 are out of every later window; pages 0 and 1 (0..127) go
    assert win.pages.held_count == 2
    assert win.table_row(s, 6)[2:4] == win.seq_pages[s][2:4]
    c.plan([s], [1]); c.commit([s], [1])
    assert win.pages.held_count == 3 and full.pages.held_count == 5
    c.check()
    c.close(s)
    assert win.pages.held_count == 0 and full.pages.held_count == 0
    c.check()


def test_state_is_zeroed_when_a_slot_is_opened():
    c = make_cache(state=True, max_slots=2)
    s = c.open()
    c.view(3).state[s] += 5.0
    c.close(s)
    s2 = c.open()
    assert s2 == s and float(c.view(3).state[s2].abs().sum()) == 0.0


def test_reading_another_entrys_cache():
    reqs = [KVRequest(1, 4), KVRequest(1, 4)]
    c = SequenceCache(reqs, [None, 0], 64, dtype=torch.float32, device="cpu")
    assert c.view(1) is c.view(0) and c.groups[0].k.shape[0] == 1
    with pytest.raises(CacheError):
        SequenceCache([None, KVRequest(1, 4)], [None, 0], 64, dtype=torch.float32, device="cpu")


def test_random_traffic_keeps_the_books():
    rng = random.Random(0)
    c = make_cache(max_tokens=64 * 12, window=40, max_slots=5)
    live = {}
    for _ in range(400):
        op = rng.random()
        if op < 0.3 and c.slots.free_count:
            live[c.open()] = 0
        elif op < 0.5 and live:
            s = rng.choice(list(live))
            c.close(s); del live[s]
        elif live:
            ss = rng.sample(list(live), rng.randint(1, len(live)))
            ns = [rng.randint(1, 90) for _ in ss]
            try:
                c.plan(ss, ns)
            except CacheFull:
                pass
            else:
                c.commit(ss, ns)
                for s, n in zip(ss, ns):
                    live[s] += n
        c.check()
        for s, n in live.items():
            assert c.length(s) == n
    for s in list(live):
        c.close(s)
    c.check()
    assert all(g.pages.held_count == 0 for g in c.groups) and c.slots.held_count == 0


def test_truncate_gives_pages_back_and_restart_empties_the_slot():
    c = SequenceCache([KVRequest(1, 4)], [None], 64 * 6, dtype=torch.float32)
    a, b = c.open(), c.open()
    c.plan([a, b], [200, 10]); c.commit([a, b], [200, 10])
    free = c.free_tokens()
    assert c.truncate(a, 200) and c.free_tokens() == free
    assert c.truncate(a, 65)
    assert c.length(a) == 65 and c.free_tokens() == free + 2 * 64
    c.check()
    c.plan([a], [64]); c.commit([a], [64])            # grows again from where it was cut
    assert c.length(a) == 129 and c.free_tokens() == free + 64
    with pytest.raises(CacheError):
        c.truncate(a, 130)
    c.restart(a)
    assert c.length(a) == 0 and c.length(b) == 10 and c.live_slots == 2
    c.check()
    c.close(a); c.close(b)
    assert c.free_tokens() == 64 * 6
    c.check()


def test_truncate_refuses_what_a_window_or_a_state_has_let_go():
    c = SequenceCache([KVRequest(1, 4, window=70)], [None], 64 * 8, dtype=torch.float32)
    s = c.open()
    c.plan([s], [200]); c.commit([s], [200])          # positions below 131 have left the window: pages 0 and 1 are gone
    assert c.truncate(s, 199)                         # reads 130..198: page 2 onwards
    assert not c.truncate(s, 190) and c.length(s) == 199      # would read 121..: page 1 is gone
    c.check()
    c2 = SequenceCache([StateRequest((3,))], [None], 64 * 2, dtype=torch.float32, max_slots=2)
    s2 = c2.open()
    c2.plan([s2], [5]); c2.commit([s2], [5])
    assert c2.truncate(s2, 5) and not c2.truncate(s2, 4)
    c2.restart(s2)
    assert c2.length(s2) == 0


def test_a_step_that_fails_after_plan_gives_its_pages_back_and_entries_get_a_status_each():
    """`Stepper` on the CPU with a model stand-in: everything up to the first launch is host code."""
    from types import SimpleNamespace
    from gogguf_b200.engine.step import StepEntry, StepError, Stepper
    cache = SequenceCache([KVRequest(1, 4), KVRequest(1, 4, window=70)], [None, None], 64 * 6, dtype=torch.float32)
    spec = SimpleNamespace(vocab_size=50, max_positions=200, hidden_size=8, schedule=())
    model = SimpleNamespace(spec=spec, rt=SimpleNamespace(device=torch.device("cpu"), dtype=torch.float32),
                            blocks=[], parts=lambda: [])
    st = Stepper(model, cache)
    ran = []

    def fake_layers(ctx, taps=None, tap_rows=None):
        ran.append(int(ctx.n_tokens))
        if fail[0]:
            raise RuntimeError("a launcher refused")
        return torch.zeros(ctx.n_tokens, 8)

    st.run_layers = fake_layers
    st.run_head = lambda ctx, x, rows, n: torch.zeros(n, 50)
    fail = [True]
    a, b = cache.open(), cache.open()
    st_before = (cache.free_tokens(), list(cache.lengths))
    with pytest.raises(RuntimeError):
        st.step([StepEntry(a, [1] * 100, want=[99]), StepEntry(b, [2] * 70)])
    cache.check()
    assert (cache.free_tokens(), list(cache.lengths)) == st_before        # nothing stays reserved
    fail[0] = False
    # per-entry status: the bad ones are named, the others run
    c = cache.open()
    out = st.try_step([StepEntry(a, [1, 2, 3], want=[2]),
                       StepEntry(b, [1, 99]),                # token outside the vocabulary
                       StepEntry(7, [1]),                    # not an open slot
                       StepEntry(a, [4]),                    # the same slot twice
                       StepEntry(c, [1] * 201),              # longer than the context
                       StepEntry(c, [5, 6], want=[0, 1])])
    assert [s.code if s else None for s in out.status] == [None, "bad_token", "unknown_slot", "duplicate_slot",
                                                           "context_overflow", None]
    assert out.ran == [0, 5] and out.logits.shape == (3, 50)
    assert cache.length(a) == 3 and cache.length(b) == 0 and cache.length(c) == 2
    # the cache holds 6 pages: a and c hold one each; b wants 3, a fourth sequence wants 2 -> left out from the end
    d = cache.open()
    out = st.try_step([StepEntry(b, [1] * 150), StepEntry(d, [1] * 100)])
    assert [s.code if s else None for s in out.status] == [None, "cache_full"]
    assert cache.length(b) == 150 and cache.length(d) == 0
    with pytest.raises(CacheFull):                   # the strict form refuses the whole step, cache untouched
        st.step([StepEntry(d, [1] * 100)])
    with pytest.raises(StepError):
        st.step([StepEntry(d, [1]), StepEntry(b, [77])])
    assert cache.length(d) == 0
    cache.check()
    for s in (a, b, c, d):
        cache.close(s)
    cache.check()
    assert cache.free_tokens() == 64 * 6
