"""A step's packed metadata: in a step that mixes single tokens with longer portions the single tokens come
first in the flat batch, and the wanted rows keep the caller's order."""
import torch

from qwen_decoder_b200.cache import CacheLayout, CacheManager, PagedKV
from qwen_decoder_b200.engine.batch import StepEntry, build_context


def manager():
    layout = CacheLayout.from_needs([PagedKV(2, 16)], [None])
    return CacheManager(layout, num_pages=16, page_size=16, max_requests=8, device=torch.device("cpu"))


def opened(m, name, held):
    rc = m.open(name)
    m.ensure(rc, held)
    m.commit(rc, held)
    return rc


def test_single_tokens_come_first_and_logits_keep_their_order():
    m = manager()
    a, b, c, d = opened(m, "a", 0), opened(m, "b", 20), opened(m, "c", 7), opened(m, "d", 33)
    entries = [StepEntry(a, [1, 2, 3, 4, 5], [4]), StepEntry(b, [9], [0]), StepEntry(c, [6, 7, 8], []),
               StepEntry(d, [11], [0])]
    for e in entries:
        m.ensure(e.cache, e.cache.num_tokens + len(e.tokens))
    ctx = build_context(entries, m, "cpu", 100, 1000)
    assert not ctx.all_decode and ctx.num_decode == 2 and ctx.decode_max_context == 34
    assert ctx.tokens.tolist() == [9, 11, 1, 2, 3, 4, 5, 6, 7, 8]
    assert ctx.positions.tolist() == [20, 33, 0, 1, 2, 3, 4, 7, 8, 9]
    assert ctx.token_request.tolist() == [0, 1, 2, 2, 2, 2, 2, 3, 3, 3]
    assert ctx.cu_tokens.tolist() == [0, 1, 2, 7, 10] and ctx.start_pos.tolist() == [20, 33, 0, 7]
    # wanted rows in the caller's order: a's last token, b's token, d's token
    assert ctx.logit_rows.tolist() == [6, 0, 1]
    # the block table rows follow the step's own order of requests
    assert ctx.groups[0].block_table[0, :2].tolist() == b.tables[0].pages[:2]
    assert ctx.groups[0].block_table[2, :1].tolist() == a.tables[0].pages[:1]


def test_steps_that_are_not_mixed_keep_the_given_order():
    m = manager()
    a, b = opened(m, "a", 3), opened(m, "b", 18)
    for rc in (a, b):
        m.ensure(rc, rc.num_tokens + 2)
    ctx = build_context([StepEntry(a, [1, 2], [1]), StepEntry(b, [3, 4], [0, 1])], m, "cpu", 100, 1000)
    assert ctx.num_decode == 0 and ctx.tokens.tolist() == [1, 2, 3, 4] and ctx.logit_rows.tolist() == [1, 2, 3]
    ctx = build_context([StepEntry(a, [5], [0]), StepEntry(b, [6], [0])], m, "cpu", 100, 1000)
    assert ctx.all_decode and ctx.num_decode == 0 and ctx.tokens.tolist() == [5, 6]


def test_random_batches_keep_every_token_with_its_request():
    """Random mixes of single tokens and portions: whatever the order inside the step, every wanted row is
    the token the caller meant, at its position, in a slot of its own request's pages."""
    import random
    rng = random.Random(4)
    for trial in range(60):
        m = manager()
        n = rng.randint(1, 6)
        held = [rng.randint(0, 30) for _ in range(n)]
        rcs = [opened(m, f"r{i}", held[i]) for i in range(n)]
        entries, next_token = [], 1
        for i, rc in enumerate(rcs):
            k = 1 if rng.random() < 0.5 else rng.randint(2, 9)
            toks = list(range(next_token, next_token + k))
            next_token += k
            want = sorted(rng.sample(range(k), rng.randint(0, min(k, 2))))
            m.ensure(rc, held[i] + k)
            entries.append(StepEntry(rc, toks, want))
        ctx = build_context(entries, m, "cpu", 1000, 1000)
        tokens, positions = ctx.tokens.tolist(), ctx.positions.tolist()
        req, slots = ctx.token_request.tolist(), ctx.groups[0].slot_map.tolist()
        table = ctx.groups[0].block_table.tolist()
        rows = ctx.logit_rows.tolist()
        expect = [(e, w) for e in entries for w in e.want]
        assert len(rows) == len(expect)
        for row, (e, w) in zip(rows, expect):
            assert tokens[row] == e.tokens[w] and positions[row] == e.cache.num_tokens + w
        assert sorted(tokens) == list(range(1, next_token))
        for t in range(ctx.num_tokens):
            owner = next(e for e in entries if tokens[t] in e.tokens)
            page, off = divmod(positions[t], 16)
            assert slots[t] == owner.cache.tables[0].pages[page] * 16 + off
            assert table[req[t]][:len(owner.cache.tables[0].pages)] == owner.cache.tables[0].pages
        singles = sum(1 for e in entries if len(e.tokens) == 1)
        assert ctx.num_decode == (singles if 0 < singles < n else 0)
        if ctx.num_decode:
            assert all(ctx.cu_tokens.tolist()[i + 1] - ctx.cu_tokens.tolist()[i] == 1 for i in range(singles))


def test_a_step_refuses_what_it_cannot_run():
    """Limits checked by the step function itself: tokens in a step, positions, pages, token ids, wanted places."""
    import pytest
    from qwen_decoder_b200.engine.batch import StepError
    m = manager()
    a, b = opened(m, "a", 0), opened(m, "b", 20)
    m.ensure(a, 8)
    m.ensure(b, 21)
    ok = [StepEntry(a, [1, 2, 3, 4, 5], [4]), StepEntry(b, [9], [0])]
    build_context(ok, m, "cpu", 100, 1000, max_step_tokens=6)
    with pytest.raises(StepError, match="more than max_step_tokens = 5"):
        build_context(ok, m, "cpu", 100, 1000, max_step_tokens=5)
    with pytest.raises(StepError, match="exceed the model's 21 positions"):
        build_context([StepEntry(b, [9, 9], [0])], m, "cpu", 100, 21)
    with pytest.raises(StepError, match="pages for its 30 new tokens are missing"):
        build_context([StepEntry(a, list(range(30)), [])], m, "cpu", 100, 1000)
    with pytest.raises(StepError, match="token id 100 is outside the vocabulary"):
        build_context([StepEntry(a, [1, 100], [])], m, "cpu", 100, 1000)
    with pytest.raises(StepError, match="wanted place 2 is outside its 2 tokens"):
        build_context([StepEntry(a, [1, 2], [2])], m, "cpu", 100, 1000)
    with pytest.raises(StepError, match="appears twice"):
        build_context([StepEntry(a, [1], []), StepEntry(a, [2], [])], m, "cpu", 100, 1000)
