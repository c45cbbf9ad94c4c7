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
