"""How a step's batch is laid out in its one buffer (no GPU): the general layout and the shortcut for decode steps."""
from types import SimpleNamespace

import numpy as np
import pytest

from rust_mlx_b200.cache.page_table import GroupGeometry, PageTable
from rust_mlx_b200.engine.batch import BatchLayout, SequenceInput


def pools_with(lengths: dict, page: int = 4):
    table = PageTable([GroupGeometry(32, page, 0)], 8)
    for req, n in lengths.items():
        table.open(req)
        table.reserve(req, n)
        table.commit(req, n)
    return SimpleNamespace(table=table, paged_groups=[SimpleNamespace(table_index=0)], page_size=page)


def filled(seqs, pools, rows, entries=4, **kw):
    layout = BatchLayout(sum(len(s.tokens) for s in seqs), len(seqs), rows, [entries])
    buf = np.zeros(layout.total, dtype=np.int32)
    for s in seqs:
        pools.table.reserve(s.req, s.start + len(s.tokens))
    facts = layout.fill(buf, seqs, pools, 100, **kw)
    return layout, buf, facts


def test_general_layout_of_a_mixed_step():
    pools = pools_with({1: 5, 2: 0, 3: 9})
    seqs = [SequenceInput(1, 5, [7], [0]), SequenceInput(2, 0, [1, 2, 3], [2]), SequenceInput(3, 9, [4, 5], [0, 1])]
    layout, buf, facts = filled(seqs, pools, 4, temperatures=[0.0, 0.5, 0.0, 0.25], uniforms=[0.0, 0.1, 0.0, 0.9])
    part = lambda i, n=None: layout.part(buf, i, n)   # noqa: E731
    assert part(0).tolist() == [7, 1, 2, 3, 4, 5]
    assert part(1).tolist() == [5, 0, 1, 2, 9, 10]               # positions
    assert part(2).tolist() == [0, 1, 1, 1, 2, 2]                # sequence of every token
    assert part(3).tolist() == [0, 1, 4, 6] and part(4).tolist() == [6, 3, 11]
    assert part(6).tolist() == [0, 3, 4, 5]                      # wanted rows, in the order of the entries and of want
    slots = [pools.table.slot(r) for r in (1, 2, 3)]
    assert part(5).tolist() == slots and part(10).tolist() == [slots[0], slots[1], slots[2], slots[2]]
    assert part(7).view(np.float32).tolist() == [0.0, 0.5, 0.0, 0.25]
    tables = part(11).reshape(3, 4)
    assert (tables[0][:2] >= 0).all() and tables[0][2] == -1 and (tables[2][:3] >= 0).all()
    assert facts["max_q_len"] == 3 and facts["max_seq_len"] == 11 and not facts["any_from_last"]
    with pytest.raises(ValueError, match="place"):
        filled([SequenceInput(1, 6, [7], [1])], pools, 1)
    with pytest.raises(ValueError, match="vocabulary"):
        filled([SequenceInput(1, 6, [100], [0])], pools, 1)


def test_the_decode_shortcut_is_taken_only_when_every_sequence_wants_its_one_row():
    """One token per sequence and as many wanted rows as sequences is not yet a decode step: a sequence may want its
    row twice and another not at all.  Then the general layout must be written (rows 0, 0), not rows 0, 1."""
    pools = pools_with({1: 5, 2: 7})
    odd = [SequenceInput(1, 5, [7], [0, 0]), SequenceInput(2, 7, [9], [])]
    layout, buf, _ = filled(odd, pools, 2)
    slot1 = pools.table.slot(1)
    assert layout.part(buf, 6).tolist() == [0, 0] and layout.part(buf, 10).tolist() == [slot1, slot1]
    plain = [SequenceInput(1, 6, [7], [0]), SequenceInput(2, 8, [9], [0], from_last=True)]
    layout, buf, facts = filled(plain, pools, 2)
    assert layout.part(buf, 6).tolist() == [0, 1] and layout.part(buf, 9).tolist() == [0, 1] and facts["any_from_last"]
    assert layout.part(buf, 1).tolist() == [6, 8] and layout.part(buf, 4).tolist() == [7, 9]
    with pytest.raises(ValueError, match="place"):
        filled([SequenceInput(1, 7, [7], [1]), SequenceInput(2, 9, [9], [0])], pools, 2)
