"""The work list of talking-heads attention for the tensor-core form: tiles, parts and rows of partial sums."""
import numpy as np
import pytest

from rustingstrata_b200.parts import talking_attention as TA
from rustingstrata_b200.parts.base import HostBatch


def make_part(mma_q=16, window=0, chunk=0):
    att = TA.TalkingAttention.__new__(TA.TalkingAttention)
    att.q_per_cta, att.mma_q, att.window, att.chunk = 8, mma_q, window, chunk
    att.n_heads, att.n_kv, att.dk, att.dv = 16, 4, 64, 64
    return att


def batch(q_lens, kv_lens, bucketed=False):
    q_lens, kv_lens = np.asarray(q_lens, dtype=np.int32), np.asarray(kv_lens, dtype=np.int32)
    q_start = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
    return HostBatch(n_tokens=int(q_lens.sum()), n_seqs=len(q_lens), q_lens=q_lens, kv_lens=kv_lens, q_start=q_start,
                     state_slots=np.arange(len(q_lens), dtype=np.int32), first_step=np.zeros(len(q_lens), np.int32),
                     page_size=16, max_blocks=[1], bucketed=bucketed)


def rows_of(plan):
    return plan["work"].reshape(-1, 5)


def test_single_tokens_share_out_long_contexts():
    plan = make_part().build_plan(batch([1, 1, 1], [4000, 40, 700]))
    w = rows_of(plan)
    assert plan["qt"] == TA.MMA_SINGLE_Q and plan["any_parts"] == 1
    by_seq = {s: w[w[:, 0] == s] for s in range(3)}
    assert len(by_seq[1]) == 1 and by_seq[1][0, 3] == 1                      # two key tiles: one CTA
    assert len(by_seq[0]) == by_seq[0][0, 3] == min(TA.MAX_PARTS, TA.FILL_CTAS // 3, 125 // TA.MIN_PART_TILES)
    assert len(by_seq[2]) == by_seq[2][0, 3] == 22 // TA.MIN_PART_TILES
    assert (w[:-1, 0] != w[1:, 0]).sum() == 2                                # a tile's parts are neighbours
    # rows of partial sums do not overlap
    spans = sorted((r[4], r[4] + r[3]) for r in w if r[2] == 0 and r[3] > 1)
    assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:]))
    for s in (0, 2):
        assert list(by_seq[s][:, 2]) == list(range(len(by_seq[s])))


def test_a_full_step_is_not_shared_out():
    plan = make_part().build_plan(batch([2048] * 4, [2048] * 4))
    w = rows_of(plan)
    assert plan["any_parts"] == 0 and (w[:, 3] == 1).all() and len(w) == 4 * 128 and plan["qt"] == 16
    first = w[:, 1]
    assert (np.diff(first) <= 0).all()                                       # most keys first


def test_one_long_portion_is_shared_out_in_two():
    plan = make_part().build_plan(batch([2048], [2048]))
    w = rows_of(plan)
    heads = w[w[:, 2] == 0]
    assert len(heads) == 128 and plan["any_parts"] == 1
    assert (heads[heads[:, 1] >= 8 * 16 * 2, 3] == 2).all()                  # tiles with at least 8 key tiles: two parts
    assert (heads[heads[:, 1] < 7 * 16 * 2 - 16, 3] == 1).all()              # short walks stay whole


def test_captured_steps_keep_their_shape():
    a = make_part().build_plan(batch([1] * 8, [100 + i for i in range(8)], bucketed=True))
    b = make_part().build_plan(batch([1] * 8, [3000 + 17 * i for i in range(8)], bucketed=True))
    assert a["n_work"] == b["n_work"] and (a["work"] == b["work"]).all() and a["any_parts"] == b["any_parts"] == 1


def test_windows_bound_the_parts():
    plan = make_part(window=256).build_plan(batch([1], [5000]))
    w = rows_of(plan)
    assert len(w) == (256 // TA.KEY_TILE + 1) // TA.MIN_PART_TILES


def test_rows_of_partial_sums_fit_the_workspace():
    plan = make_part().build_plan(batch([16 * 9], [200000]))
    w = rows_of(plan)
    used = sum(int(r[3]) * 16 for r in w if r[2] == 0 and r[3] > 1)
    assert 0 < used <= TA.PARTIAL_ROWS


def test_the_other_form_gets_plain_tiles():
    plan = make_part(mma_q=0).build_plan(batch([20, 1], [20, 90]))
    assert plan["work"].reshape(-1, 2).tolist() == [[1, 0], [0, 16], [0, 8], [0, 0]] and plan["qt"] == 8


def test_blocks_of_positions_bound_the_keys_that_are_shared_out():
    """With blocks of 1,024 positions a single token at position 3,999 walks the 928 keys of its block (29 key tiles), and
    one at position 1,024 walks one key: the parts follow the block, not the sequence's length."""
    plan = make_part(chunk=1024).build_plan(batch([1, 1], [4000, 1025]))
    w = rows_of(plan)
    by_seq = {s: w[w[:, 0] == s] for s in range(2)}
    assert len(by_seq[0]) == by_seq[0][0, 3] == 29 // TA.MIN_PART_TILES
    assert len(by_seq[1]) == 1 and by_seq[1][0, 3] == 1
