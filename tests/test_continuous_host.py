"""The continuous-batching scheduler on the CPU: admission in arrival order, block accounting,
teacher forcing inside a prompt, completion by length and by end-of-sequence token."""
import pytest

from tilemega_b200.serving.continuous import BlockPool, Request, SlotScheduler


def test_block_pool_keeps_the_scratch_block_and_recycles():
    pool = BlockPool(6)
    first = pool.take(3)
    assert first == [1, 2, 3] and pool.take(3) is None      # block 0 is never handed out
    pool.give_back(first)
    assert sorted(pool.take(5)) == [1, 2, 3, 4, 5]
    with pytest.raises(ValueError):
        BlockPool(1)


def test_requests_join_and_leave_between_steps():
    scheduler = SlotScheduler(slots=2, num_blocks=8, max_blocks_per_sequence=4)
    a, b, c = Request(0, [5, 6, 7], 2), Request(1, [9], 3, eos=42), Request(2, [1, 2], 40)
    for request in (a, b, c):
        scheduler.submit(request)
    assert scheduler.admit() == [0, 1] and scheduler.admit() == []      # two slots: c waits
    assert scheduler.forced_token(0) == 6 and scheduler.forced_token(1) is None
    assert scheduler.advance({0: 100, 1: 200}) == []                     # a is inside its prompt: 100 is discarded
    assert a.generated == [] and b.generated == [200]
    assert scheduler.forced_token(0) == 7
    assert scheduler.advance({0: 101, 1: 42}) == [b]                     # b meets its end-of-sequence token
    assert b.generated == [200, 42] and scheduler.active() == [0]
    assert scheduler.admit() == [1]                                      # c takes b's slot (it needs 3 blocks: 2 + 40 + 1 tokens)
    assert scheduler.slots[1].position == 0 and len(scheduler.slots[1].blocks) == 3
    assert scheduler.forced_token(0) is None
    assert scheduler.advance({0: 300, 1: 7}) == [] and a.generated == [300] and c.generated == []
    assert scheduler.advance({0: 301, 1: 8}) == [a] and a.generated == [300, 301] and c.generated == [8]
    assert not scheduler.idle()
    # the pool is whole again once everything has ended
    while not scheduler.idle():
        scheduler.advance({index: 1 for index in scheduler.active()})
    assert len(scheduler.pool.free) == 7


def test_admission_waits_for_blocks_in_arrival_order():
    scheduler = SlotScheduler(slots=3, num_blocks=5, max_blocks_per_sequence=4)
    big, small = Request(0, [1] * 20, 30), Request(1, [1], 2)        # 4 blocks, 1 block
    other = Request(2, [1] * 10, 10)                                  # 2 blocks
    for request in (other, big, small):
        scheduler.submit(request)
    assert scheduler.admit() == [0]              # `other` fits; `big` needs 4 of the 2 blocks left, and `small` does not overtake it
    with pytest.raises(ValueError):
        scheduler.submit(Request(3, [1] * 60, 10))   # longer than a sequence's share of the table
    with pytest.raises(ValueError):
        scheduler.submit(Request(4, [], 3))


def test_prefilled_slot_starts_behind_its_prompt():
    from tilemega_b200.serving.prefill import pack_rows
    scheduler = SlotScheduler(slots=1, num_blocks=8, max_blocks_per_sequence=4)
    scheduler.submit(Request(0, [5, 6, 7, 8], 2))
    scheduler.submit(Request(1, [9], 1))
    assert scheduler.admit() == [0]
    assert scheduler.prefilled(0, 42) is None
    assert scheduler.slots[0].position == 4 and scheduler.forced_token(0) is None
    ended = scheduler.advance({0: 43})
    assert [r.generated for r in ended] == [[42, 43]]
    assert scheduler.admit() == [0]
    done = scheduler.prefilled(0, 11)                 # one new token: the prefill's sample ends the request
    assert done is not None and done.generated == [11] and scheduler.idle()
    assert len(scheduler.pool.free) == 7
    # rows are packed sequence after sequence, positions ascending, chunks of at most `rows`
    chunks = pack_rows([3, 1, 4], rows=4)
    assert chunks == [[(0, 0), (0, 1), (0, 2), (1, 0)], [(2, 0), (2, 1), (2, 2), (2, 3)]]
