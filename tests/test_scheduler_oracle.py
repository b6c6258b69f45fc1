"""CPU tests of the scheduler oracle itself: hand-worked vectors traced through
csrc/smxx/get_mla_metadata.cu:25-88 and schedule invariants on random batches."""
import random

from oracle import scheduler


def test_hand_traced_vectors():
    # 8 requests x 64 blocks, 4 parts: total = 8*(64+5) = 552, payload = 138+5 = 143
    # -> each part takes exactly two whole requests (2*69 = 138 <= 143), nothing is split.
    md, ns = scheduler.get_mla_metadata_ref([4096] * 8, 4)
    assert md == [[0, 0, 1, 64, 0, 0, 0, 0], [2, 0, 3, 64, 0, 0, 0, 0], [4, 0, 5, 64, 0, 0, 0, 0], [6, 0, 7, 64, 0, 0, 0, 0]]
    assert ns == list(range(9))
    # one request of 16 blocks, 3 parts: total = 21, payload = 7+5 = 12 -> 7 blocks, 7 blocks, 2 blocks
    md, ns = scheduler.get_mla_metadata_ref([1024], 3)
    assert md == [[0, 0, 0, 7, 0, 0, 0, 0], [0, 7, 0, 14, 1, 0, 0, 0], [0, 14, 0, 16, 2, 0, 0, 0]]
    assert ns == [0, 3]
    # zero-length request counts as one block and ends at block 0
    md, ns = scheduler.get_mla_metadata_ref([0], 2)
    assert md[0] == [0, 0, 0, 0, 0, 0, 0, 0] and md[1][0] == 1 and ns == [0, 1]
    # sparse: every request is scheduled with topk tokens whatever its cache length
    md_a, ns_a = scheduler.get_mla_metadata_ref([7, 9000, 0], 5, topk=2048)
    md_b, ns_b = scheduler.get_mla_metadata_ref([2048] * 3, 5)
    assert md_a == md_b and ns_a == ns_b


def test_invariants_random():
    rng = random.Random(0)
    for _ in range(200):
        b = rng.randint(1, 40)
        lens = [rng.choice([0, 1, 63, 64, 65, rng.randint(1, 9000)]) for _ in range(b)]
        parts = rng.choice([1, 2, 7, 37, 74, 148])
        md, ns = scheduler.get_mla_metadata_ref(lens, parts)
        scheduler.check_schedule_invariants(md, ns, lens)
        assert ns[-1] <= b + parts


def test_cut_schedule_invariants_and_balance():
    """The schedule this library computes: valid for any batch, never needs more partial slots than the caller
    provides (batch + parts), and as balanced as the reference's greedy walk on the benchmark shapes."""
    rng = random.Random(1)
    for _ in range(300):
        b = rng.choice([1, 2, 3, 5, 8, 64, 128, 200])
        lens = [rng.choice([0, 1, 63, 64, 65, rng.randint(1, 9000), rng.randint(3072, 5120)]) for _ in range(b)]
        parts = rng.choice([1, 2, 7, 37, 74, 148])
        md, ns = scheduler.schedule_cut_ref(lens, parts)
        scheduler.check_schedule_invariants(md, ns, lens)
        assert ns[-1] <= b + parts
    lens = [rng.randint(3072, 5120) for _ in range(128)]
    for parts in (74, 37):
        ours = scheduler.max_part_cost(scheduler.schedule_cut_ref(lens, parts)[0], lens)
        theirs = scheduler.max_part_cost(scheduler.get_mla_metadata_ref(lens, parts)[0], lens)
        assert ours <= theirs + 1
    md, ns = scheduler.schedule_cut_ref([2048] * 64, 74, topk=2048)     # one request per part, nothing split
    assert ns[-1] == 64 and scheduler.max_part_cost(md, [2048] * 64, 2048) == 37
    md, ns = scheduler.schedule_cut_ref([1 << 20], 8)                    # one long context over 8 parts
    assert ns == [0, 8] and [row[4] for row in md] == list(range(8))


def test_num_sm_parts():
    assert scheduler.num_sm_parts_ref(148, 128, 1, 128, False) == 74
    assert scheduler.num_sm_parts_ref(148, 256, 1, 128, False) == 37
    assert scheduler.num_sm_parts_ref(148, 128, 1, 128, True) == 74
    assert scheduler.num_sm_parts_ref(148, 256, 1, 128, True) == 37
    assert scheduler.num_sm_parts_ref(132, 16, 1, 16, False) == 132
