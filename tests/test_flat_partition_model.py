"""Host-side model of the flat tile partition of the decode attention kernel (csrc/attn/decode_paged.cu,
``decode_attn_flat_kernel``): the index arithmetic restated in Python and checked for random lengths and grid sizes.

The kernel deals all KV tiles of a step (ordered sequence, item = KV head x group slice, tile) out in equal ranges, one per
CTA; an item cut by a range boundary leaves partials in slot 1 of the CTA it starts in and slot 0 of the following CTAs,
and the merge kernel's CTA p combines the item that starts in attention CTA p.  Checked here: every tile is streamed exactly
once, ranges differ by at most the rounding of one division, a CTA never needs more than its two partial slots, and the
merge reads exactly the slots that were written, once each."""
import random


def partition(lens, items_per_seq, num_ctas, tile, min_tiles):
    n = [(l + tile - 1) // tile for l in lens]
    cum = [0]
    for x in n:
        cum.append(cum[-1] + x)
    total = items_per_seq * cum[-1]
    per_cta = max((total + num_ctas - 1) // num_ctas, min_tiles)

    def locate(f):                                   # flat_locate
        lo, hi = 0, len(lens)
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if items_per_seq * cum[mid] <= f:
                lo = mid
            else:
                hi = mid
        r = f - items_per_seq * cum[lo]
        return lo, r // n[lo], r % n[lo]

    streamed, written, direct, metas = [], {}, set(), {}
    for p in range(num_ctas):
        f0, f1 = p * per_cta, min((p + 1) * per_cta, total)
        if f0 >= f1:
            continue
        b, h, t = locate(f0)
        f = f0
        while f < f1:
            seg = min(n[b] - t, f1 - f)
            streamed += [(b, h, t + i) for i in range(seg)]
            starts_here, whole = t == 0, t == 0 and seg == n[b]
            if whole:
                assert (b, h) not in direct
                direct.add((b, h))
            else:
                slot = (p, 1 if starts_here else 0)
                assert slot not in written, "a CTA needs more than its two partial slots"
                written[slot] = (b, h)
                if starts_here:
                    item_end = f + n[b]
                    metas[p] = ((b, h), (item_end - 1) // per_cta - p + 1)
            f += seg
            t = 0                                    # flat_next_item
            h += 1
            if h == items_per_seq:
                h = 0
                b += 1
                while b < len(lens) and n[b] == 0:
                    b += 1
    return n, per_cta, streamed, written, direct, metas


def test_flat_partition_covers_every_tile_once_and_merge_slots_match():
    rng = random.Random(0)
    for trial in range(300):
        B = rng.randint(1, 40)
        lens = [rng.choice([0, 0, 1, 2, 63, 64, 65, rng.randint(1, 3000)]) for _ in range(B)]
        if not any(lens):
            lens[rng.randrange(B)] = 5
        items_per_seq = rng.choice([1, 2, 8, 16])
        num_ctas = rng.choice([1, 3, 16, 148, 296])
        tile = rng.choice([16, 32, 64])
        n, per_cta, streamed, written, direct, metas = partition(lens, items_per_seq, num_ctas, tile, rng.choice([1, 2, 4]))
        want = [(b, h, t) for b in range(B) for h in range(items_per_seq) for t in range(n[b])]
        assert streamed == want                                      # every tile once, in order
        read = set()
        for first, (item, parts) in metas.items():                   # what the merge kernel reads
            assert parts >= 2
            for k in range(parts):
                slot = (first + k, 1 if k == 0 else 0)
                assert written.get(slot) == item, (trial, slot, item)
                assert slot not in read
                read.add(slot)
        assert read == set(written)                                  # nothing written that nobody merges
        items = {(b, h) for b in range(B) for h in range(items_per_seq) if n[b] > 0}
        assert direct | {v for v in written.values()} == items and not (direct & set(written.values()))
