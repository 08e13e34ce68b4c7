"""Writes tests/golden/select_kat.json: known-answer vectors for "keep the `cap` smallest
under a total order, duplicates included", re-encoding the input sequences of the reference's
DualHeap unit tests (diffcache_cpu/src/dualheap.rs:198,216,246,267,285) and its LCG regression
(dualheap.rs:173-187,305-338: seed 0xC0FFEE, 8 (d, cap) configurations x 300 pushes in
[-1000, 1000]).  The expected answer is the reference tests' own baseline: sort ascending,
truncate to cap (dualheap.rs:116-121).

Run from the repository root:  python tests/golden/make_select_kat.py
"""
import json
import os

MASK = (1 << 64) - 1


class Lcg:
    def __init__(self, seed):
        self.s = seed

    def next_u32(self):
        self.s = (self.s * 6364136223846793005 + 1) & MASK
        return self.s >> 32

    def next_i32_range(self, lo, hi):
        return lo + self.next_u32() % (hi - lo + 1)


def main():
    cases = []

    def add(name, seq, cap):
        cases.append({"name": name, "cap": cap, "values": list(seq), "expected": sorted(seq)[:cap]})

    add("len_less_than_d", [7, 3, 9, 1], 10)
    add("d_equals_cap_no_rest", [10, 9, 8, 7, 6, 100, 1], 5)
    add("cap_greater_than_d", [50, 40, 30, 20, 60, 10, 70, 25, 5, 100, 15], 6)
    add("duplicates_and_ties", [5, 5, 5, 5, 4, 4, 6, 6, 3, 3, 3, 7, 2, 2], 7)
    add("extend_and_from_iter", [9, 1, 8, 2, 7, 3, 6, 4, 5, 0, 10, -1], 10)
    add("kept_max_not_full", [3, 1, 4, 1, 5], 10)
    rng = Lcg(0xC0FFEE)
    for d, cap in [(1, 1), (1, 10), (3, 3), (3, 10), (10, 10), (10, 100), (100, 100), (100, 1000)]:
        seq = [rng.next_i32_range(-1000, 1000) for _ in range(300)]
        # every prefix is checked by the reference test; keep a few prefixes per configuration
        for n in (1, cap, min(300, cap + 1), 150, 300):
            add(f"lcg_d{d}_cap{cap}_n{n}", seq[:n], cap)
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "select_kat.json")
    with open(out, "w") as f:
        json.dump(cases, f)
    print(f"{len(cases)} cases -> {out}")


if __name__ == "__main__":
    main()
