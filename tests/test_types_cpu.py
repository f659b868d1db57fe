"""`nx_b200.types` against the doctests of nx/lib/nx/type.ex (merge :397-447, merge_number :498-533,
to_floating :241-248, to_aggregate :315-324, infer :165-168) and an exhaustive check of `merge` against the
rule of type.ex:463-492."""
import itertools

import pytest

from nx_b200 import types as T


MERGE = [(("s", 8), ("s", 8), ("s", 8)), (("s", 8), ("s", 64), ("s", 64)),
         (("s", 8), ("u", 8), ("s", 16)), (("s", 16), ("u", 8), ("s", 16)), (("s", 8), ("u", 16), ("s", 32)),
         (("s", 32), ("u", 8), ("s", 32)), (("s", 8), ("u", 32), ("s", 64)), (("s", 64), ("u", 8), ("s", 64)),
         (("s", 8), ("u", 64), ("s", 64)),
         (("u", 8), ("f", 32), ("f", 32)), (("u", 64), ("f", 32), ("f", 32)), (("s", 8), ("f", 32), ("f", 32)),
         (("s", 64), ("f", 32), ("f", 32)),
         (("u", 8), ("f", 64), ("f", 64)), (("u", 64), ("f", 64), ("f", 64)), (("s", 8), ("f", 64), ("f", 64)),
         (("s", 64), ("f", 64), ("f", 64)),
         (("u", 8), ("bf", 16), ("bf", 16)), (("u", 64), ("bf", 16), ("bf", 16)), (("s", 8), ("bf", 16), ("bf", 16)),
         (("s", 64), ("bf", 16), ("bf", 16)),
         (("f", 32), ("bf", 16), ("f", 32)), (("f", 64), ("bf", 16), ("f", 64))]

MERGE_NUMBER = [(("u", 8), 0, ("u", 8)), (("u", 8), 255, ("u", 8)), (("u", 8), 256, ("u", 16)), (("u", 8), -1, ("s", 16)),
                (("u", 8), -32767, ("s", 16)), (("u", 8), -32768, ("s", 16)), (("u", 8), -32769, ("s", 32)),
                (("s", 8), 0, ("s", 8)), (("s", 8), 127, ("s", 8)), (("s", 8), -128, ("s", 8)), (("s", 8), 128, ("s", 16)),
                (("s", 8), -129, ("s", 16)), (("s", 8), 1.0, ("f", 32)), (("u", 64), -1337, ("s", 64)),
                (("f", 32), 1, ("f", 32)), (("f", 32), 1.0, ("f", 32)), (("f", 64), 1.0, ("f", 64))]


@pytest.mark.parametrize("a,b,want", MERGE)
def test_merge_doctests(a, b, want):
    assert T.merge(a, b) == want
    assert T.merge(b, a) == want


@pytest.mark.parametrize("type,number,want", MERGE_NUMBER)
def test_merge_number_doctests(type, number, want):
    assert T.merge_number(type, number) == want


def test_merge_follows_the_rule_for_every_pair():
    rank = {"u": 0, "s": 1, "bf": 2, "f": 3}
    every = [("u", b) for b in (8, 16, 32, 64)] + [("s", b) for b in (8, 16, 32, 64)] + [("bf", 16), ("f", 16), ("f", 32), ("f", 64)]
    for a, b in itertools.product(every, every):
        if a[0] == b[0]:
            want = (a[0], max(a[1], b[1]))
        else:
            lo, hi = sorted((a, b), key=lambda x: rank[x[0]])
            want = ("s", max(min(lo[1] * 2, 64), hi[1])) if (lo[0], hi[0]) == ("u", "s") else hi
        assert T.merge(a, b) == want, (a, b)


def test_conversions_and_inference():
    assert [T.to_floating(x) for x in (("s", 8), ("s", 32), ("bf", 16), ("f", 32))] == [("f", 32), ("f", 32), ("bf", 16), ("f", 32)]
    assert [T.to_aggregate(x) for x in (("s", 8), ("u", 16), ("s", 64), ("bf", 16), ("f", 32), ("u", 64))] == \
        [("s", 32), ("u", 32), ("s", 64), ("bf", 16), ("f", 32), ("s", 64)]
    assert T.infer(1) == ("s", 32) and T.infer(1.0) == ("f", 32)
    assert T.normalize("bf16") == ("bf", 16) and T.short(("u", 8)) == "u8" and T.itemsize(("f", 64)) == 8
    assert T.min_value(("s", 8)) == -128 and T.max_value(("u", 16)) == 65535
