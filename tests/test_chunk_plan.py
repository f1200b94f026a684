"""How a step cuts an arena into pieces (host logic, no GPU): the pieces tile the
arena exactly and every boundary keeps the shards on 512-value boundaries."""
import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from nntrain_b200.reducers import chunk_spans


def check(elements, world, spans, longest):
    assert spans[0][0] == 0 and spans[-1][1] == elements
    for (a, b), (c, d) in zip(spans, spans[1:]):
        assert b == c and a < b
    assert all(a % (512 * world) == 0 for a, _ in spans)
    assert longest == max(b - a for a, b in spans)


@settings(max_examples=200, deadline=None)
@given(st.integers(1, 1 << 31), st.integers(1, 8), st.one_of(st.none(), st.integers(1, 1 << 29)))
def test_equal_pieces_tile_the_arena(elements, world, chunk):
    spans, longest = chunk_spans(elements, world, chunk, None)
    check(elements, world, spans, longest)
    if chunk is None or chunk >= elements:
        assert len(spans) == (1 if (world == 1 or elements < (64 << 20)) else len(spans))


@settings(max_examples=200, deadline=None)
@given(st.integers(1, 1 << 31), st.integers(1, 8), st.lists(st.integers(0, 1 << 29), min_size=1, max_size=9))
def test_an_explicit_plan_tiles_the_arena(elements, world, plan):
    spans, longest = chunk_spans(elements, world, None, plan)
    check(elements, world, spans, longest)


@pytest.mark.parametrize("world", (2, 4, 8))
def test_default_plan_of_the_large_arena(world):
    elements = 1_543_714_304
    spans, longest = chunk_spans(elements, world)
    check(elements, world, spans, longest)
    assert len(spans) == 7
    lengths = [b - a for a, b in spans]
    assert lengths[0] < lengths[1] < lengths[2] and lengths[-1] < lengths[-2] < lengths[-3]
    assert chunk_spans(elements, 1) == ([(0, elements)], elements)        # one rank: one piece
    assert chunk_spans(1 << 20, world) == ([(0, 1 << 20)], 1 << 20)       # small arenas: one piece
