"""Host model of the decode kernel's work schedule (csrc/skinny.cu: the unit ranges, SegIter's walk order
and the split-tile hand-over), checked for the properties the kernel relies on.

The (row tile, k group) units of a layer are dealt out to the CTAs of the persistent grid as equal contiguous
ranges. A tile whose k range is shared by several CTAs is added up by the CTA that owns its first unit; every
other piece is only published. The owner waits for the published pieces, so the schedule must never let a CTA
wait before it has published everything somebody else may be waiting for - otherwise two CTAs could wait for
each other. The shapes are the benchmark's layers and a few ragged ones; the grid is 148 CTAs and smaller."""
import pytest

SHAPES = [(34816, 5120), (5120, 17408), (16384, 5120), (5120, 8192), (8192, 5120), (5120, 6144), (17408, 5120),
          (248320, 5120), (1040, 640), (128, 128), (208, 1024), (31040, 5120)]


def ranges(tiles, G, grid):
    U = tiles * G
    return [U * b // grid for b in range(grid + 1)]


def walk(u0, u1, G, tail_last):
    """Segments (tile, g0, L, kind) of one CTA in processing order; kind is 'head', 'tail' or 'whole'."""
    t_first, t_last = u0 // G, (u1 - 1) // G
    head_g0, tail_g1 = u0 - t_first * G, u1 - t_last * G
    single = t_first == t_last
    head_partial = (not (head_g0 == 0 and tail_g1 == G)) if single else head_g0 != 0
    tail_partial = False if single else tail_g1 != G
    segs = []
    if head_partial:
        segs.append((t_first, head_g0, (tail_g1 if single else G) - head_g0, "head"))
    tail = (t_last, 0, tail_g1, "tail")
    if tail_partial and not tail_last:
        segs.append(tail)
    for t in range(t_first, t_last + 1):
        if (t == t_first and head_partial) or (t == t_last and tail_partial):
            continue
        segs.append((t, 0, G, "whole"))
    if tail_partial and tail_last:
        segs.append(tail)
    return segs


@pytest.mark.parametrize("N,K", SHAPES)
@pytest.mark.parametrize("grid_max", [148, 132, 7])
@pytest.mark.parametrize("tail_last", [False, True])
def test_every_unit_once_and_no_wait_before_publishing(N, K, grid_max, tail_last):
    tiles, G = (N + 127) // 128, K // 128
    U = tiles * G
    grid = min(U, grid_max)
    us = ranges(tiles, G, grid)
    covered = [0] * U
    pieces = {}  # tile -> list of (cta, position of the piece in the CTA's walk, segments in that walk)
    for b in range(grid):
        segs = walk(us[b], us[b + 1], G, tail_last)
        assert sum(L for _, _, L, _ in segs) == us[b + 1] - us[b]
        assert sum(1 for s in segs if s[3] != "whole") <= 2, "a unit range has at most two split pieces"
        for pos, (t, g0, L, kind) in enumerate(segs):
            for g in range(g0, g0 + L):
                covered[t * G + g] += 1
            if kind != "whole":
                pieces.setdefault(t, []).append((b, pos, len(segs), kind))
    assert all(c == 1 for c in covered), "every (tile, group) unit is multiplied exactly once"
    for t, ps in pieces.items():
        ctas = [b for b, _, _, _ in ps]
        assert ctas == list(range(ctas[0], ctas[-1] + 1)) and len(ps) >= 2, "a split tile's pieces: consecutive CTAs"
        owner = ps[0]
        assert us[owner[0]] <= t * G < us[owner[0] + 1], "the CTA that adds up owns the tile's first unit"
        # the owner's piece is the last segment of its walk, whole tiles aside
        b, pos, n, kind = owner
        later = walk(us[b], us[b + 1], G, tail_last)[pos + 1:]
        assert all(s[3] == "whole" for s in later)
        if tail_last:
            assert pos == n - 1, "with tail_last nothing follows the piece whose owner has to wait"
        # every piece the owner waits for is published before its CTA can come to wait for anything:
        # it is the first segment of that CTA's walk
        for b2, pos2, _, _ in ps[1:]:
            assert pos2 == 0, (t, b2, pos2)


def test_helper_mailbox_is_used_at_most_once_per_cta():
    """M = 1 without the fused argmax (tail_last = False): the waiting goes to the helper warp only for the piece
    at the end of a range that has whole tiles after it, i.e. at most one mailbox entry per lane quarter."""
    for N, K in SHAPES:
        tiles, G = (N + 127) // 128, K // 128
        grid = min(tiles * G, 148)
        us = ranges(tiles, G, grid)
        for b in range(grid):
            segs = walk(us[b], us[b + 1], G, False)
            handed = [i for i, s in enumerate(segs) if s[3] == "tail" and i < len(segs) - 1]
            assert len(handed) <= 1
