"""Work distribution of the persistent forward attention kernel, restated in Python.

The kernel (``csrc/kernels/attention_sm100.cuh``: ``fwd_rank`` / ``fwd_item``) gives CTA ``c`` of ``G`` the items of
rank ``k * G + c`` (even ``k``) and ``(k + 1) * G - 1 - c`` (odd ``k``) of the heavy-first list, where rank ``w`` is query
tile ``n_qt - 1 - w // H`` of head ``w % H`` and costs ``qt + 1`` key tiles. The properties the kernel relies on are
checked here without a GPU: every item is taken exactly once, the ranks of a CTA increase (so the first rank past the
list ends its loop), and the key-tile counts of the CTAs are balanced."""
import pytest


def _rank(k: int, c: int, G: int) -> int:
    return (k + 1) * G - 1 - c if k & 1 else k * G + c


def _schedule(T: int, H: int, n_sm: int):
    n_qt = (T + 127) // 128
    n_items = n_qt * H
    G = min(n_items, n_sm)
    per_cta = []
    for c in range(G):
        ranks, k = [], 0
        while _rank(k, c, G) < n_items:
            ranks.append(_rank(k, c, G))
            k += 1
        per_cta.append(ranks)
    return n_qt, n_items, per_cta


@pytest.mark.parametrize("T,H", [(2048, 32), (1024, 8), (4096, 32), (300, 4), (2048, 16), (8192, 8), (128, 1)])
@pytest.mark.parametrize("n_sm", [148, 132])
def test_every_item_once_and_monotone(T, H, n_sm):
    n_qt, n_items, per_cta = _schedule(T, H, n_sm)
    seen = sorted(w for ranks in per_cta for w in ranks)
    assert seen == list(range(n_items))
    for ranks in per_cta:
        assert ranks == sorted(ranks) and len(set(ranks)) == len(ranks)
        assert len(ranks) >= 1


@pytest.mark.parametrize("T,H", [(2048, 32), (4096, 32), (8192, 8), (2048, 16)])
def test_key_tiles_are_balanced(T, H):
    n_qt, n_items, per_cta = _schedule(T, H, 148)
    tiles = [sum(n_qt - w // H for w in ranks) for ranks in per_cta]
    mean = sum(tiles) / len(tiles)
    # the boustrophedon over the heavy-first list keeps every CTA within one heavy item of the mean
    assert max(tiles) - mean <= n_qt
    assert max(tiles) <= 1.2 * mean


def test_stream_tiles_alternate_between_the_two_softmax_groups():
    """Group g owns the stream tiles t with t & 1 == g, across item boundaries: the group that does not own an item's
    last tile owns the first tile of the next item (which is what lets it defer its half of the epilogue past it)."""
    n_qt, n_items, per_cta = _schedule(2048, 32, 148)
    for ranks in per_cta[:8]:
        t = 0
        for i, w in enumerate(ranks):
            n_kv = n_qt - w // 32
            last_owner = (t + n_kv - 1) & 1
            t += n_kv
            if i + 1 < len(ranks):
                assert (t & 1) == (last_owner ^ 1)
