"""Host-side logic of the copy-engine transport between stages (the transfers themselves need GPUs:
``tests/test_multigpu.py``)."""

from elf_b200.execution.channels import _CopyLink, _arena_layout


def _v_roles(n_ranks):
    """(producer, consumer) of every channel of a V placement, numbered as ``ChannelTable`` does."""
    placement = list(range(n_ranks)) + list(range(n_ranks - 1, -1, -1))
    roles, idx = {}, 0
    for a in range(len(placement) - 1):
        b = a + 1
        if placement[a] == placement[b]:
            continue
        roles[idx] = (placement[a], placement[b])
        roles[idx + 1] = (placement[b], placement[a])
        idx += 2
    return roles


def test_arena_layout_gives_every_end_a_region_of_its_own():
    depth = 4
    for n_ranks in (2, 4, 8):
        roles = _v_roles(n_ranks)
        sizes = [1000 + 300 * i if i % 5 else 0 for i in range(len(roles))]  # some channels never used
        offsets, total = _arena_layout(sizes, roles, n_ranks, depth)
        assert set(offsets) == {i for i, n in enumerate(sizes) if n}
        regions = {r: [] for r in range(n_ranks)}
        for idx, (at_producer, at_consumer, slot) in offsets.items():
            producer, consumer = roles[idx]
            assert slot >= sizes[idx] and slot % 256 == 0 and at_producer % 256 == 0 and at_consumer % 256 == 0
            regions[producer].append((at_producer, at_producer + _CopyLink.FLAG_BYTES))
            regions[consumer].append((at_consumer, at_consumer + depth * slot + _CopyLink.FLAG_BYTES))
        for rank, spans in regions.items():
            spans.sort()
            assert all(a[1] <= b[0] for a, b in zip(spans, spans[1:])), (rank, spans)
            assert not spans or spans[-1][1] <= total
        # the ring lives on the consuming rank only: the arena is far smaller than one ring per channel and rank
        assert total < sum(depth * ((n + 255) // 256 * 256) + 256 for n in sizes if n)


def test_arena_layout_without_traffic_is_empty():
    roles = _v_roles(2)
    assert _arena_layout([0] * len(roles), roles, 2, 4) == ({}, 0)
