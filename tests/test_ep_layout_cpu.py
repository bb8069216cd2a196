"""Offsets of an expert-parallel dispatch, checked on CPU against their Python restatement."""


def test_expert_parallel_layout_never_leaves_the_receive_buffer():
    """The offsets of an expert-parallel call, restated in Python: whatever the routing (balanced, or every token on
    one expert), nothing the owner indexes lies beyond its capacity, and the rows the owner counts as real are exactly
    the rows their senders did not drop."""
    import torch

    from art_b200.parallel.ep import reference_exchange_layout

    g = torch.Generator().manual_seed(0)
    for P, E, cap_tiles, skew in ((2, 8, 6, False), (2, 8, 3, True), (8, 128, 40, False), (8, 128, 12, True), (4, 16, 1, True)):
        El = E // P
        cnt = torch.randint(0, 60, (P, E), generator=g)
        if skew:
            cnt[:, 1] += 900                         # every source floods expert 1 (owner: rank 0)
            cnt[:, E - 1] = 0
        cap = cap_tiles * 128
        for owner in range(P):
            lay = reference_exchange_layout(cnt, owner, cap_tiles)
            seg, real, te = lay["seg_off"].tolist(), lay["real_rows"].tolist(), lay["tile_expert"].tolist()
            assert all(0 <= a <= b <= cap for a, b in zip(seg, seg[1:])) and seg[-1] % 128 == 0
            assert all(seg[j] + real[j] <= max(seg[j + 1], seg[j]) for j in range(El)), (seg, real)
            assert all(t == -1 or seg[t] <= i * 128 < seg[t + 1] for i, t in enumerate(te))
            kept = [0] * El                          # rows that senders store, from their own send_off
            for s in range(P):
                so = reference_exchange_layout(cnt, s, cap_tiles)["send_off"].tolist()
                for j in range(El):
                    e = owner * El + j
                    kept[j] += sum(1 for i in range(int(cnt[s, e])) if so[e] + i < cap)
                    # a source's rows sit where the owner expects them
                    if seg[j] < cap:
                        assert so[e] == seg[j] + int(lay["src_start"][j, s])
            assert kept == real, (P, E, cap_tiles, skew, owner, kept, real)


def test_worst_case_capacity_drops_nothing_whatever_the_routing():
    """``capacity_factor=None`` sizes an owner's receive buffer for every rank sending all its rows there: with that
    many tiles the layout keeps every row even when the router puts all tokens on one expert."""
    import torch

    from art_b200.parallel.ep import reference_exchange_layout

    for P, E, rows_per_rank in ((2, 8, 500), (8, 128, 1000), (4, 16, 128)):
        El = E // P
        cap_tiles = (P * rows_per_rank + El * 127 + 127) // 128          # what ExpertParallel allocates for None
        for pattern in ("one-expert", "one-owner", "uneven"):
            cnt = torch.zeros(P, E, dtype=torch.long)
            if pattern == "one-expert":
                cnt[:, 3] = rows_per_rank
            elif pattern == "one-owner":
                cnt[:, :El] = rows_per_rank // El
                cnt[:, 0] += rows_per_rank - (rows_per_rank // El) * El
            else:
                g = torch.Generator().manual_seed(P)
                w = torch.rand(P, E, generator=g) ** 8
                cnt = (w / w.sum(1, keepdim=True) * rows_per_rank).long()
            for owner in range(P):
                lay = reference_exchange_layout(cnt, owner, cap_tiles)
                want = [int(cnt[:, owner * El + j].sum()) for j in range(El)]
                assert lay["real_rows"].tolist() == want, (P, E, pattern, owner)
