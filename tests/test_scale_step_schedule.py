"""The feeder warps of the block-scaled expert GEMM (csrc/kernels/expert_gemm.cu) write one scale
group (four K blocks) in four steps spread over the stages of the group before.  This is a host-side
model of that schedule, checked for every K extent: groups come out in order, each is published
before the first of its stages is fed, every group's scales were fetched at least one stage before
they are packed (except the tile's first two), and a store never needs a slot of the four-slot
ring that the MMA warp cannot have released yet given the four-stage operand ring."""

import pytest

STAGES = 4          # operand ring
SLOTS = 4           # scale-slot ring


def schedule(num_kb):
    """(stage index, action, group) in the order a feeder warp executes them within one tile."""
    out = [(-1, "fetch", 0)]

    def pack_cols(kb, g):
        out.append((kb, "pack_cols", g))
        if 4 * g + 4 < num_kb:
            out.append((kb, "fetch", g + 1))

    for kb in range(num_kb):
        out.append((kb, "copies", kb))
        g, step, nxt = kb >> 2, kb & 3, 4 * (kb >> 2) + 4
        if kb == 0:
            out.append((kb, "pack_rows", 0))
            pack_cols(kb, 0)
            out += [(kb, "store", 0), (kb, "publish", 0)]
        elif nxt < num_kb:
            if step == 0:
                out.append((kb, "pack_rows", g + 1))
            if step == 1:
                if g == 0:
                    out.append((kb, "pack_rows", g + 1))
                pack_cols(kb, g + 1)
            if step == 2:
                out.append((kb, "store", g + 1))
            if step == 3:
                out.append((kb, "publish", g + 1))
    return out


@pytest.mark.parametrize("num_kb", list(range(1, 70)) + [112, 113, 127, 128])
def test_schedule_invariants(num_kb):
    groups = (num_kb + 3) // 4
    events = schedule(num_kb)
    at = {}
    for order, (kb, action, g) in enumerate(events):
        if action != "copies":
            assert (action, g) not in at, "every step once per group"
            at[(action, g)] = (kb, order)
    for g in range(groups):
        for action in ("fetch", "pack_rows", "pack_cols", "store", "publish"):
            assert (action, g) in at, (action, g)
        order = [at[(a, g)][1] for a in ("fetch", "pack_rows", "pack_cols", "store", "publish")]
        assert order == sorted(order), "fetch -> pack -> store -> publish"
        if g + 1 < groups:      # one set of registers: the next fetch must follow both packs of this group
            assert at[("fetch", g + 1)][1] > at[("pack_cols", g)][1]
        if g >= 1:
            # published before the copies of the group's first stage go out, so the MMAs never wait for it
            first_copy = next(i for i, ev in enumerate(events) if ev == (4 * g, "copies", 4 * g))
            assert at[("publish", g)][1] < first_copy
        if g >= 2:
            assert at[("pack_rows", g)][0] - at[("fetch", g)][0] >= 3, "the loads have three stages to land"
        # The feeder is about to wait for stage kb + 1's buffer when it stores at stage kb; having fed
        # stage kb means the MMA warp released stage kb - STAGES, i.e. finished every group up to
        # (kb - STAGES - 3) // 4.  The slot of group g was last used by group g - SLOTS.
        kb = at[("store", g)][0]
        if g >= SLOTS:
            assert (kb - STAGES - 3) // 4 >= g - SLOTS, "the slot has been released without the feeder's help"
    assert ("fetch", groups) not in at and ("publish", groups) not in at
