"""A host-side model of the peer exchange's handshake (csrc/hkv_basic.cuh: store_partial,
hkv_merge_published_kernel), run under random interleavings of the ranks.

Per exchange every rank, in stream order:
    publish   write its partial into parity (epoch & 1) of its own mailbox
    release   store epoch + 1 into the flag word it owns in every rank's mailbox
    wait      until every flag word in its OWN mailbox has reached epoch + 1
    read      every rank's partial of parity (epoch & 1), straight from that rank's mailbox
    close     epoch += 1
The model checks what the two-parity mailbox relies on: a rank may be one exchange ahead of a
peer that is still reading, never two, so no partial is overwritten before every reader is done
with it; and a reader never sees a partial of another epoch. A mailbox with ONE parity must fail
the same check (the model is able to see the hazard)."""
import random

import pytest


class Rank:
    def __init__(self, rank, world, parities):
        self.rank, self.world, self.parities = rank, world, parities
        self.epoch = 0
        self.flags = [0] * world            # flag words in THIS rank's mailbox, written by the peers
        self.partial = [None] * parities    # (writer, epoch) per parity
        self.phase = 0                      # 0 publish, 1 release, 2 wait, 3.. read rank (phase - 3), then close
        self.steps_done = 0


def run(world, steps, parities, seed):
    rng = random.Random(seed)
    ranks = [Rank(r, world, parities) for r in range(world)]
    hazards = 0
    while any(r.steps_done < steps for r in ranks):
        movable = [r for r in ranks if r.steps_done < steps and not (r.phase == 2 and min(r.flags) < r.epoch + 1)]
        assert movable, "the handshake deadlocked"
        me = rng.choice(movable)
        e = me.epoch
        if me.phase == 0:
            me.partial[e % parities] = (me.rank, e)
            me.phase = 1
        elif me.phase == 1:
            for peer in ranks:
                peer.flags[me.rank] = e + 1
            me.phase = 2
        elif me.phase == 2:
            me.phase = 3
        elif me.phase < 3 + world:
            src = ranks[me.phase - 3]
            if src.partial[e % parities] != (src.rank, e):
                hazards += 1                 # the partial of this epoch is not (or no longer) there
            me.phase += 1
        else:
            me.epoch += 1
            me.steps_done += 1
            me.phase = 0
    return hazards, [r.epoch for r in ranks]


@pytest.mark.parametrize("world", [2, 3, 8])
def test_two_parities_are_enough_under_any_interleaving(world):
    for seed in range(200):
        hazards, epochs = run(world, steps=6, parities=2, seed=seed)
        assert hazards == 0, f"seed {seed}: a reader saw a partial of another epoch"
        assert epochs == [6] * world


def test_one_parity_is_not_and_the_model_sees_it():
    assert sum(run(4, steps=6, parities=1, seed=s)[0] for s in range(200)) > 0
