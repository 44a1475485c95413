"""CPU: a small model of the tensor-parallel exchange protocol (csrc/fsvd_exchange.h) under random
schedules.  Every rank runs push(1), reduce(1), push(2), reduce(2), ... in order; a push is N
independent deliveries (data, then flag, per destination) that the schedule may delay at will; a
reduce waits for the N flags of its own region and then reads the N slots.  The claim under test:
with slots and flags doubled by the parity of the exchange number, a reduce never reads a slot that
a later exchange has already overwritten — and with a single buffer it does."""
import random


def run(world: int, exchanges: int, parities: int, seed: int) -> bool:
    """True when every reduce read exactly the partial sums of its own exchange."""
    rng = random.Random(seed)
    # region[dst][parity][src] = (number of the exchange whose data the slot holds, flag value)
    data = [[[0] * world for _ in range(parities)] for _ in range(world)]
    flag = [[[0] * world for _ in range(parities)] for _ in range(world)]
    step = [0] * world            # per rank: 2 (k - 1) = about to push k, 2 (k - 1) + 1 = about to reduce k
    inflight = []                 # deliveries issued and not yet performed: (src, dst, k, what)
    ok = True
    while min(step) < 2 * exchanges:
        moves = [("deliver", i) for i in range(len(inflight))]
        for r in range(world):
            if step[r] >= 2 * exchanges:
                continue
            k = step[r] // 2 + 1
            if step[r] % 2 == 0:
                moves.append(("push", r))
            elif all(flag[r][k % parities][q] >= k for q in range(world)):
                moves.append(("reduce", r))
        kind, arg = rng.choice(moves)
        if kind == "deliver":
            src, dst, k, what = inflight.pop(arg)
            if what == "data":
                data[dst][k % parities][src] = k
                inflight.append((src, dst, k, "flag"))      # the flag of a destination follows its data
            else:
                flag[dst][k % parities][src] = k
        elif kind == "push":
            k = step[arg] // 2 + 1
            inflight.extend((arg, dst, k, "data") for dst in range(world))
            step[arg] += 1
        else:
            k = step[arg] // 2 + 1
            ok = ok and all(data[arg][k % parities][q] == k for q in range(world))
            step[arg] += 1
    return ok


def test_two_parities_are_enough_under_any_schedule():
    for world in (2, 3, 8):
        for seed in range(40):
            assert run(world, exchanges=7, parities=2, seed=seed), (world, seed)


def test_a_single_buffer_is_overwritten_too_early():
    assert not all(run(3, exchanges=7, parities=1, seed=seed) for seed in range(40))
