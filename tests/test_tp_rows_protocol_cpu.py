"""The exchange protocol of the tensor-parallel row kernels (csrc/norm_mix.cu: tp_rows_push / tp_rows_sum), restated
in NumPy and run under random interleavings of P simulated ranks - no GPU, no process group.

What the kernels rely on, and what is checked here for every interleaving:
  * wire format: a row of D fp16 values travels as D/2 units of 8 bytes {4 bytes of payload, call number}; vector v
    (8 values) of the row occupies units 4v .. 4v+3; a unit is written whole (8-byte atomicity), never half;
  * a reader accepts a unit only when its tag equals the call number, so it can never take an older call's payload;
  * two inbox buffers alternate by call number; a rank starts call e+1 only when it has finished call e (received every
    peer's rows) - therefore a writer of call e+2 never lands on a unit of call e that its owner has not read yet;
  * the sum runs in rank order in fp32 and is rounded to fp16: every rank holds the same bits, equal to the
    stand-alone all-reduce kernel's result (oracle: the same arithmetic written once more, vectorised).
"""
import numpy as np
import pytest


def tag_of(call: int) -> int:
    return call if call else 1  # never 0: fresh memory is zero


class Rank:
    """One rank's view: its inbox [2 buffers][P slots][rows * D/2 units][2 words] and its call counter."""

    def __init__(self, rank, world, rows, D):
        self.rank, self.world, self.rows, self.D = rank, world, rows, D
        self.units = rows * D // 2
        self.inbox = np.zeros((2, world, self.units, 2), dtype=np.uint32)
        self.unread = np.zeros((2, world, self.units), dtype=bool)  # written for a call, not yet consumed by its owner
        self.calls_done = 0
        self.result = None


def payload_words(partial):
    """[rows, D] fp16 -> [rows * D/2] uint32 payload words in memory order."""
    return np.ascontiguousarray(partial).view(np.uint32).reshape(-1)


def push_unit(dst: Rank, src_rank, call, unit, word):
    buf = call & 1
    # landing on a unit whose previous payload the owner has not consumed would lose data
    assert not dst.unread[buf, src_rank, unit], "a writer overtook the reader of the same buffer"
    dst.inbox[buf, src_rank, unit] = (word, tag_of(call))  # one aligned 8-byte store: payload and tag together
    dst.unread[buf, src_rank, unit] = True


def try_sum(me: Rank, call, partial):
    """The reader's side for the whole tensor: None while any unit of any peer lacks the tag, else the rounded sum."""
    buf = call & 1
    acc = np.zeros(me.units * 2, dtype=np.float32)
    for s in range(me.world):  # rank order
        if s == me.rank:
            words = payload_words(partial)
        else:
            box = me.inbox[buf, s]
            if not np.all(box[:, 1] == tag_of(call)):
                return None
            words = box[:, 0].copy()
        acc = acc + words.view(np.float16).astype(np.float32)
    for s in range(me.world):
        if s != me.rank:
            me.unread[buf, s, :] = False
    return acc.astype(np.float16).reshape(me.rows, me.D)


def oracle_sum(partials):
    acc = np.zeros(partials[0].shape, dtype=np.float32)
    for p in partials:  # rank order
        acc = acc + p.astype(np.float32)
    return acc.astype(np.float16)


@pytest.mark.parametrize("world,rows,D,calls,seed", [(2, 3, 16, 7, 0), (3, 2, 16, 6, 1), (4, 1, 32, 5, 2), (8, 1, 8, 4, 3)])
def test_rows_exchange_under_random_interleavings(world, rows, D, calls, seed):
    rng = np.random.default_rng(seed)
    data = [[rng.standard_normal((rows, D)).astype(np.float16) for _ in range(world)] for _ in range(calls + 1)]
    for trial in range(20):
        ranks = [Rank(r, world, rows, D) for r in range(world)]
        # per rank: the list of its pending unit stores for the current call (shuffled: stores of a kernel land in any
        # order), and whether it has pushed already
        pending = [None] * world
        results = [[] for _ in range(world)]
        while any(r.calls_done < calls for r in ranks):
            r = ranks[int(rng.integers(world))]
            if r.calls_done >= calls:
                continue
            call = r.calls_done + 1
            part = data[call][r.rank]
            if pending[r.rank] is None:  # the kernel of this call starts: queue its stores to every peer
                words = payload_words(part)
                stores = [(p, u) for p in range(world) if p != r.rank for u in range(r.units)]
                rng.shuffle(stores)
                pending[r.rank] = (call, words, stores)
            c, words, stores = pending[r.rank]
            if stores:  # let a random number of this rank's stores land
                n = int(rng.integers(1, len(stores) + 1))
                for p, u in stores[:n]:
                    push_unit(ranks[p], r.rank, c, u, words[u])
                del stores[:n]
                continue
            got = try_sum(r, call, part)  # all pushed: poll
            if got is not None:
                results[r.rank].append(got)
                r.calls_done = call
                pending[r.rank] = None
        for call in range(1, calls + 1):
            want = oracle_sum(data[call])
            for r in range(world):
                assert np.array_equal(results[r][call - 1].view(np.uint16), want.view(np.uint16))


def test_stale_tag_is_never_accepted():
    """Buffer reuse: call 3 polls the buffer that still holds call 1's units; it must wait until EVERY unit carries 3."""
    me, peer_part = Rank(0, 2, 1, 16), np.arange(16, dtype=np.float16).reshape(1, 16)
    mine = np.ones((1, 16), dtype=np.float16)
    for u, w in enumerate(payload_words(peer_part)):
        push_unit(me, 1, 1, u, w)
    assert try_sum(me, 1, mine) is not None
    assert try_sum(me, 3, mine) is None  # same buffer, old tags
    words = payload_words(peer_part * 2)
    for u in range(me.units - 1):
        push_unit(me, 1, 3, u, words[u])
    assert try_sum(me, 3, mine) is None  # one unit still shows call 1
    push_unit(me, 1, 3, me.units - 1, words[-1])
    got = try_sum(me, 3, mine)
    assert np.array_equal(got, (peer_part * 2 + 1).astype(np.float16))


def test_first_call_numbers_use_distinct_tags_and_buffers():
    assert tag_of(0) == 1 and tag_of(1) == 1 and (0 & 1) != (1 & 1)  # the wrapped call 0 shares its tag with call 1, not its buffer
    assert all(tag_of(c) == c for c in (2, 3, 2**32 - 1))
