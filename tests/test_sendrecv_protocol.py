"""The SendRecv flag protocol (comm.message_words) on a CPU model of eight ranks in a 4 x 2 double ring.

Each rank is a thread that walks the message sequence of the emitted double-ring program (inner hops,
one outer hop, inner hops), using the words and values message_words() names; memory is a dict of
int words with plain last-writer-wins stores, waits spin until a word reaches the value.  One inner
ring is held back by two steps while the other group runs ahead, which is the situation in which a
flag word shared by two writers breaks: the outer neighbour's grant for message 3 lands before the
inner neighbour's grant for message 1 (same slot).  The model checks, at every copy, that the receiver
really granted THAT message, and at every receive that the slot holds the expected message.
"""
import threading
import time

import pytest

from mercury_artifact_b200 import comm, mesh

SHAPE = (4, 2)
WORLD = 8
ROUNDS = 2   # forwards back to back: message numbers keep growing, slots and words are reused


def _messages(rank):
    """(to_rank, from_rank) of every message of one forward, in program order (codegen.py:471-491)."""
    me = mesh.one_dim_to_n_dim(rank, SHAPE)
    out = []
    for outer in range(SHAPE[1]):
        for inner in range(SHAPE[0]):
            if inner + 1 != SHAPE[0]:
                d = 0
            elif outer + 1 != SHAPE[1]:
                d = 1
            else:
                continue
            to = mesh.n_dim_to_one_dim(mesh.shift_tuple_element(me, d, 1, SHAPE[d]), SHAPE)
            frm = mesh.n_dim_to_one_dim(mesh.shift_tuple_element(me, d, -1, SHAPE[d]), SHAPE)
            out.append((to, frm))
    return out


def _run(word_key, hold_back=True, timeout=20.0):
    words, inbox, grants = {}, {}, set()
    lock = threading.Lock()
    errors = []
    outer_granted = threading.Event()
    deadline = time.time() + timeout

    def store(word, value):
        with lock:
            words[word_key(word)] = value          # plain store: a smaller value lowers the word

    def wait_ge(word, value, who):
        while True:
            with lock:
                if words.get(word_key(word), 0) >= value:
                    return True
            if errors or time.time() > deadline:
                errors.append(f"rank {who}: wait for {word} >= {value} never satisfied")
                return False
            time.sleep(0.0005)

    def body(rank):
        seq = 0
        pending = None
        for _ in range(ROUNDS):
            for i, (to, frm) in enumerate(_messages(rank)):
                if pending is not None:                                     # wait() of the previous message
                    w, pfrm, pseq = pending
                    if not wait_ge(w["wait_ready"], w["value"], rank):
                        return
                    with lock:
                        got = inbox.get((rank, w["slot"]))
                    if got != (pfrm, pseq):
                        errors.append(f"rank {rank}: slot {w['slot']} holds {got}, expected message {pseq} from {pfrm}")
                        return
                w = comm.message_words(seq, rank, to, frm)
                if hold_back and rank == 1 and seq == 1:
                    outer_granted.wait(timeout)                             # the inner ring 0-3 lags behind
                store(w["grant"], w["value"])                               # commit(): grant, wait credit, copy, ready
                with lock:
                    grants.add((rank, frm, seq))
                if rank == 4 and seq == 3:
                    outer_granted.set()                                     # group 4-7 is two steps ahead
                if not wait_ge(w["wait_credit"], w["value"], rank):
                    return
                with lock:
                    if (to, rank, seq) not in grants:
                        errors.append(f"rank {rank}: copies message {seq} into rank {to} slot {w['slot']} "
                                      "before that rank released it")
                        return
                    inbox[(to, w["slot"])] = (rank, seq)
                store(w["raise_ready"], w["value"])
                pending = (w, frm, seq)
                seq += 1

    threads = [threading.Thread(target=body, args=(r,)) for r in range(WORLD)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout + 5)
    return errors


def test_one_writer_per_word_survives_a_lagging_inner_ring():
    assert _run(lambda word: word) == []
    assert _run(lambda word: word, hold_back=False) == []


def test_the_model_catches_a_word_shared_by_two_writers():
    """Same run with the peer index dropped from the word's key (one word per slot): the early grant of
    the outer neighbour satisfies the wait meant for the inner neighbour."""
    errs = _run(lambda word: (word[0], word[1], word[3]), timeout=5.0)
    assert errs and any("before that rank released it" in e or "never satisfied" in e for e in errs)


def test_words_have_distinct_addresses_per_peer_and_kind():
    class FakeBuf:
        def ptr(self, rank, off):
            return rank * (1 << 20) + off

    ch = comm._Channel.__new__(comm._Channel)
    ch.slot_bytes, ch.buf = 4096, FakeBuf()
    seen = set()
    for peer in range(comm.MAX_PEERS):
        for slot in (0, 1):
            for kind in ("ready", "credit"):
                p = ch.word_ptr((3, kind, peer, slot))
                assert p not in seen and 3 * (1 << 20) + 2 * 4096 <= p < 3 * (1 << 20) + 2 * 4096 + ch.FLAG_BYTES
                seen.add(p)
    with pytest.raises(ValueError):
        ch.word_ptr((0, "ready", comm.MAX_PEERS, 0))
