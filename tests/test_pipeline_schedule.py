"""Order of forward / backward / message operations that the pipeline engine issues on every stage, with the compute and
the point-to-point layer replaced by recorders (reference schedules: galvatron/core/runtime/pipeline/pipeline.py:375-701
1F1B-flush, :718-883 GPipe). Checks the schedule's shape (warm-up, steady 1F1B, cool-down), the bound on in-flight
micro-batches that the memory cost model relies on, and that the messages of neighbouring stages pair up."""
from types import SimpleNamespace

import pytest
import torch

from hetu_galvatron_b200.parallel.pipeline import PipelineParallel


def _trace(pp, stage, chunks, kind):
    p = object.__new__(PipelineParallel)
    p.mesh = SimpleNamespace(pp_deg=pp, stage=stage)
    p.pipeline_type, p.chunks = kind, chunks
    p.is_first, p.is_last = stage == 0, stage == pp - 1
    p.prev, p.next = stage - 1, stage + 1
    p.recv_shape_fn = lambda micro: [torch.Size([1])]
    events = []

    def fwd(micro, inputs):
        events.append(("F", micro["i"]))
        out = torch.zeros(1)
        return [out], (out if p.is_last else None)

    def bwd(inputs, outputs, grads, last):
        events.append(("B", None, last))
        return [] if p.is_first else [torch.zeros(1)]

    class Posted:
        def __init__(self, ident, bufs):
            self.ident, self.bufs = ident, bufs

        def wait(self):
            if self.ident is not None:
                events.append(("wait", self.ident))
            return self.bufs

    def post(send_to, send_tensors, recv_from, recv_shapes):
        if send_to is not None and send_tensors:
            events.append(("send", send_to))
        if recv_from is not None and recv_shapes:
            ident = sum(1 for e in events if e[0] == "recv")
            events.append(("recv", recv_from, ident))
            return Posted(ident, [torch.zeros(1) for _ in recv_shapes])
        return Posted(None, [])

    p._forward_compute, p._backward_compute, p._post = fwd, bwd, post
    p._exchange = lambda *a: post(*a).wait()
    p._inflight, p._pool = [], {}
    p.forward_backward([{"i": i} for i in range(chunks)])
    return events


@pytest.mark.parametrize("pp,chunks", [(2, 2), (2, 8), (4, 8), (4, 3), (8, 16)])
def test_1f1b_flush_shape_and_in_flight_bound(pp, chunks):
    for stage in range(pp):
        ev = [e for e in _trace(pp, stage, chunks, "pipedream_flush") if e[0] in "FB"]
        kinds = "".join(e[0] for e in ev)
        warm = min(pp - stage - 1, chunks)
        steady = chunks - warm
        assert kinds == "F" * warm + "FB" * steady + "B" * warm, (stage, kinds)
        assert [e[1] for e in ev if e[0] == "F"] == list(range(chunks))            # micro-batches in order
        assert [e[2] for e in ev if e[0] == "B"] == [False] * (chunks - 1) + [True]  # gradient reduction after the last one
        live = peak = 0
        for k in kinds:
            live += 1 if k == "F" else -1
            peak = max(peak, live)
        assert peak == min(pp - stage, chunks)                                      # what MemoryCostModel's 1F1B ratio assumes


@pytest.mark.parametrize("pp,chunks", [(2, 4), (4, 8)])
def test_gpipe_runs_all_forwards_first(pp, chunks):
    for stage in range(pp):
        kinds = "".join(e[0] for e in _trace(pp, stage, chunks, "gpipe") if e[0] in "FB")
        assert kinds == "F" * chunks + "B" * chunks


@pytest.mark.parametrize("kind", ["pipedream_flush", "gpipe"])
@pytest.mark.parametrize("pp,chunks", [(2, 4), (4, 8), (4, 2)])
def test_messages_between_neighbouring_stages_pair_up(pp, chunks, kind):
    traces = [_trace(pp, s, chunks, kind) for s in range(pp)]
    for s in range(pp - 1):
        down_sends = sum(1 for e in traces[s] if e == ("send", s + 1))
        down_recvs = sum(1 for e in traces[s + 1] if e[:2] == ("recv", s))
        up_sends = sum(1 for e in traces[s + 1] if e == ("send", s))
        up_recvs = sum(1 for e in traces[s] if e[:2] == ("recv", s + 1))
        assert down_sends == down_recvs == chunks and up_sends == up_recvs == chunks
    assert not any(e[0] in ("send", "recv") and e[1] < 0 for e in traces[0])
    assert not any(e[0] in ("send", "recv") and e[1] >= pp for e in traces[-1])


@pytest.mark.parametrize("kind", ["pipedream_flush", "gpipe"])
@pytest.mark.parametrize("pp,chunks", [(2, 2), (2, 8), (4, 8), (4, 3), (8, 16)])
def test_posted_messages_cannot_deadlock_and_receives_run_ahead(pp, chunks, kind):
    """Replays the stages' traces against each other: a wait on the k-th receive from a peer completes once that peer
    has posted its k-th send to this stage (messages between a pair match in posting order per direction). Every stage
    must finish, and receives of forward inputs are posted before the compute that precedes their use."""
    traces = [_trace(pp, s, chunks, kind) for s in range(pp)]
    pos = [0] * pp
    sent = {}                      # (src, dst) -> number of sends posted
    recv_index = [{} for _ in range(pp)]   # stage -> receive id -> (peer, k-th receive from that peer)
    for s, tr in enumerate(traces):
        per_peer = {}
        for e in tr:
            if e[0] == "recv":
                k = per_peer.get(e[1], 0)
                per_peer[e[1]] = k + 1
                recv_index[s][e[2]] = (e[1], k)
    progress = True
    while progress:
        progress = False
        for s, tr in enumerate(traces):
            while pos[s] < len(tr):
                e = tr[pos[s]]
                if e[0] == "send":
                    sent[(s, e[1])] = sent.get((s, e[1]), 0) + 1
                elif e[0] == "wait":
                    peer, k = recv_index[s][e[1]]
                    if sent.get((peer, s), 0) <= k:
                        break
                pos[s] += 1
                progress = True
    assert all(pos[s] == len(traces[s]) for s in range(pp)), [(pos[s], len(traces[s])) for s in range(pp)]
    # one micro-batch ahead: on a stage that receives forward inputs, the receive of input i + 1 is posted before the
    # forward pass of micro-batch i whenever another input is still to come
    for s in range(1, pp):
        tr = traces[s]
        posted = 0
        for e in tr:
            if e[:2] == ("recv", s - 1):
                posted += 1
            if e[0] == "F" and e[1] + 1 < chunks and kind == "gpipe":
                assert posted >= e[1] + 2, (s, e, posted)
        if kind == "pipedream_flush":
            # in the steady phase the receive of the next input precedes the backward pass before it
            idx = [i for i, e in enumerate(tr) if e[0] == "B"]
            for i in idx[:-1]:
                nxt_f = next((j for j in range(i, len(tr)) if tr[j][0] == "F"), None)
                if nxt_f is not None:
                    assert any(tr[j][:2] == ("recv", s - 1) for j in range(0, i)), (s, i)


def _group_trace(pp, stage, chunks, kind):
    """Like ``_trace`` but every posted group is one event: ("post", [("send", peer) | ("recv", peer), ...], receive id)."""
    p = object.__new__(PipelineParallel)
    p.mesh = SimpleNamespace(pp_deg=pp, stage=stage)
    p.pipeline_type, p.chunks = kind, chunks
    p.is_first, p.is_last = stage == 0, stage == pp - 1
    p.prev, p.next = stage - 1, stage + 1
    p.recv_shape_fn = lambda micro: [torch.Size([1])]
    p._connected = True
    events = []

    class Posted:
        def __init__(self, ident, bufs):
            self.ident, self.bufs = ident, bufs

        def wait(self):
            if self.ident is not None:
                events.append(("wait", self.ident))
            return self.bufs

    def post(send_to, send_tensors, recv_from, recv_shapes):
        ops, ident = [], None
        if send_to is not None and send_tensors:
            ops.append(("send", send_to))
        if recv_from is not None and recv_shapes:
            ops.append(("recv", recv_from))
            ident = sum(1 for e in events if e[0] == "post" and e[2] is not None)
        if ops:
            events.append(("post", ops, ident))
        return Posted(ident, [torch.zeros(1) for _ in (recv_shapes or [])] if ident is not None else [])

    p._forward_compute = lambda micro, inputs: (events.append(("F", micro["i"])) or ([torch.zeros(1)], torch.zeros(1) if p.is_last else None))
    p._backward_compute = lambda inputs, outputs, grads, last: (events.append(("B",)) or ([] if p.is_first else [torch.zeros(1)]))
    p._post = post
    p._exchange = lambda *a: post(*a).wait()
    p._inflight, p._pool = [], {}
    p.forward_backward([{"i": i} for i in range(chunks)])
    return events


def _replay_with_first_use_rules(traces, connected):
    """Replays host programs under two first-use rules of the real libraries: (1) posting a group that contains the first
    message of a (source, destination) direction blocks the HOST until the peer has reached its own first message of that
    direction (connection set-up); (2) the first backward pass of a stage loads kernels, which waits until every receive
    posted before it on that stage has completed (device synchronisation). A receive completes once the matching send has
    been posted. Returns the positions reached."""
    pp = len(traces)
    pos = [0] * pp
    sent, reached = {}, set(connected)       # reached: (stage, direction) whose first message the stage's host has arrived at
    first_b_done = [False] * pp

    def recv_complete(stage, upto):
        """every receive of ``stage`` posted at trace positions < upto has its matching send posted"""
        need = {}
        for e in traces[stage][:upto]:
            if e[0] == "post":
                for kind, peer in e[1]:
                    if kind == "recv":
                        need[peer] = need.get(peer, 0) + 1
        return all(sent.get((peer, stage), 0) >= k for peer, k in need.items())

    progress = True
    while progress:
        progress = False
        for s, tr in enumerate(traces):
            while pos[s] < len(tr):
                e = tr[pos[s]]
                if e[0] == "post":
                    dirs = [((s, peer) if kind == "send" else (peer, s)) for kind, peer in e[1]]
                    for d in dirs:
                        reached.add((s, d))                       # this host has arrived at the set-up of direction d
                    if any((d[0] if d[0] != s else d[1], d) not in reached and d not in connected for d in dirs):
                        break                                      # the peer has not arrived yet: host blocked
                    for d in dirs:
                        connected.add(d)
                    for kind, peer in e[1]:
                        if kind == "send":
                            sent[(s, peer)] = sent.get((s, peer), 0) + 1
                elif e[0] == "B" and not first_b_done[s]:
                    if not recv_complete(s, pos[s]):
                        break
                    first_b_done[s] = True
                elif e[0] == "wait":
                    k = e[1]
                    posts = [x for x in tr if x[0] == "post" and x[2] is not None]
                    peer = next(pr for kind, pr in posts[k][1] if kind == "recv")
                    nth = sum(1 for x in posts[:k + 1] if any(kind == "recv" and pr == peer for kind, pr in x[1]))
                    if sent.get((peer, s), 0) < nth:
                        break
                pos[s] += 1
                progress = True
    return pos


@pytest.mark.parametrize("pp,chunks", [(2, 4), (4, 8)])
def test_first_use_setup_inside_the_schedule_can_deadlock_and_preconnection_removes_it(pp, chunks):
    """The hang seen on two GPUs: stage 0 blocks in the set-up of the gradient direction (grouped with the send of the next
    activation), stage 1's receive for that activation is posted ahead and pending, and stage 1's first backward pass waits
    for it. With every neighbour direction connected before the schedule (what ``_connect_neighbours`` does) every stage
    finishes."""
    traces = [_group_trace(pp, s, chunks, "pipedream_flush") for s in range(pp)]
    stuck = _replay_with_first_use_rules(traces, connected=set())
    assert any(stuck[s] < len(traces[s]) for s in range(pp))
    every_direction = {(a, b) for a in range(pp) for b in (a - 1, a + 1) if 0 <= b < pp}
    done = _replay_with_first_use_rules(traces, connected=set(every_direction))
    assert all(done[s] == len(traces[s]) for s in range(pp))
