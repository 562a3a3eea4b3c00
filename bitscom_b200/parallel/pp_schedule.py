"""1F1B pipeline schedule over NCCL point-to-point.

The reference trainer drives its stages with torch's ``ScheduleGPipe``
(``benchmarks/train_llama7b_dp_pp_lowbit.py:240-264``: all forwards, then all
backwards).  This is an own one-forward-one-backward schedule: stage ``s`` of ``P`` runs
``min(P - s - 1, M)`` warm-up forwards, then alternates forward/backward, then drains the
remaining backwards, so at most ``P - s`` micro-batches of activations are alive.

``build_1f1b(stage, stages, microbatches)`` returns the action list (pure Python, tested
on CPU); ``PipelineRunner`` executes it: activations and their gradients travel as bf16
tensors through ``batch_isend_irecv`` on the pipeline group (NCCL runs them on its own
stream; the compute stream only waits where a tensor is consumed), a send that follows a
compute step is posted together with the receive the next step needs, which keeps
neighbouring stages from blocking each other.
"""

from __future__ import annotations

import contextlib
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from .deferred import DeferredWork

Action = Tuple[str, int]  # ("F" | "B", micro-batch index)


def build_1f1b(stage: int, stages: int, microbatches: int) -> List[Action]:
    warm = min(stages - stage - 1, microbatches)
    actions: List[Action] = [("F", i) for i in range(warm)]
    f, b = warm, 0
    for _ in range(microbatches - warm):
        actions.append(("F", f))
        f += 1
        actions.append(("B", b))
        b += 1
    while b < microbatches:
        actions.append(("B", b))
        b += 1
    return actions


def max_live_microbatches(actions: Sequence) -> int:
    """Most forwards whose backward has not run yet, at any point of an action list (plain
    ``(kind, mb)`` or interleaved ``(kind, mb, chunk)`` actions): the activation memory a rank
    needs, in units of one micro-batch through one stage (plain) or one chunk (interleaved;
    ``(P - rank - 1) * 2 + (chunks - 1) * P + 1`` chunk activations, each 1 / chunks of a
    stage's)."""
    live = peak = 0
    for action in actions:
        live += 1 if action[0] == "F" else -1
        peak = max(peak, live)
    return peak


def simulate_timeline(stages: int, microbatches: int, t_forward: float = 1.0,
                      t_input_grad: float = 1.0, t_weight_grad: float = 1.0,
                      defer_wgrad: bool = False, t_send: float = 0.0,
                      defer_last: bool = False) -> dict:
    """Event simulation of one 1F1B step: every stage executes ``build_1f1b`` in order, a
    forward waits for the previous stage's forward of the same micro-batch (plus ``t_send``), a
    backward for the next stage's input gradient.  A backward step costs ``t_input_grad +
    t_weight_grad``; with ``defer_wgrad`` the input gradient is released after
    ``t_input_grad`` and the weight-gradient part runs behind it on the same stage, for every
    backward but the step's last, or for all of them with ``defer_last`` (as ``PipelineRunner``
    does).  Returns the step time, the ideal time (no waiting) and their ratio.  At equal costs
    2 stages x 8 micro-batches give 0.889 without deferral, 0.889 with it and 0.923 with
    ``defer_last``: the pipeline drains through the last micro-batch's backward steps, so only
    deferring those takes weight-gradient time off the critical path."""
    plans = [build_1f1b(s, stages, microbatches) for s in range(stages)]
    pos = [0] * stages
    clock = [0.0] * stages
    fwd_done = [[None] * microbatches for _ in range(stages)]   # when the activation is sent
    grad_out = [[None] * microbatches for _ in range(stages)]   # when the input gradient is sent
    remaining = sum(len(p) for p in plans)
    while remaining:
        progressed = False
        for s in range(stages):
            if pos[s] >= len(plans[s]):
                continue
            kind, mb = plans[s][pos[s]]
            if kind == "F":
                ready = 0.0 if s == 0 else fwd_done[s - 1][mb]
            else:
                ready = 0.0 if s == stages - 1 else grad_out[s + 1][mb]
            if ready is None:
                continue
            start = max(clock[s], ready + (t_send if ready else 0.0))
            if kind == "F":
                clock[s] = start + t_forward
                fwd_done[s][mb] = clock[s]
            else:
                last_backward = mb == microbatches - 1
                if defer_wgrad and (defer_last or not last_backward):
                    grad_out[s][mb] = start + t_input_grad
                else:
                    grad_out[s][mb] = start + t_input_grad + t_weight_grad
                clock[s] = start + t_input_grad + t_weight_grad
            pos[s] += 1
            remaining -= 1
            progressed = True
        if not progressed:
            raise RuntimeError("the schedule deadlocks")
    ideal = microbatches * (t_forward + t_input_grad + t_weight_grad)
    step = max(clock)
    return {"step_time": step, "ideal_time": ideal, "efficiency": ideal / step}


class Comm:
    """Point-to-point traffic posted as ONE batch after a compute step."""

    __slots__ = ("send_next", "send_prev", "recv_prev", "recv_next")

    def __init__(self, send_next=False, send_prev=False, recv_prev=False, recv_next=False):
        self.send_next, self.send_prev = send_next, send_prev
        self.recv_prev, self.recv_next = recv_prev, recv_next

    def any(self) -> bool:
        return self.send_next or self.send_prev or self.recv_prev or self.recv_next

    def __repr__(self):
        names = [n for n in self.__slots__ if getattr(self, n)]
        return "Comm(" + ",".join(names) + ")"


def communication_plan(stage: int, stages: int, microbatches: int
                       ) -> List[Tuple[str, int, Comm]]:
    """[(kind, micro-batch, traffic posted after the step)], preceded by a ("P", -1, comm)
    priming entry when the stage must receive its first input.  A send that follows a
    compute step shares its batch with the receive the next step needs."""
    first, last = stage == 0, stage == stages - 1
    actions = build_1f1b(stage, stages, microbatches)
    plan: List[Tuple[str, int, Comm]] = []
    if not first and actions and actions[0][0] == "F":
        plan.append(("P", -1, Comm(recv_prev=True)))
    for pos, (kind, mb) in enumerate(actions):
        nxt = actions[pos + 1][0] if pos + 1 < len(actions) else None
        if kind == "F":
            comm = Comm(send_next=not last,
                        recv_prev=(nxt == "F" and not first),
                        recv_next=(nxt == "B" and not last))
        else:
            comm = Comm(send_prev=not first,
                        recv_prev=(nxt == "F" and not first),
                        recv_next=(nxt == "B" and not last))
        plan.append((kind, mb, comm))
    return plan


class PipelineRunner:
    """Executes one training step of one pipeline stage.

    ``forward_fn(mb_index, input_or_None) -> output`` runs the stage on a micro-batch
    (first stage ignores the input, last stage returns the scalar loss);
    ``act_shape`` is the shape of the hidden states exchanged between stages.
    """

    def __init__(self, stage: int, stages: int, group, prev_rank: Optional[int],
                 next_rank: Optional[int], act_shape: Tuple[int, ...],
                 dtype: torch.dtype = torch.bfloat16, device="cuda", defer_wgrad: bool = False,
                 defer_last: bool = False):
        # defer_wgrad: backward steps queue their weight-gradient GEMMs and run them after the
        # input gradient has been handed to the transport.  The step's last backward is left
        # alone unless defer_last is set: data-parallel bucket hooks that fire during it rely on
        # finished weight gradients.  Without such hooks defer_last should be set: the drain of
        # the pipeline runs through exactly that backward (see simulate_timeline), so it is the
        # one deferral that shortens the step.
        self.defer_wgrad = defer_wgrad
        self.defer_last = defer_last
        self.stage, self.stages, self.group = stage, stages, group
        self.prev_rank, self.next_rank = prev_rank, next_rank
        self.act_shape, self.dtype, self.device = tuple(act_shape), dtype, device
        self.is_first, self.is_last = stage == 0, stage == stages - 1

    def _exchange(self, comm: Comm, to_next=None, to_prev=None, between=None):
        """Issue the step's sends / receives; ``between`` runs after they have been issued and
        before they are waited for (work that overlaps the transfer)."""
        ops, got_prev, got_next = [], None, None
        if comm.send_prev:
            ops.append(dist.P2POp(dist.isend, to_prev, self.prev_rank, self.group))
        if comm.recv_prev:
            got_prev = torch.empty(self.act_shape, dtype=self.dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, got_prev, self.prev_rank, self.group))
        if comm.send_next:
            ops.append(dist.P2POp(dist.isend, to_next, self.next_rank, self.group))
        if comm.recv_next:
            got_next = torch.empty(self.act_shape, dtype=self.dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, got_next, self.next_rank, self.group))
        reqs = dist.batch_isend_irecv(ops) if ops else []
        if between is not None:
            between()
        for req in reqs:
            req.wait()  # stream-ordered wait; the host does not block
        return got_prev, got_next

    def run(self, microbatches: int, forward_fn: Callable, on_last_backward: Optional[
            Callable[[], None]] = None) -> List[torch.Tensor]:
        """Returns the per-micro-batch losses (last stage) or an empty list."""
        plan = communication_plan(self.stage, self.stages, microbatches)
        last_b = max((i for i, (k, _, _) in enumerate(plan) if k == "B"), default=-1)
        inputs: dict = {}
        outputs: dict = {}
        losses: List[torch.Tensor] = []
        next_input = next_grad = None
        flush = None  # weight-gradient work queued by the current backward step
        for pos, (kind, mb, comm) in enumerate(plan):
            if flush is not None:  # the previous step had nothing to send: run its queue now
                flush()
                flush = None
            to_next = to_prev = None
            if kind == "F":
                x = None
                if not self.is_first:
                    x = next_input.requires_grad_()
                    next_input = None
                    inputs[mb] = x
                out = forward_fn(mb, x)
                outputs[mb] = out
                if self.is_last:
                    losses.append(out.detach())
                else:
                    to_next = out.detach()
            elif kind == "B":
                out = outputs.pop(mb)
                if pos == last_b and on_last_backward is not None:
                    on_last_backward()
                deferred = DeferredWork() if (
                    self.defer_wgrad and (pos != last_b or self.defer_last)) else None
                with deferred if deferred is not None else contextlib.nullcontext():
                    if self.is_last:
                        out.backward()
                    else:
                        torch.autograd.backward(out, grad_tensors=next_grad)
                        next_grad = None
                if not self.is_first:
                    to_prev = inputs.pop(mb).grad
                if deferred is not None:
                    flush = deferred.flush
            if comm.any():
                got_prev, got_next = self._exchange(comm, to_next, to_prev, between=flush)
                flush = None
                if comm.recv_prev:
                    next_input = got_prev
                if comm.recv_next:
                    next_grad = got_next
        if flush is not None:
            flush()
        return losses


# ----------------------------------------------------------------------------------
# Interleaved 1F1B: several model chunks per rank ("virtual stages")
# ----------------------------------------------------------------------------------
# With v chunks per rank the model is cut into V = P * v virtual stages; virtual stage s lives
# on rank s % P as chunk s // P, so a micro-batch visits every rank v times and the pipeline's
# fill / drain costs (P - 1) / v stage times instead of P - 1: the idle share of a step drops
# from (P - 1) / (M + P - 1) to (P - 1) / (v M + P - 1) (2 stages x 8 micro-batches: 11.1 % ->
# 5.9 % with two chunks).  The price is v times as many (smaller) point-to-point messages and
# up to (P - r - 1) * 2 + (v - 1) * P + 1 live micro-batch activations on rank r.  The reference
# has no pipeline schedule of its own (torch's GPipe, train_llama7b_dp_pp_lowbit.py:240-264).

VAction = Tuple[str, int, int]  # ("F" | "B", micro-batch, chunk)


def interleaved_warmup(rank: int, stages: int, microbatches: int, chunks: int) -> int:
    """Forwards a rank runs before its first backward."""
    P, M, v = stages, microbatches, chunks
    if v == 1:
        return min(P - rank - 1, M)
    # with exactly P micro-batches the first ranks would run all their forwards first while the
    # last ones alternate, and their batches no longer line up: every rank then runs all
    # forwards before any backward
    return M * v if M == P else min((P - rank - 1) * 2 + (v - 1) * P, M * v)


def build_interleaved(rank: int, stages: int, microbatches: int, chunks: int) -> List[VAction]:
    """Action list of ``rank``: micro-batches go through the chunks in groups of ``stages``
    (the first P micro-batches through chunk 0, the same P through chunk 1, ..., then the next
    P), backwards with the chunks reversed; ``(P - rank - 1) * 2 + (chunks - 1) * P`` warm-up
    forwards, then one forward / one backward, then the remaining backwards.
    ``microbatches`` must be a multiple of ``stages``."""
    P, M, v = stages, microbatches, chunks
    if v == 1:
        return [(k, mb, 0) for k, mb in build_1f1b(rank, P, M)]
    if M % P:
        raise ValueError(f"interleaved schedule: micro-batches ({M}) must be a multiple of the "
                         f"pipeline stages ({P})")
    total = M * v

    def fwd(k: int) -> Tuple[int, int]:
        group, within = divmod(k, P * v)
        chunk, pos = divmod(within, P)
        return group * P + pos, chunk

    def bwd(k: int) -> Tuple[int, int]:
        mb, chunk = fwd(k)
        return mb, v - 1 - chunk

    warm = interleaved_warmup(rank, P, M, v)
    actions: List[VAction] = [("F",) + fwd(k) for k in range(warm)]
    f, b = warm, 0
    while f < total:
        actions.append(("F",) + fwd(f))
        f += 1
        actions.append(("B",) + bwd(b))
        b += 1
    while b < total:
        actions.append(("B",) + bwd(b))
        b += 1
    return actions


class Message:
    """One tensor on the wire: activation ("act") of micro-batch ``mb`` leaving virtual stage
    ``vstage``, or gradient ("grad") w.r.t. the input of virtual stage ``vstage``."""

    __slots__ = ("kind", "mb", "vstage", "src", "dst")

    def __init__(self, kind: str, mb: int, vstage: int, src: int, dst: int):
        self.kind, self.mb, self.vstage, self.src, self.dst = kind, mb, vstage, src, dst

    def tag(self) -> Tuple[str, int, int]:
        return (self.kind, self.mb, self.vstage)

    def __repr__(self):
        return f"{self.kind}(mb{self.mb}, vs{self.vstage}, {self.src}->{self.dst})"


def _needs(rank: int, P: int, v: int, action: VAction) -> Optional[Message]:
    kind, mb, chunk = action
    vs, V = chunk * P + rank, P * v
    if kind == "F":
        return None if vs == 0 else Message("act", mb, vs - 1, (rank - 1) % P, rank)
    return None if vs == V - 1 else Message("grad", mb, vs + 1, (rank + 1) % P, rank)


def _yields(rank: int, P: int, v: int, action: VAction) -> Optional[Message]:
    kind, mb, chunk = action
    vs, V = chunk * P + rank, P * v
    if kind == "F":
        return None if vs == V - 1 else Message("act", mb, vs, rank, (rank + 1) % P)
    return None if vs == 0 else Message("grad", mb, vs, rank, (rank - 1) % P)


def schedule_units(actions: Sequence[VAction], warmup: int) -> List[List[VAction]]:
    """Cuts an action list into the units after which a rank communicates: each of the
    ``warmup`` leading forwards, then forward + backward pairs, then single backwards."""
    units: List[List[VAction]] = [[a] for a in actions[:warmup]]
    i = warmup
    while i < len(actions):
        if actions[i][0] == "F":
            units.append([actions[i], actions[i + 1]])
            i += 2
        else:
            units.append([actions[i]])
            i += 1
    return units


def virtual_plan(rank: int, stages: int, microbatches: int, chunks: int
                 ) -> List[Tuple[List[VAction], List[Message], List[Message]]]:
    """[(unit, sends, receives)]: after the actions of ``unit`` (empty for the priming entry)
    the rank posts ONE batch that sends what the unit produced and receives what the NEXT
    unit consumes, activations before gradients in both lists.  In the steady state a unit is
    one forward plus one backward, so the gradient of the next backward arrives a whole unit
    before it is used: that slack is what keeps neighbouring ranks, whose units are offset
    against each other, from waiting on one another in a cycle (a receive posted only one
    ACTION ahead deadlocks: the peer's matching send sits behind a receive of its own)."""
    actions = build_interleaved(rank, stages, microbatches, chunks)
    units = schedule_units(actions, interleaved_warmup(rank, stages, microbatches, chunks))

    def needs(unit):
        got = [m for m in (_needs(rank, stages, chunks, a) for a in unit) if m is not None]
        return sorted(got, key=lambda m: m.kind)      # "act" < "grad"

    def yields(unit):
        out = [m for m in (_yields(rank, stages, chunks, a) for a in unit) if m is not None]
        return sorted(out, key=lambda m: m.kind)

    plan: List[Tuple[List[VAction], List[Message], List[Message]]] = []
    if units and needs(units[0]):
        plan.append(([], [], needs(units[0])))
    for i, unit in enumerate(units):
        plan.append((unit, yields(unit), needs(units[i + 1]) if i + 1 < len(units) else []))
    return plan


def check_virtual_plan(stages: int, microbatches: int, chunks: int) -> int:
    """Plays all ranks' plans under NCCL's rules and raises ``RuntimeError`` on a deadlock or a
    mismatched tensor; returns the number of messages delivered.  Rules: the operations of a
    batch run concurrently; between one (sender, receiver) pair messages match in the order
    they were posted on both sides (inside a batch: list order); a rank moves on when every
    operation of its batch has matched; a backward runs only after its forward."""
    P = stages
    plans = [[(u, list(s), list(r)) for u, s, r in virtual_plan(k, P, microbatches, chunks)]
             for k in range(P)]
    pos = [0] * P
    sends: List[List[Message]] = [[] for _ in range(P)]
    recvs: List[List[Message]] = [[] for _ in range(P)]
    have: List[set] = [set() for _ in range(P)]     # tags of the inputs a rank holds
    seen_fwd: List[set] = [set() for _ in range(P)]

    def load(k: int) -> None:
        if pos[k] < len(plans[k]):
            unit, s, r = plans[k][pos[k]]
            for act in unit:                          # the unit's compute comes first
                need = _needs(k, P, chunks, act)
                if need is not None and need.tag() not in have[k]:
                    raise RuntimeError(f"rank {k} runs {act} before it holds {need}")
                if act[0] == "F":
                    seen_fwd[k].add(act[1:])
                elif act[1:] not in seen_fwd[k]:
                    raise RuntimeError(f"rank {k} runs {act} before its forward")
            sends[k], recvs[k] = list(s), list(r)

    for k in range(P):
        load(k)
    delivered = 0
    for _ in range(16 * P * microbatches * chunks + 64):
        if all(pos[k] >= len(plans[k]) for k in range(P)):
            return delivered
        progressed = False
        for k in range(P):
            for s in list(sends[k]):
                first_to_dst = next(m for m in sends[k] if m.dst == s.dst)
                if first_to_dst is not s:
                    continue
                r = next((m for m in recvs[s.dst] if m.src == k), None)
                if r is None:
                    continue
                if r.tag() != s.tag():
                    raise RuntimeError(f"rank {s.dst} expected {r} but rank {k} sent {s}")
                sends[k].remove(s)
                recvs[s.dst].remove(r)
                have[s.dst].add(s.tag())
                delivered += 1
                progressed = True
        for k in range(P):
            if pos[k] < len(plans[k]) and not sends[k] and not recvs[k]:
                pos[k] += 1
                load(k)
                progressed = True
        if not progressed:
            raise RuntimeError(f"the plan deadlocks at positions {pos}: sends {sends}, "
                               f"receives {recvs}")
    raise RuntimeError("the plan did not terminate")


def simulate_interleaved_timeline(stages: int, microbatches: int, chunks: int,
                                  t_forward: float = 1.0, t_backward: float = 2.0) -> dict:
    """Event simulation of the interleaved schedule with per-chunk costs ``t_forward / chunks``
    and ``t_backward / chunks`` (a chunk is 1 / chunks of a stage): step time, ideal time and
    their ratio."""
    P, v = stages, chunks
    plans = [build_interleaved(k, P, microbatches, v) for k in range(P)]
    tf, tb = t_forward / v, t_backward / v
    done: dict = {}
    clock = [0.0] * P
    pos = [0] * P
    remaining = sum(len(p) for p in plans)
    while remaining:
        progressed = False
        for k in range(P):
            if pos[k] >= len(plans[k]):
                continue
            act = plans[k][pos[k]]
            need = _needs(k, P, v, act)
            ready = 0.0
            if need is not None:
                if need.tag() not in done:
                    continue
                ready = done[need.tag()]
            start = max(clock[k], ready)
            clock[k] = start + (tf if act[0] == "F" else tb)
            out = _yields(k, P, v, act)
            if out is not None:
                done[out.tag()] = clock[k]
            pos[k] += 1
            remaining -= 1
            progressed = True
        if not progressed:
            raise RuntimeError("the schedule deadlocks")
    ideal = microbatches * (t_forward + t_backward)
    return {"step_time": max(clock), "ideal_time": ideal, "efficiency": ideal / max(clock)}


def simulate_plan_timeline(stages: int, microbatches: int, chunks: int,
                           t_forward: float = 1.0, t_backward: float = 2.0) -> dict:
    """Like ``simulate_interleaved_timeline`` but with the coupling the batches add: a send or
    receive completes when BOTH sides have posted it, and a rank starts its next unit only when
    its whole batch has completed (transfers themselves take no time).  For two or more chunks
    the unit-batched plan loses nothing against the pure data-flow bound; for ONE chunk it
    halves the throughput (the steady-state unit then waits for a gradient the peer can only
    produce after this unit's activation), which is why a single chunk runs under
    ``PipelineRunner`` with its batch-per-action plan instead."""
    P, v = stages, chunks
    plans = [[(u, list(s), list(r)) for u, s, r in virtual_plan(k, P, microbatches, v)]
             for k in range(P)]
    pos, post, last = [0] * P, [0.0] * P, [0.0] * P
    sends: List[List[Message]] = [[] for _ in range(P)]
    recvs: List[List[Message]] = [[] for _ in range(P)]

    def load(k: int, now: float) -> None:
        if pos[k] < len(plans[k]):
            unit, s, r = plans[k][pos[k]]
            post[k] = now + sum((t_forward if a[0] == "F" else t_backward) / v for a in unit)
            last[k] = post[k]
            sends[k], recvs[k] = list(s), list(r)

    for k in range(P):
        load(k, 0.0)
    while not all(pos[k] >= len(plans[k]) for k in range(P)):
        progressed = False
        for k in range(P):
            for s in list(sends[k]):
                if next(m for m in sends[k] if m.dst == s.dst) is not s:
                    continue
                r = next((m for m in recvs[s.dst] if m.src == k), None)
                if r is None:
                    continue
                when = max(post[k], post[s.dst])
                last[k], last[s.dst] = max(last[k], when), max(last[s.dst], when)
                sends[k].remove(s)
                recvs[s.dst].remove(r)
                progressed = True
        for k in range(P):
            if pos[k] < len(plans[k]) and not sends[k] and not recvs[k]:
                pos[k] += 1
                load(k, last[k])
                progressed = True
        if not progressed:
            raise RuntimeError("the plan deadlocks")
    ideal = microbatches * (t_forward + t_backward)
    return {"step_time": max(last), "ideal_time": ideal, "efficiency": ideal / max(last)}


class InterleavedRunner:
    """Executes one training step of one rank that holds ``chunks`` >= 2 model chunks.

    ``forward_fn(mb, chunk, input_or_None) -> output`` runs chunk ``chunk`` on micro-batch
    ``mb`` (virtual stage 0 ignores the input, the last virtual stage returns the scalar
    loss).  ``ring`` lists the global ranks of the pipeline group in stage order; activations
    leave the last rank for the first one between chunks, gradients the other way round."""

    def __init__(self, rank: int, stages: int, chunks: int, group, ring: Sequence[int],
                 act_shape: Tuple[int, ...], dtype: torch.dtype = torch.bfloat16, device="cuda",
                 defer_wgrad: bool = False):
        if chunks < 2:
            raise ValueError("InterleavedRunner needs two or more chunks per rank; one chunk "
                             "runs under PipelineRunner")
        self.rank, self.stages, self.chunks, self.group = rank, stages, chunks, group
        self.ring = list(ring)
        self.act_shape, self.dtype, self.device = tuple(act_shape), dtype, device
        self.defer_wgrad = defer_wgrad

    def run(self, microbatches: int, forward_fn: Callable) -> List[torch.Tensor]:
        """Returns the per-micro-batch losses (rank of the last virtual stage) or []."""
        P, v, rank = self.stages, self.chunks, self.rank
        held: dict = {}      # tag -> tensor received and not yet consumed
        inputs: dict = {}    # (mb, chunk) -> leaf input of a forward awaiting its backward
        outputs: dict = {}
        losses: List[torch.Tensor] = []
        for unit, sends, recvs in virtual_plan(rank, P, microbatches, v):
            payload: dict = {}
            flush = None
            for action in unit:
                kind, mb, chunk = action
                need = _needs(rank, P, v, action)
                out_msg = _yields(rank, P, v, action)
                if kind == "F":
                    x = None
                    if need is not None:
                        x = held.pop(need.tag()).requires_grad_()
                        inputs[(mb, chunk)] = x
                    out = forward_fn(mb, chunk, x)
                    outputs[(mb, chunk)] = out
                    if out_msg is None:
                        losses.append(out.detach())
                    else:
                        payload[out_msg.tag()] = out.detach()
                else:
                    out = outputs.pop((mb, chunk))
                    deferred = DeferredWork() if self.defer_wgrad else None
                    with deferred if deferred is not None else contextlib.nullcontext():
                        if need is None:
                            out.backward()
                        else:
                            torch.autograd.backward(out, grad_tensors=held.pop(need.tag()))
                    if out_msg is not None:
                        payload[out_msg.tag()] = inputs.pop((mb, chunk)).grad
                    if deferred is not None:
                        flush = deferred.flush
            ops = [dist.P2POp(dist.isend, payload[m.tag()], self.ring[m.dst], self.group)
                   for m in sends]
            for m in recvs:
                buf = torch.empty(self.act_shape, dtype=self.dtype, device=self.device)
                held[m.tag()] = buf
                ops.append(dist.P2POp(dist.irecv, buf, self.ring[m.src], self.group))
            reqs = dist.batch_isend_irecv(ops) if ops else []
            if flush is not None:      # weight-gradient GEMMs overlap the transfer
                flush()
            for req in reqs:
                req.wait()             # stream-ordered; the host does not block
        return losses
