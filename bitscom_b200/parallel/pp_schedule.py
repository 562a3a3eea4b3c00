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


def max_live_microbatches(actions: Sequence[Action]) -> int:
    live = peak = 0
    for kind, _ in actions:
        live += 1 if kind == "F" else -1
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
