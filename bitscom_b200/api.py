"""``LowBitGroup``: low-bit collectives over a ``torch.distributed`` process group.

Public surface and path selection follow the reference wrapper
(``python/bitscom/api.py:313-1519`` in Squirrel7ang/bitscom):

    backend_allreduce -> local-only -> hierarchical pipeline-A -> flat low-bit -> dense

The flat low-bit all-reduce has three interchangeable engines that produce the same
bits (nearest rounding) for the same inputs:

* **fused** (CUDA tensors on one NVSwitch domain): one hand-written sm_100a kernel per
  bucket that quantizes, pushes packed shards into the peers' receive slots, reduces,
  re-quantizes, gathers and dequantizes (``bitscom_b200.parallel.fused``);
* **list collectives**: two ``dist.all_to_all`` + two ``dist.all_gather`` of packed
  bytes and fp16 scales, the reference's own composition (``api.py:703-875``);
* **single-tensor collectives** for backends without list all-to-all (gloo):
  ``all_to_all_single`` on stacked ``[W, bytes]`` tensors.

Beyond the reference, the Python engines also carry first- and second-stage error
feedback (the reference has it only inside its C++ backend,
``cpp/src/process_group_lowbit.cc:696-770,1136-1170``) and a seedable stochastic
rounding stream.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Tuple

import torch
import torch.distributed as dist

from .quantization import (
    DEFAULT_BLOCK_SIZE,
    SUPPORTED_BITWIDTHS,
    _HAS_CUDA_KERNELS,  # noqa: F401  (re-exported: callers of the reference patch it here)
    CompressedTensor,
    compress_tensor,
    decompress_tensor,
    quantize_pack_tensor_blockwise,
    roundtrip_tensor,
    stage1_stream,
    unpack_dequantize_tensor_blockwise,
)
from .utils import timing as _timing

_TRUE = {"1", "true", "yes", "on"}


def _env_flag(name: str) -> bool:
    return os.environ.get(name, "0").strip().lower() in _TRUE


# ----------------------------------------------------------------------------------
# Work-like handles
# ----------------------------------------------------------------------------------

class _ImmediateWork:
    """Handle for an operation that already finished on the host."""

    def wait(self):
        return True

    def is_completed(self) -> bool:
        return True

    def block_current_stream(self):
        return True


class _CudaEventWork:
    """Handle backed by a CUDA event recorded on the stream that ran the collective."""

    def __init__(self, event: "torch.cuda.Event", keepalive: Optional[list] = None,
                 on_complete=None):
        self.event = event
        self.keepalive = keepalive or []
        self._on_complete = on_complete

    def _finish(self):
        if self._on_complete is not None:
            cb, self._on_complete = self._on_complete, None
            cb()

    def wait(self):
        self.event.synchronize()
        self._finish()
        return True

    def block_current_stream(self):
        torch.cuda.current_stream().wait_event(self.event)
        return True

    def is_completed(self) -> bool:
        done = bool(self.event.query())
        if done:
            self._finish()
        return done


@dataclass
class ShardPlan:
    """How a flat bucket of ``numel`` elements is cut into ``world`` equal shards."""

    world: int
    numel: int

    @property
    def shard_len(self) -> int:
        return -(-self.numel // self.world)

    @property
    def padded(self) -> int:
        return self.shard_len * self.world


class ErrorFeedbackState:
    """Residuals of one bucket: stage 1 over the padded bucket, stage 2 over the shard
    this rank reduces.  fp32, allocated on first use, checkpointable."""

    def __init__(self):
        self.stage1: Optional[torch.Tensor] = None
        self.stage2: Optional[torch.Tensor] = None
        self.carry_over = False  # set by LowBitGroup.rebind: the world size is about to change

    def ensure(self, plan: ShardPlan, device, stage2: bool):
        if self.stage1 is not None and self.stage1.device != torch.device(device):
            # residuals restored from a checkpoint that was loaded on another device
            self.stage1 = self.stage1.to(device)
            if self.stage2 is not None:
                self.stage2 = self.stage2.to(device)
        if self.stage1 is None or self.stage1.numel() != plan.padded:
            fresh = torch.zeros(plan.padded, dtype=torch.float32, device=device)
            if self.carry_over and self.stage1 is not None:
                # same bucket, new shard plan: the stage-1 residual is per element of this
                # rank's own gradient and stays valid (the padding's residual is zero)
                n = min(plan.numel, int(self.stage1.numel()))
                fresh[:n] = self.stage1[:n]
            self.stage1 = fresh
            self.stage2 = None
        self.carry_over = False
        if stage2 and (self.stage2 is None or self.stage2.numel() != plan.shard_len):
            self.stage2 = torch.zeros(plan.shard_len, dtype=torch.float32, device=device)

    def state_dict(self):
        return {"stage1": self.stage1, "stage2": self.stage2}

    def load_state_dict(self, sd):
        self.stage1 = sd.get("stage1")
        self.stage2 = sd.get("stage2")


def _uses_single_tensor_alltoall(group) -> bool:
    """gloo implements only ``all_to_all_single``; NCCL (and test fakes) take lists."""
    try:
        return str(dist.get_backend(group)).lower() == "gloo"
    except Exception:
        return False


class _FlatLowBitAllReduce:
    """One flat low-bit all-reduce, split in the two halves the async Work needs.

    ``start()`` quantizes the shards and launches the two all-to-alls;
    ``finish()`` reduces, re-quantizes, gathers and writes the result back.
    """

    def __init__(self, owner: "LowBitGroup", flat: torch.Tensor, group,
                 ef: Optional[ErrorFeedbackState] = None, async_first: bool = False):
        self.owner = owner
        self.group = group
        self.flat_in = flat
        self.ef = ef
        self.world = dist.get_world_size(group)
        self.plan = ShardPlan(self.world, int(flat.numel()))
        self.single = _uses_single_tensor_alltoall(group)
        self.async_first = async_first
        self.works: list = []
        self.result: Optional[torch.Tensor] = None
        self._seed = owner._next_sr_seed()

    # -- first half --------------------------------------------------------------
    def start(self):
        o, plan = self.owner, self.plan
        flat = self.flat_in
        if plan.padded != plan.numel:
            flat = torch.nn.functional.pad(flat, (0, plan.padded - plan.numel))
        if self.ef is not None:
            self.ef.ensure(plan, flat.device, o.stage2_error_feedback)
            flat = flat.to(torch.float32) + self.ef.stage1
        S = plan.shard_len
        packed_out, scales_out = [], []
        stream1 = stage1_stream(dist.get_rank(self.group))
        for j in range(self.world):
            shard = flat[j * S:(j + 1) * S]
            p, s, _ = quantize_pack_tensor_blockwise(
                shard, o.bitwidth, block_size=o.block_size,
                stochastic_rounding=o.stochastic_rounding,
                sr_seed=self._seed, sr_offset=j * S, sr_stream=stream1)
            packed_out.append(p)
            scales_out.append(s)
            if self.ef is not None:
                sent = unpack_dequantize_tensor_blockwise(
                    p, s, o.bitwidth, S, block_size=o.block_size,
                    dtype=torch.float32, device=flat.device)
                self.ef.stage1[j * S:(j + 1) * S] = shard - sent

        if self.single:
            send_p, send_s = torch.stack(packed_out), torch.stack(scales_out)
            self.recv_packed, self.recv_scales = torch.empty_like(send_p), torch.empty_like(send_s)
            self.works = [
                dist.all_to_all_single(self.recv_packed, send_p, group=self.group,
                                       async_op=self.async_first),
                dist.all_to_all_single(self.recv_scales, send_s, group=self.group,
                                       async_op=self.async_first),
            ]
        else:
            self.recv_packed = [torch.empty_like(packed_out[0]) for _ in range(self.world)]
            self.recv_scales = [torch.empty_like(scales_out[0]) for _ in range(self.world)]
            self.works = [
                dist.all_to_all(self.recv_packed, packed_out, group=self.group,
                                async_op=self.async_first),
                dist.all_to_all(self.recv_scales, scales_out, group=self.group,
                                async_op=self.async_first),
            ]
        self._keep = (packed_out, scales_out)
        return self

    def wait_first(self):
        for w in self.works:
            if w is not None and hasattr(w, "wait"):
                w.wait()

    # -- second half -------------------------------------------------------------
    def reduce_and_requantize(self):
        o, S = self.owner, self.plan.shard_len
        dev = self.flat_in.device
        acc = torch.zeros(S, dtype=torch.float32, device=dev)
        for src in range(self.world):  # ascending source order is part of the wire contract
            acc.add_(unpack_dequantize_tensor_blockwise(
                self.recv_packed[src], self.recv_scales[src], o.bitwidth, S,
                block_size=o.block_size, dtype=torch.float32, device=dev))
        use_s2 = self.ef is not None and o.stage2_error_feedback
        if use_s2:
            acc = acc + self.ef.stage2
        rank = dist.get_rank(self.group)
        p, s, _ = quantize_pack_tensor_blockwise(
            acc, o.bitwidth, block_size=o.block_size,
            stochastic_rounding=o.stochastic_rounding,
            sr_seed=self._seed, sr_offset=rank * S, sr_stream=1)
        if use_s2:
            self.ef.stage2 = acc - unpack_dequantize_tensor_blockwise(
                p, s, o.bitwidth, S, block_size=o.block_size, dtype=torch.float32, device=dev)
        return p, s

    def gather(self, p, s, async_op=False):
        self.gathered_packed = [torch.empty_like(p) for _ in range(self.world)]
        self.gathered_scales = [torch.empty_like(s) for _ in range(self.world)]
        return [
            dist.all_gather(self.gathered_packed, p, group=self.group, async_op=async_op),
            dist.all_gather(self.gathered_scales, s, group=self.group, async_op=async_op),
        ]

    def restore(self) -> torch.Tensor:
        o, S = self.owner, self.plan.shard_len
        dev = self.flat_in.device
        parts = [
            unpack_dequantize_tensor_blockwise(
                self.gathered_packed[j], self.gathered_scales[j], o.bitwidth, S,
                block_size=o.block_size, dtype=torch.float32, device=dev)
            for j in range(self.world)
        ]
        self.result = torch.cat(parts)[: self.plan.numel]
        return self.result

    def finish(self) -> torch.Tensor:
        p, s = self.reduce_and_requantize()
        self.gather(p, s)
        return self.restore()


class _NativeLowBitAllReduceWork:
    """Async handle of the list-collective engine (reference ``api.py:91-310``).

    The two all-to-alls are in flight when the constructor returns.  The second half
    runs at ``wait()``; with ``BITSCOM_UNSAFE_FULL_ASYNC_CHAIN=1`` it is chained on the
    collectives' futures instead and may finish before ``wait()`` is called.
    """

    def __init__(self, owner: "LowBitGroup", tensor: torch.Tensor, group,
                 ef: Optional[ErrorFeedbackState] = None):
        self.owner = owner
        self.tensor = tensor
        self.completed = False
        self.final_future: torch.futures.Future = torch.futures.Future()
        self._wait_driven = True
        if tensor.numel() == 0:
            self._op = None
            self._done()
            return
        self._op = _FlatLowBitAllReduce(
            owner, tensor.contiguous().view(-1), group, ef=ef, async_first=True).start()
        if owner._full_async_chain_enabled():
            futs = [getattr(w, "get_future", lambda: None)() for w in self._op.works]
            if all(f is not None for f in futs):
                self._wait_driven = False
                torch.futures.collect_all(futs).then(self._guard(self._second_half_chained))

    def _guard(self, fn):
        def run(fut):
            try:
                fut.wait()
                fn()
            except BaseException as exc:  # surfaced at wait()
                self.final_future.set_exception(exc)
        return run

    def _second_half_chained(self):
        p, s = self._op.reduce_and_requantize()
        works = self._op.gather(p, s, async_op=True)
        futs = [getattr(w, "get_future", lambda: None)() for w in works]
        if all(f is not None for f in futs):
            torch.futures.collect_all(futs).then(self._guard(self._write_back))
        else:
            for w in works:
                w.wait()
            self._write_back()

    def _write_back(self):
        out = self._op.restore()
        self.tensor.copy_(out.view_as(self.tensor).to(self.tensor.dtype))
        self._done()

    def _done(self):
        self.completed = True
        self.final_future.set_result(True)

    def wait(self):
        if self._wait_driven and not self.completed:
            self._op.wait_first()
            p, s = self._op.reduce_and_requantize()
            for w in self._op.gather(p, s, async_op=True):
                w.wait()
            self._write_back()
        self.final_future.wait()
        return True

    def is_completed(self) -> bool:
        return self.completed

    def get_future(self):
        return self.final_future


# ----------------------------------------------------------------------------------
# LowBitGroup
# ----------------------------------------------------------------------------------

class LowBitGroup:
    """Low-bit communication primitives on top of a process group.

    Usage::

        import bitscom_b200 as bitscom
        dist.init_process_group("nccl")                # or bitscom.init(); backend="lowbit"
        group = bitscom.LowBitGroup(bitwidth=4, error_feedback=True)
        group.all_reduce(grad_bucket)                   # caller divides by world size

    Constructor arguments up to ``backend_allreduce`` are the reference's
    (``api.py:331-361``).  Added: ``error_feedback`` / ``stage2_error_feedback``
    (residuals kept per bucket, keyed by ``ef_key`` or the tensor's storage address),
    ``sr_seed`` (reproducible stochastic rounding), ``fused`` (None = use the fused
    sm_100a kernel whenever the tensor is on CUDA and the group fits one NVSwitch
    domain; False = never; True = require it).
    """

    def __init__(
        self,
        bitwidth: int = 4,
        process_group: Optional[dist.ProcessGroup] = None,
        simulate_quantization: bool = False,
        stochastic_rounding: bool = False,
        block_size: int = DEFAULT_BLOCK_SIZE,
        backend_allreduce: bool = False,
        *,
        error_feedback: bool = False,
        stage2_error_feedback: bool = False,
        sr_seed: Optional[int] = None,
        fused: Optional[bool] = None,
    ):
        if bitwidth not in SUPPORTED_BITWIDTHS:
            raise ValueError(
                f"bitwidth must be one of {SUPPORTED_BITWIDTHS}, got {bitwidth}"
            )
        if block_size <= 0:
            raise ValueError(f"block_size must be > 0, got {block_size}")
        self.bitwidth = bitwidth
        self.pg = process_group or dist.distributed_c10d._get_default_group()
        self.simulate_quantization = simulate_quantization
        self.stochastic_rounding = stochastic_rounding
        self.block_size = int(block_size)
        self.backend_allreduce = bool(backend_allreduce)
        self.error_feedback = bool(error_feedback or stage2_error_feedback)
        self.stage2_error_feedback = bool(stage2_error_feedback)
        self.sr_seed = sr_seed
        self.fused = fused
        self._sr_calls = 0
        self._ef_states: Dict[Hashable, ErrorFeedbackState] = {}
        self._fused_comms: Dict[int, object] = {}
        self.health = None  # optional utils.health.HealthMonitor, see attach_health

    # -- backend progress / scheduled handles (reference api.py:363-391) -----------
    def _backend_attr(self, name: str):
        """An extra method of the lowbit backend: on the group object itself, or on the
        CUDA backend behind a ``ProcessGroup`` wrapper."""
        fn = getattr(self.pg, name, None)
        if fn is not None:
            return fn
        getter = getattr(self.pg, "_get_backend", None)
        if getter is None:
            return None
        try:
            return getattr(getter(torch.device("cuda")), name, None)
        except Exception:
            return None

    def progress_lowbit(self, block: bool = False) -> bool:
        fn = self._backend_attr("progress_lowbit")
        return bool(fn(bool(block))) if fn is not None else False

    def schedule_lowbit_allreduce(self, tensor: torch.Tensor):
        fn = self._backend_attr("schedule_lowbit_allreduce")
        if fn is None:
            raise RuntimeError("lowbit backend does not expose schedule_lowbit_allreduce")
        return fn(tensor)

    def _launch_handle(self, handle, method: str, pg_method: str, label: str) -> bool:
        fn = getattr(handle, method, None)
        if fn is not None:
            return bool(fn())
        fn = self._backend_attr(pg_method)
        if fn is None:
            raise RuntimeError(f"lowbit backend does not expose {label}")
        return bool(fn(handle))

    def launch_lowbit_phase2(self, handle) -> bool:
        return self._launch_handle(handle, "launch_phase2",
                                   "launch_scheduled_lowbit_phase2", "launch_lowbit_phase2")

    def launch_lowbit_restore(self, handle) -> bool:
        return self._launch_handle(handle, "launch_restore",
                                   "launch_scheduled_lowbit_restore", "launch_lowbit_restore")

    # -- debugging aids ------------------------------------------------------------
    def _comm_debug_enabled(self) -> bool:
        return _env_flag("BITSCOM_COMM_DEBUG")

    def _full_async_chain_enabled(self) -> bool:
        return _env_flag("BITSCOM_UNSAFE_FULL_ASYNC_CHAIN")

    def _trace_explain_enabled(self) -> bool:
        return _env_flag("TRACE_EXPLAIN")

    def _safe_rank(self) -> int:
        try:
            return dist.get_rank(self.pg)
        except Exception:
            return -1

    def _comm_debug(self, message: str) -> None:
        if self._comm_debug_enabled():
            print(f"[bitscom-debug rank={self._safe_rank()} bitwidth={self.bitwidth}] "
                  f"{message}", flush=True)

    def _comm_evidence(self, action: str, message: str) -> None:
        if self._trace_explain_enabled():
            print(f"[trace-evidence rank={self._safe_rank()}] component=bitscom "
                  f"action={action} bitwidth={self.bitwidth} {message}", flush=True)

    # -- properties ----------------------------------------------------------------
    @property
    def rank(self) -> int:
        return dist.get_rank(self.pg)

    @property
    def world_size(self) -> int:
        return dist.get_world_size(self.pg)

    # -- state ---------------------------------------------------------------------
    def _next_sr_seed(self) -> Optional[int]:
        """Per-call seed; identical on every rank when ``sr_seed`` was given."""
        if self.sr_seed is None:
            return None
        self._sr_calls += 1
        return (int(self.sr_seed) * 0x9E3779B97F4A7C15 + self._sr_calls) & 0xFFFFFFFFFFFFFFFF

    def _ef_for(self, tensor: torch.Tensor, ef_key: Optional[Hashable]
                ) -> Optional[ErrorFeedbackState]:
        if not self.error_feedback:
            return None
        key = ef_key if ef_key is not None else (
            "addr", tensor.data_ptr(), int(tensor.numel()), str(tensor.dtype))
        state = self._ef_states.get(key)
        if state is None:
            state = self._ef_states[key] = ErrorFeedbackState()
        return state

    def residual_norms(self) -> Dict[Hashable, Tuple[float, float]]:
        """L2 norms of the stage-1 and stage-2 error-feedback residuals per bucket key (0.0
        where a stage is not in use).  A residual norm that keeps growing means the codec is
        too coarse for the gradients it is fed; the call synchronises the device."""
        out = {}
        for key, st in self._ef_states.items():
            n1 = float(st.stage1.float().norm().item()) if st.stage1 is not None else 0.0
            n2 = float(st.stage2.float().norm().item()) if st.stage2 is not None else 0.0
            out[key] = (n1, n2)
        return out

    def state_dict(self) -> dict:
        """Residuals and the stochastic-rounding call counter, for exact resume."""
        return {
            "sr_calls": self._sr_calls,
            "residuals": {k: v.state_dict() for k, v in self._ef_states.items()},
        }

    def load_state_dict(self, sd: dict) -> None:
        self._sr_calls = int(sd.get("sr_calls", 0))
        self._ef_states = {}
        for k, v in sd.get("residuals", {}).items():
            st = ErrorFeedbackState()
            st.load_state_dict(v)
            self._ef_states[k] = st

    def attach_health(self, monitor) -> None:
        """Consult ``monitor`` (a ``utils.health.HealthMonitor``) before every collective of
        this group: a peer that has left, failed or fallen silent then raises
        ``PeerLostError`` on the host, before anything is launched that would wait for it on
        the device.  The check reads state the monitor's thread keeps current; it costs no
        store round trip.  ``None`` detaches."""
        self.health = monitor

    def _precheck(self) -> None:
        monitor = getattr(self, "health", None)
        if monitor is not None:
            monitor.check()

    def rebind(self, process_group=None) -> None:
        """Point this group at another process group, typically the one built among the
        survivors after a rank was lost (``utils.health.shrink_process_group``).  Stage-1
        residuals are kept (they belong to this rank's own gradient elements) and re-laid
        out for the new shard plan on first use; stage-2 residuals belong to shards whose
        owners have changed and are dropped; fused communicators of the old group are
        released.  Call it between steps, on every surviving rank."""
        self.pg = process_group or dist.distributed_c10d._get_default_group()
        if any(self._fused_comms.values()):
            from .parallel.fused import FusedLowBitComm

            # communicators are cached per process-group object; the old group's symmetric
            # blocks map memory of peers that may be gone
            FusedLowBitComm.drop_cache()
        self._fused_comms = {}
        for st in self._ef_states.values():
            st.carry_over = True
            st.stage2 = None

    def check_status(self) -> None:
        """Raise ``FusedCollectiveError`` if a fused kernel launched through this group has
        given up on a bounded wait (a peer never arrived): the tensors of that collective
        hold partial results.  Reads the communicators' host-mapped status records; no device
        synchronisation, so a kernel still running is not waited for."""
        for comm in self._fused_comms.values():
            if comm and comm.native.handle is not None:
                comm.check_status()

    def close(self) -> None:
        """Collective: release the fused communicators this group has used (see
        ``FusedLowBitComm.close``).  Every rank of the group calls it, between steps, before
        ``destroy_process_group``; the group falls back to creating a fresh communicator if it
        is used again.  ``bitscom_b200.shutdown()`` does this for every group at once."""
        comms = [c for c in self._fused_comms.values() if c]
        self._fused_comms = {}
        for comm in comms:
            comm.close()

    def check_agreement(self, tensor: torch.Tensor) -> None:
        """Collective debugging aid: raises ``RuntimeError`` on every rank unless all ranks
        hold bit-identical copies of ``tensor``.  A low-bit all-reduce must leave the same bits
        everywhere (every rank dequantizes the same packed shards); a difference means a shard
        was damaged in transit or the ranks ran with different options.  Costs one pass over
        the tensor and an all-gather of two integers."""
        flat = tensor.detach().contiguous().view(-1)
        words = flat.view({1: torch.uint8, 2: torch.int16, 4: torch.int32,
                           8: torch.int64}[flat.element_size()]).to(torch.int64)
        weights = (torch.arange(words.numel(), device=words.device, dtype=torch.int64)
                   % 65521) + 1
        digest = torch.stack([words.sum(), (words * weights).sum(),
                              torch.tensor(words.numel(), device=words.device)])
        everyone = [torch.empty_like(digest) for _ in range(self.world_size)]
        dist.all_gather(everyone, digest, group=self.pg)
        mine = everyone[0]
        bad = [r for r, d in enumerate(everyone) if not torch.equal(d, mine)]
        if bad:
            raise RuntimeError(f"ranks disagree on the tensor's bits: ranks {bad} differ from "
                               "rank 0")

    def check_consistency(self) -> None:
        """Collective: every rank of the group must have been built with the same codec
        options, otherwise packed shards of different sizes would meet on the wire.
        Raises ``RuntimeError`` on every rank when they differ."""
        mine = (self.bitwidth, self.block_size, self.stochastic_rounding, self.error_feedback,
                self.stage2_error_feedback, self.sr_seed)
        everyone = [None] * self.world_size
        dist.all_gather_object(everyone, mine, group=self.pg)
        if any(o != everyone[0] for o in everyone):
            raise RuntimeError(
                "LowBitGroup options differ between ranks: "
                + "; ".join(f"rank {r}: {o}" for r, o in enumerate(everyone)))

    # -- engine selection ------------------------------------------------------------
    def _fused_comm(self, tensor: torch.Tensor, group):
        """The fused communicator of ``group`` if this tensor can use it, else None."""
        if self.fused is False or not tensor.is_cuda:
            if self.fused is True and not tensor.is_cuda:
                raise RuntimeError("fused=True needs CUDA tensors")
            return None
        comm = self._fused_comms.get(id(group))
        if comm and comm.native.handle is None:
            comm = None  # closed (``close`` / ``bitscom_b200.shutdown``): build a fresh one
        if comm is None:
            from .parallel.fused import FusedLowBitComm, FusedUnavailable

            try:
                comm = FusedLowBitComm.for_group(group, tensor.device)
            except FusedUnavailable:
                # benign: several hosts / too many ranks.  A missing native library is not
                # caught here: on a GPU machine it must fail loudly.
                if self.fused is True:
                    raise
                comm = False
            self._fused_comms[id(group)] = comm
        if comm is False or not comm.supports(tensor.dtype, self.bitwidth, self.block_size):
            if self.fused is True:
                raise RuntimeError("fused low-bit path unavailable for this configuration")
            return None
        return comm

    # -- all_reduce ----------------------------------------------------------------
    def all_reduce(
        self,
        tensor: torch.Tensor,
        op: dist.ReduceOp = dist.ReduceOp.SUM,
        async_op: bool = False,
        local_group: Optional[dist.ProcessGroup] = None,
        inter_group: Optional[dist.ProcessGroup] = None,
        chunk_size: Optional[int] = None,
        local_quantize: bool = False,
        ef_key: Optional[Hashable] = None,
    ):
        """Sum ``tensor`` over the group in place (the caller divides by world size).

        Low-bit only for ``bitwidth < 8``, ``SUM`` and more than one rank; otherwise a
        dense all-reduce (preceded by a quantize round trip when
        ``simulate_quantization`` is set).  Returns ``None`` when synchronous, a
        Work-like object with ``wait()`` otherwise.
        """
        self._precheck()
        if self._comm_debug_enabled():
            self._comm_debug(
                f"all_reduce entry numel={int(tensor.numel())} dtype={tensor.dtype} "
                f"device={tensor.device} op={op} async_op={async_op} "
                f"local_group={local_group is not None} inter_group={inter_group is not None} "
                f"local_quantize={local_quantize} chunk_size={chunk_size}")

        if self.backend_allreduce:
            self._comm_debug("path=backend_lowbit_allreduce")
            return self._dense(tensor, op, self.pg, async_op)

        lowbit_op = self.bitwidth < 8 and op == dist.ReduceOp.SUM

        if local_group is not None and inter_group is None and lowbit_op:
            if not local_quantize:
                self._comm_debug("path=local_group_dense")
                return self._dense(tensor, op, local_group, async_op)
            self._comm_debug("path=local_group_lowbit")
            if async_op:
                return self._lowbit_allreduce_via_alltoall_async(tensor, local_group, ef_key)
            self._lowbit_allreduce_via_alltoall_into_(tensor, local_group, ef_key)
            return None

        if self._should_use_pipeline_a(op, local_group, inter_group):
            self._comm_debug("path=hierarchical_lowbit_pipeline_a")
            # ef_key only when given: callers' stand-ins for this method keep the reference's
            # signature
            extra = {} if ef_key is None else {"ef_key": ef_key}
            self._hierarchical_lowbit_allreduce_pipeline_a(
                tensor, local_group=local_group, inter_group=inter_group,
                chunk_size=chunk_size, local_quantize=local_quantize, **extra)
            # pipeline-A runs its ordered local/inter/finalize phases to completion
            return _ImmediateWork() if async_op else None

        if self._should_use_lowbit_path(op):
            self._comm_debug("path=flat_lowbit_alltoall")
            if async_op:
                return self._lowbit_allreduce_via_alltoall_async(tensor, self.pg, ef_key)
            self._lowbit_allreduce_via_alltoall_into_(tensor, self.pg, ef_key)
            return None

        if self.simulate_quantization:
            self._comm_debug("path=dense_with_quantization_simulation")
            tensor.copy_(roundtrip_tensor(tensor, self.bitwidth))
        else:
            self._comm_debug("path=dense_all_reduce")
        return self._dense(tensor, op, self.pg, async_op)

    @staticmethod
    def _dense(tensor, op, group, async_op):
        work = dist.all_reduce(tensor, op=op, group=group, async_op=True)
        if async_op:
            return work
        work.wait()
        return None

    def all_reduce_stream(
        self,
        tensor: torch.Tensor,
        *,
        stream: "torch.cuda.Stream",
        op: dist.ReduceOp = dist.ReduceOp.SUM,
        group: Optional[dist.ProcessGroup] = None,
        post_scale: float = 1.0,
        ef_key: Optional[Hashable] = None,
        max_ctas: Optional[int] = None,
    ):
        """Enqueue the whole all-reduce on ``stream`` and return an event-backed handle
        (``wait`` / ``block_current_stream`` / ``is_completed``); ``post_scale`` is
        applied to the result on the same stream (reference ``api.py:577-629``).
        ``max_ctas`` caps the fused kernel's grid for launches that overlap other kernels."""
        self._precheck()
        pg = group or self.pg
        lowbit = op == dist.ReduceOp.SUM and self._should_use_lowbit_path_for_group(op, pg)

        if not tensor.is_cuda:
            if lowbit:
                self._lowbit_allreduce_via_alltoall_into_(tensor, pg, ef_key)
            else:
                dist.all_reduce(tensor, op=op, group=pg)
            if post_scale != 1.0:
                tensor.mul_(post_scale)
            return _ImmediateWork()

        stream.wait_stream(torch.cuda.current_stream(tensor.device))
        if not lowbit:
            with torch.cuda.stream(stream):
                work = dist.all_reduce(tensor, op=op, group=pg, async_op=True)
                self._block_work_on_current_stream(work)
                if post_scale != 1.0:
                    tensor.mul_(post_scale)
                done = torch.cuda.Event()
                done.record(stream)
            return _CudaEventWork(done)
        return self._lowbit_allreduce_via_alltoall_stream_(
            tensor, pg, stream=stream, post_scale=post_scale, ef_key=ef_key,
            max_ctas=max_ctas)

    def _should_use_lowbit_path(self, op) -> bool:
        return self.bitwidth < 8 and self.world_size > 1 and op == dist.ReduceOp.SUM

    def _should_use_lowbit_path_for_group(self, op, group) -> bool:
        return (self.bitwidth < 8 and dist.get_world_size(group) > 1
                and op == dist.ReduceOp.SUM)

    @staticmethod
    def _block_work_on_current_stream(work) -> None:
        """Order the current stream after ``work`` without blocking the host when the
        Work supports it."""
        blocker = getattr(work, "block_current_stream", None)
        with _timing.span("block_work_on_current_stream"):
            if blocker is not None:
                blocker()
            else:
                work.wait()

    def _should_use_pipeline_a(self, op, local_group, inter_group) -> bool:
        return (local_group is not None and inter_group is not None
                and self.bitwidth < 8 and op == dist.ReduceOp.SUM)

    def _split_flat_chunks(self, flat: torch.Tensor, chunk_size: int) -> List[torch.Tensor]:
        if chunk_size <= 0:
            raise ValueError(f"chunk_size must be > 0, got {chunk_size}")
        return list(flat.split(chunk_size))

    def _should_use_dual_stream_pipeline(self, *, is_cuda: bool, local_size: int,
                                         global_size: int) -> bool:
        # two streams only pay off when an inter-node stage exists to overlap with
        return is_cuda and local_size < global_size

    # -- flat low-bit all-reduce -----------------------------------------------------
    def _lowbit_allreduce_via_alltoall_group(self, flat: torch.Tensor, group,
                                             ef: Optional[ErrorFeedbackState] = None
                                             ) -> torch.Tensor:
        """Returns the reduced bucket as fp32 ``[numel]`` (list / single-tensor engines)."""
        if flat.numel() == 0:
            return flat
        with _timing.span("lowbit_allreduce_host_engine"):
            world = dist.get_world_size(group)
            shard = -(-int(flat.numel()) // world)
            wire = (shard * self.bitwidth + 7) // 8 + 2 * -(-shard // self.block_size)
            _timing.add("host_engine_calls")
            _timing.add("host_engine_payload_bytes", flat.numel() * flat.element_size())
            _timing.add("host_engine_wire_bytes", 2 * (world - 1) * wire)
            return _FlatLowBitAllReduce(self, flat, group, ef=ef).start().finish()

    def _lowbit_allreduce_via_alltoall(self, tensor: torch.Tensor) -> None:
        self._lowbit_allreduce_via_alltoall_into_(tensor, self.pg)

    def _lowbit_allreduce_via_alltoall_into_(self, tensor: torch.Tensor, group,
                                             ef_key: Optional[Hashable] = None) -> None:
        ef = self._ef_for(tensor, ef_key)
        comm = self._fused_comm(tensor, group) if tensor.is_contiguous() else None
        if comm is not None:
            comm.all_reduce(
                tensor, bitwidth=self.bitwidth, block_size=self.block_size,
                stochastic=self.stochastic_rounding, seed=self._next_sr_seed(), ef=ef,
                stage2=self.stage2_error_feedback)
            return
        flat = tensor.contiguous().view(-1)
        restored = self._lowbit_allreduce_via_alltoall_group(flat, group, ef) if ef is not None \
            else self._lowbit_allreduce_via_alltoall_group(flat, group)
        tensor.copy_(restored.view_as(tensor).to(dtype=tensor.dtype))

    def _lowbit_allreduce_via_alltoall_async(self, tensor: torch.Tensor, group,
                                             ef_key: Optional[Hashable] = None):
        ef = self._ef_for(tensor, ef_key)
        comm = self._fused_comm(tensor, group) if tensor.is_contiguous() else None
        if comm is not None:
            return comm.all_reduce(
                tensor, bitwidth=self.bitwidth, block_size=self.block_size,
                stochastic=self.stochastic_rounding, seed=self._next_sr_seed(), ef=ef,
                stage2=self.stage2_error_feedback, async_op=True)
        return _NativeLowBitAllReduceWork(self, tensor, group, ef=ef)

    def _lowbit_allreduce_via_alltoall_stream_(self, tensor: torch.Tensor, group, *,
                                               stream, post_scale: float,
                                               ef_key: Optional[Hashable] = None,
                                               max_ctas: Optional[int] = None):
        """Stream-ordered variant; the caller has already ordered ``stream`` after the
        producer of ``tensor``."""
        done = torch.cuda.Event()
        if tensor.numel() == 0:
            done.record(stream)
            return _CudaEventWork(done)
        ef = self._ef_for(tensor, ef_key)
        comm = self._fused_comm(tensor, group) if tensor.is_contiguous() else None
        with torch.cuda.stream(stream):
            if comm is not None:
                comm.all_reduce(
                    tensor, bitwidth=self.bitwidth, block_size=self.block_size,
                    stochastic=self.stochastic_rounding, seed=self._next_sr_seed(), ef=ef,
                    stage2=self.stage2_error_feedback, post_scale=post_scale,
                    max_ctas=max_ctas)
                done.record(stream)
                return _CudaEventWork(done, on_complete=comm.check_status)
            keep: list = []
            op = _FlatLowBitAllReduce(self, tensor.contiguous().view(-1), group, ef=ef,
                                      async_first=True)
            with torch.profiler.record_function("bitscom:_lowbit_stream:all_to_all"):
                op.start()
                for w in op.works:
                    self._block_work_on_current_stream(w)
            p, s = op.reduce_and_requantize()
            with torch.profiler.record_function("bitscom:_lowbit_stream:all_gather"):
                for w in op.gather(p, s, async_op=True):
                    self._block_work_on_current_stream(w)
            out = op.restore()
            tensor.copy_(out.view_as(tensor).to(tensor.dtype))
            if post_scale != 1.0:
                tensor.mul_(post_scale)
            keep.append(op)
            done.record(stream)
        return _CudaEventWork(done, keepalive=keep)

    # -- hierarchical pipeline-A -------------------------------------------------------
    def _hierarchical_lowbit_allreduce_pipeline_a(self, tensor: torch.Tensor, *, local_group,
                                                  inter_group, chunk_size: Optional[int],
                                                  local_quantize: bool,
                                                  ef_key: Optional[Hashable] = None) -> None:
        from .parallel.pipeline_a import run_pipeline_a

        run_pipeline_a(self, tensor, local_group=local_group, inter_group=inter_group,
                       chunk_size=chunk_size, local_quantize=local_quantize, ef_key=ef_key)

    # -- passthrough collectives (reference api.py:1460-1505) ---------------------------
    def _maybe_simulate(self, tensor: torch.Tensor) -> torch.Tensor:
        if self.simulate_quantization:
            return roundtrip_tensor(tensor, self.bitwidth)
        return tensor

    def all_gather(self, tensor_list: List[torch.Tensor], tensor: torch.Tensor,
                   async_op: bool = False):
        work = dist.all_gather(tensor_list, self._maybe_simulate(tensor), group=self.pg,
                               async_op=True)
        if async_op:
            return work
        work.wait()
        return None

    def reduce_scatter(self, output: torch.Tensor, input_list: List[torch.Tensor],
                       op: dist.ReduceOp = dist.ReduceOp.SUM, async_op: bool = False):
        if self.simulate_quantization:
            input_list = [roundtrip_tensor(t, self.bitwidth) for t in input_list]
        work = dist.reduce_scatter(output, input_list, op=op, group=self.pg, async_op=True)
        if async_op:
            return work
        work.wait()
        return None

    def broadcast(self, tensor: torch.Tensor, src: int = 0, async_op: bool = False):
        if self.simulate_quantization and self.rank == src:
            tensor.copy_(roundtrip_tensor(tensor, self.bitwidth))
        work = dist.broadcast(tensor, src=src, group=self.pg, async_op=True)
        if async_op:
            return work
        work.wait()
        return None

    # -- low-bit sharded collectives (not in the reference's Python API) ---------------
    def reduce_scatter_lowbit(self, output: torch.Tensor, input: torch.Tensor, *,
                              ef_key: Optional[Hashable] = None, async_op: bool = False):
        """Low-bit reduce-scatter of a flat ``[W * n]`` input into ``output [n]``: the
        first half of the all-reduce (quantize, exchange, ordered fp32 sum)."""
        from .parallel.sharded import lowbit_reduce_scatter

        self._precheck()
        return lowbit_reduce_scatter(self, output, input, ef_key=ef_key, async_op=async_op)

    def all_gather_lowbit(self, output: torch.Tensor, input: torch.Tensor, *,
                          ef_key: Optional[Hashable] = None, async_op: bool = False):
        """Low-bit all-gather of ``input [n]`` into a flat ``[W * n]`` output: the second
        half of the all-reduce (quantize own shard, gather, dequantize)."""
        from .parallel.sharded import lowbit_all_gather

        self._precheck()
        return lowbit_all_gather(self, output, input, ef_key=ef_key, async_op=async_op)

    # -- compress / decompress ----------------------------------------------------------
    def compress(self, tensor: torch.Tensor) -> CompressedTensor:
        return compress_tensor(tensor, self.bitwidth)

    def decompress(self, compressed: CompressedTensor, *, dtype: Optional[torch.dtype] = None,
                   device: Optional[torch.device] = None) -> torch.Tensor:
        return decompress_tensor(compressed, dtype=dtype, device=device)
