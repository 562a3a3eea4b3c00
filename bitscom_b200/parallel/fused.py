"""Fused low-bit collectives over symmetric memory (Python side).

``FusedLowBitComm`` owns one native communicator (``csrc/symm.cu``): a block of device
memory per rank with receive and gather regions, mapped into every peer through CUDA
IPC, plus the flag/arrival words the fused sm_100a kernel synchronises on
(``csrc/fused_collectives.cu``).  ``all_reduce`` / ``reduce_scatter`` / ``all_gather``
enqueue ONE kernel per bucket chunk on the current stream; nothing else touches the
wire.  It replaces the reference's chain of pack kernels and NCCL send/recv groups
(``cpp/src/process_group_lowbit.cc:641-1293``).

``EmulatedWorld`` wires W communicators on ONE device and plays all ranks in a single
cooperative launch, which lets the whole protocol be tested on one GPU.
"""

from __future__ import annotations

import ctypes
import os
import socket
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from ..ops import _native
from ..ops._native import DTYPE_CODE, NativeError, check
from ..quantization import sr_key, stage1_stream
from ..utils import timing as _timing

MODE_ALL_REDUCE, MODE_REDUCE_SCATTER, MODE_ALL_GATHER = 0, 1, 2
FUSED_BITS = (1, 2, 4, 8, 12)

_STATUS_TEXT = {
    1: "a peer never announced its packed shards (phase-1 flags)",
    2: "a peer never announced its reduced shard (phase-2 flags)",
}


class CollArgs(ctypes.Structure):
    _fields_ = [
        ("inp", ctypes.c_void_p), ("out", ctypes.c_void_p),
        ("res1", ctypes.c_void_p), ("res2", ctypes.c_void_p),
        ("n", ctypes.c_longlong), ("S", ctypes.c_longlong),
        ("dtype", ctypes.c_int), ("bits", ctypes.c_int), ("block", ctypes.c_int),
        ("mode", ctypes.c_int), ("stochastic", ctypes.c_int),
        ("key1", ctypes.c_uint), ("key2", ctypes.c_uint),
        ("post_scale", ctypes.c_float), ("max_ctas", ctypes.c_int),
        ("reserved", ctypes.c_int),
    ]


_lib = None


def _get():
    global _lib
    if _lib is None:
        lib = _native.load("bcom_comm")
        if lib is not None:
            vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
            lib.bcom_comm_create.argtypes = [ci, ci, ctypes.c_size_t, ctypes.POINTER(vp)]
            lib.bcom_comm_create_external.argtypes = [ci, ci, ctypes.c_size_t,
                                                      ctypes.POINTER(vp), vp, ctypes.POINTER(vp)]
            lib.bcom_comm_block_bytes.argtypes = [ctypes.c_size_t]
            lib.bcom_comm_block_bytes.restype = ctypes.c_size_t
            lib.bcom_comm_multicast_base.argtypes = [vp]
            lib.bcom_comm_multicast_base.restype = vp
            lib.bcom_comm_destroy.argtypes = [vp]
            lib.bcom_comm_close_peers.argtypes = [vp]
            lib.bcom_comm_check_canaries.argtypes = [vp, ctypes.POINTER(ll)]
            lib.bcom_comm_ipc_handle.argtypes = [vp, vp]
            lib.bcom_comm_open_peers.argtypes = [vp, vp]
            lib.bcom_comm_set_peer.argtypes = [vp, ci, vp]
            lib.bcom_comm_local_base.argtypes = [vp]
            lib.bcom_comm_local_base.restype = vp
            lib.bcom_comm_region_bytes.argtypes = [vp]
            lib.bcom_comm_region_bytes.restype = ctypes.c_size_t
            lib.bcom_comm_max_chunk.argtypes = [vp, ci, ci]
            lib.bcom_comm_max_chunk.restype = ll
            lib.bcom_comm_status.argtypes = [vp, ctypes.POINTER(ctypes.c_uint * 8)]
            lib.bcom_comm_status_host.argtypes = [vp]
            lib.bcom_comm_status_host.restype = vp
            lib.bcom_comm_phase_times.argtypes = [vp, ctypes.POINTER(ctypes.c_ulonglong * 6)]
            lib.bcom_comm_reset.argtypes = [vp, vp]
            lib.bcom_comm_set_timeout_ms.argtypes = [vp, ctypes.c_double]
            lib.bcom_comm_set_ll_max_bytes.argtypes = [vp, ctypes.c_longlong]
            lib.bcom_comm_epoch.argtypes = [vp]
            lib.bcom_comm_epoch.restype = ctypes.c_ulonglong
            lib.bcom_collective.argtypes = [vp, ctypes.POINTER(CollArgs), vp]
            lib.bcom_collective_emulated.argtypes = [
                ctypes.POINTER(vp), ctypes.POINTER(CollArgs), ci, vp]
            lib.bcom_collective_supported.argtypes = [ci, ci, ci]
        _lib = lib if lib is not None else False
    return _lib or None


def available() -> bool:
    return _native.cuda_present() and _get() is not None


def _flag(name: str) -> bool:
    return os.environ.get(name, "0").strip().lower() in ("1", "true", "yes", "on")


def default_region_bytes() -> int:
    # 256 MiB per region (an eighth of it is kept for the small-bucket form): a 1 GB fp32 bucket
    # at 8 ranks is one launch (three with 64 MiB) and a Llama-7B layer's gradients at 4 ranks
    # one (two); each launch has a fixed cost of about 60 us
    return int(float(os.environ.get("BITSCOM_SYMM_MB", "256")) * (1 << 20))


def default_timeout_ms() -> float:
    return float(os.environ.get("BITSCOM_TIMEOUT_MS", "30000"))


class FusedCollectiveError(RuntimeError):
    pass


class FusedUnavailable(RuntimeError):
    """The group cannot use the fused path for a benign reason (ranks on several hosts, too
    many ranks); callers fall back to NCCL collectives.  A missing or broken native library is
    NOT this: it raises ``NativeError``."""


def _keys(stochastic: bool, seed: Optional[int], rank: int):
    if not stochastic:
        return 0, 0
    if seed is None:
        from ..ops.codec import fresh_seed

        seed = fresh_seed()
    return sr_key(seed, stage1_stream(rank)), sr_key(seed, 1)


def _args(inp, out, res1, res2, n, S, dtype, bits, block, mode, stochastic, seed,
          post_scale, max_ctas, rank) -> CollArgs:
    k1, k2 = _keys(stochastic, seed, rank)
    return CollArgs(
        inp=inp.data_ptr(), out=out.data_ptr(),
        res1=0 if res1 is None else res1.data_ptr(),
        res2=0 if res2 is None else res2.data_ptr(),
        n=int(n), S=int(S), dtype=DTYPE_CODE[dtype], bits=int(bits), block=int(block),
        mode=mode, stochastic=int(bool(stochastic)), key1=k1, key2=k2,
        post_scale=float(post_scale), max_ctas=int(max_ctas), reserved=0)


def traffic_bytes(args: CollArgs, world: int):
    """(payload, wire) bytes of one collective on one rank: payload is the tensor as the
    caller sees it, wire the packed codes and fp16 block scales this rank stores into its
    peers' memory over NVLink (both halves for an all-reduce, one for the other modes)."""
    elem = {0: 4, 1: 2, 2: 2}[int(args.dtype)]
    shard = int(args.S)
    shard_wire = (shard * int(args.bits) + 7) // 8 + 2 * -(-shard // int(args.block))
    phases = 2 if int(args.mode) == MODE_ALL_REDUCE else 1
    return int(args.n) * elem, phases * (world - 1) * shard_wire


class _NativeComm:
    """Owner of one ``BcomComm*``."""

    def __init__(self, rank: int, world: int, region_bytes: int, device: torch.device,
                 external_bases: Optional[List[int]] = None, multicast_base: int = 0):
        """``external_bases``: adopt blocks mapped by somebody else (one address per rank)
        instead of allocating one and exchanging CUDA IPC handles; ``multicast_base``: the
        NVLink multicast mapping of those blocks (0 = none)."""
        self.lib = _get()
        if self.lib is None:
            raise NativeError("fused collectives need the bcom_comm library and a GPU")
        self.rank, self.world, self.device = rank, world, torch.device(device)
        self.external = external_bases is not None
        handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            if self.external:
                bases = (ctypes.c_void_p * world)(*[int(b) for b in external_bases])
                check(self.lib.bcom_comm_create_external(
                    rank, world, region_bytes, bases, ctypes.c_void_p(int(multicast_base)),
                    ctypes.byref(handle)), "bcom_comm_create_external", launches=0)
            else:
                check(self.lib.bcom_comm_create(rank, world, region_bytes,
                                                ctypes.byref(handle)), "bcom_comm_create", launches=0)
        self.handle = handle
        # live view of the pinned status record: word 0 != 0 means a kernel gave up
        self._status_view = (ctypes.c_uint * 8).from_address(
            self.lib.bcom_comm_status_host(handle))

    def failed(self) -> bool:
        return self._status_view[0] != 0

    def ipc_handle(self) -> bytes:
        buf = ctypes.create_string_buffer(64)
        check(self.lib.bcom_comm_ipc_handle(self.handle, buf), "cudaIpcGetMemHandle", launches=0)
        return buf.raw

    def open_peers(self, handles: List[bytes]) -> None:
        blob = ctypes.create_string_buffer(b"".join(handles), 64 * self.world)
        with torch.cuda.device(self.device):
            check(self.lib.bcom_comm_open_peers(self.handle, blob), "cudaIpcOpenMemHandle", launches=0)

    def status(self) -> List[int]:
        out = (ctypes.c_uint * 8)()
        self.lib.bcom_comm_status(self.handle, ctypes.byref(out))
        return list(out)

    def phase_times_us(self) -> dict:
        """Where the LAST kernel of this communicator spent its time, from the time stamps its
        first CTA wrote at the phase boundaries (microseconds; read after a synchronize):
        ``phase1`` quantize + push, ``wait1`` until every rank's phase-1 flag was seen,
        ``phase2`` reduce + re-quantize + push, ``wait2``, ``phase3`` dequantize + write."""
        t = (ctypes.c_ulonglong * 6)()
        self.lib.bcom_comm_phase_times(self.handle, ctypes.byref(t))
        names = ("phase1", "wait1", "phase2", "wait2", "phase3")
        out = {n: max(0, int(t[i + 1]) - int(t[i])) / 1e3 for i, n in enumerate(names)}
        out["total"] = max(0, int(t[5]) - int(t[0])) / 1e3
        return out

    def reset(self) -> None:
        with torch.cuda.device(self.device):
            check(self.lib.bcom_comm_reset(
                self.handle, ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)),
                "bcom_comm_reset", launches=0)

    def check_canaries(self) -> None:
        """Debugging aid (synchronises the device): raise if a store landed outside the
        regions of this rank's block, in the guard bytes in front of or behind them."""
        bad = ctypes.c_longlong(-1)
        check(self.lib.bcom_comm_check_canaries(self.handle, ctypes.byref(bad)),
              "bcom_comm_check_canaries", launches=0)
        if bad.value >= 0:
            raise FusedCollectiveError(
                f"rank {self.rank}: guard bytes of the symmetric block were overwritten at "
                f"offset {bad.value}")

    def close_peers(self) -> None:
        """Wait for this rank's kernels and unmap the peers' blocks (first step of an orderly
        teardown; the communicator cannot launch afterwards)."""
        if self.handle:
            check(self.lib.bcom_comm_close_peers(self.handle), "bcom_comm_close_peers", launches=0)

    def close(self) -> None:
        if self.handle:
            self.lib.bcom_comm_destroy(self.handle)
            self.handle = None


def _describe(status: List[int]) -> str:
    code = status[0]
    seen = status[4] | (status[5] << 32)
    want = status[6] | (status[7] << 32)
    return (f"fused low-bit collective gave up: {_STATUS_TEXT.get(code, f'code {code}')}; "
            f"rank {status[3]} waited on peer {status[2]}, saw epoch {seen}, wanted {want}")


class FusedLowBitComm:
    """Fused collectives for one process group on one device."""

    _cache: Dict[tuple, "FusedLowBitComm"] = {}

    def __init__(self, group, device: torch.device, region_bytes: Optional[int] = None,
                 timeout_ms: Optional[float] = None):
        self.group = group
        self.device = torch.device(device)
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        if self.world > 16:
            raise FusedUnavailable("fused collectives support at most 16 ranks")
        hosts: List[Optional[str]] = [None] * self.world
        dist.all_gather_object(hosts, socket.gethostname(), group=group)
        if len(set(hosts)) != 1:
            raise FusedUnavailable("fused collectives need all ranks on one NVSwitch domain")
        region = region_bytes or default_region_bytes()
        self.multicast = False
        self._symm = None  # keeps torch's symmetric allocation alive
        self.native = self._try_multicast_comm(region) if _flag("BITSCOM_NVLS") else None
        if self.native is None:
            self.native = _NativeComm(self.rank, self.world, region, self.device)
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, self.native.ipc_handle(), group=group)
            self.native.open_peers(handles)
        self.native.lib.bcom_comm_set_timeout_ms(self.native.handle,
                                                 timeout_ms or default_timeout_ms())
        # BITSCOM_LL_MAX_MB: largest all-reduce (MiB of the tensor) that runs as one
        # flag-in-data launch, at four bytes per element; unset: the library's default (64), 0: never
        if os.environ.get("BITSCOM_LL_MAX_MB", "").strip():
            self.set_ll_max_bytes(int(float(os.environ["BITSCOM_LL_MAX_MB"]) * (1 << 20)))
        self.side_stream = torch.cuda.Stream(device=self.device)
        self.max_ctas = int(os.environ.get("BITSCOM_MAX_CTAS", "0"))
        self.launches = 0
        # every rank has mapped every peer before anybody launches
        dist.barrier(group=group, device_ids=[self.device.index]
                     if dist.get_backend(group) == "nccl" else None)

    def _try_multicast_comm(self, region_bytes: int) -> Optional[_NativeComm]:
        """Blocks allocated through torch symmetric memory, which also maps them through an
        NVLink multicast object when the fabric supports it: the all-gather half of the 4- and
        8-bit collectives then sends each packed group with ONE multimem store that NVSwitch
        replicates, instead of one store per peer.  Opt-in (``BITSCOM_NVLS=1``): a rank that dies
        while its memory is bound to a multicast object can fault its peers, so failure tests
        and fault-tolerant jobs should stay on the plain peer-store path.  Returns ``None``,
        on every rank alike, when any rank could not set it up."""
        lib = _get()
        comm, hdl, buf = None, None, None
        try:
            import torch.distributed._symmetric_memory as symm_mem

            nbytes = int(lib.bcom_comm_block_bytes(region_bytes))
            buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
            hdl = symm_mem.rendezvous(buf, group=self.group)
            mc = int(hdl.multicast_ptr) if getattr(hdl, "has_multicast_support", False) else 0
            bases = [int(p) for p in hdl.buffer_ptrs]
            ok = mc != 0 and len(bases) == self.world
        except Exception:  # symmetric memory not available for this group / device
            ok = False
        votes: List[Optional[bool]] = [None] * self.world
        dist.all_gather_object(votes, bool(ok), group=self.group)
        if not all(votes):
            return None
        comm = _NativeComm(self.rank, self.world, region_bytes, self.device,
                           external_bases=bases, multicast_base=mc)
        self._symm = (buf, hdl)
        self.multicast = True
        return comm

    @classmethod
    def for_group(cls, group, device) -> "FusedLowBitComm":
        key = (id(group), torch.device(device).index)
        comm = cls._cache.get(key)
        if comm is None:
            comm = cls._cache[key] = cls(group, device)
        return comm

    @classmethod
    def drop_cache(cls) -> None:
        """Local, non-collective release of every cached communicator: for a rank whose peers
        may be gone (recovery after a lost rank).  Jobs that end normally use ``close_all``."""
        for comm in cls._cache.values():
            comm.native.close()
        cls._cache.clear()

    def _barrier(self) -> None:
        dist.barrier(group=self.group, device_ids=[self.device.index]
                     if dist.get_backend(self.group) == "nccl" else None)

    def close(self) -> None:
        """Collective, orderly teardown; every rank of the group calls it, between steps:

        1. wait for this rank's kernels, then a barrier: no rank has a kernel in flight that
           stores into a peer's block;
        2. unmap the peers' blocks, then a barrier: no rank maps this rank's block any more;
        3. free the block.

        Freeing a block that a peer still maps is undefined behaviour of CUDA IPC, and a
        process that exits with mappings and exported blocks alive leaves their release to the
        driver's process teardown, in whatever order the ranks happen to die; this makes the
        order explicit.  Idempotent."""
        if self.native is None or self.native.handle is None:
            return
        torch.cuda.synchronize(self.device)
        self._barrier()
        if not self.native.external:
            self.native.close_peers()
        self._barrier()
        self.native.close()
        self._symm = None
        for key, comm in list(self._cache.items()):
            if comm is self:
                del self._cache[key]

    @classmethod
    def close_all(cls) -> None:
        """``close()`` for every cached communicator, in an order that is the same on every
        rank (by the groups' global ranks), so that ranks that share several groups meet in
        the same barriers in the same order."""
        def order(comm):
            try:
                return tuple(dist.get_process_group_ranks(comm.group))
            except Exception:
                return ()
        for comm in sorted(cls._cache.values(), key=order):
            comm.close()
        cls._cache.clear()

    # -- capabilities / status --------------------------------------------------------
    def supports(self, dtype: torch.dtype, bitwidth: int, block_size: int) -> bool:
        return dtype in DTYPE_CODE and bool(self.native.lib.bcom_collective_supported(
            DTYPE_CODE[dtype], int(bitwidth), int(block_size)))

    def check_status(self) -> None:
        """Raise if a kernel of this communicator gave up waiting; re-arm afterwards."""
        if not self.native.failed():
            return
        status = self.native.status()
        if status[0] != 0:
            self.native.reset()
            _timing.add("fused_timeouts")
            raise FusedCollectiveError(_describe(status))

    def set_timeout_ms(self, ms: float) -> None:
        self.native.lib.bcom_comm_set_timeout_ms(self.native.handle, float(ms))

    def set_ll_max_bytes(self, nbytes: int) -> None:
        """All-reduces of at most ``nbytes`` (counted at four bytes per element whatever the dtype;
        4- or 8-bit codes, aligned tensors) run as ONE
        pass whose packed words carry their own arrival flags instead of as three phases with
        two flag handshakes; 0 switches that off.  Every rank of the group must use the same
        value (the two forms do not talk to each other)."""
        self.native.lib.bcom_comm_set_ll_max_bytes(self.native.handle, int(nbytes))

    def phase_times_us(self) -> dict:
        """Phase breakdown of this rank's last kernel (see ``_NativeComm.phase_times_us``);
        synchronises the device first."""
        torch.cuda.synchronize(self.device)
        return self.native.phase_times_us()

    def check_canaries(self) -> None:
        """Debugging aid for tests: see ``_NativeComm.check_canaries``."""
        self.native.check_canaries()

    # -- launch -------------------------------------------------------------------------
    def _launch(self, args: CollArgs, async_op: bool, keep):
        from ..api import _CudaEventWork

        if self.native.failed():
            self.check_status()
        cur = torch.cuda.current_stream(self.device)
        stream = cur
        if async_op:
            stream = self.side_stream
            stream.wait_stream(cur)
        if torch.cuda.current_device() == self.device.index:
            rc = self.native.lib.bcom_collective(
                self.native.handle, ctypes.byref(args), ctypes.c_void_p(stream.cuda_stream))
        else:
            with torch.cuda.device(self.device):
                rc = self.native.lib.bcom_collective(
                    self.native.handle, ctypes.byref(args), ctypes.c_void_p(stream.cuda_stream))
        if rc:
            check(rc, "bcom_collective")
        _native.add_launches(1)   # at least one kernel (large buckets: one per chunk)
        self.launches += 1
        _timing.add("fused_launches")
        payload, wire = traffic_bytes(args, self.world)
        _timing.add("fused_payload_bytes", payload)
        _timing.add("fused_wire_bytes", wire)
        if not async_op:
            return None
        done = torch.cuda.Event()
        done.record(stream)
        for t in keep:
            if t is not None:
                t.record_stream(stream)
        return _CudaEventWork(done, keepalive=list(keep), on_complete=self.check_status)

    def all_reduce(self, tensor: torch.Tensor, *, bitwidth: int, block_size: int,
                   stochastic: bool = False, seed: Optional[int] = None, ef=None,
                   stage2: bool = False, post_scale: float = 1.0, async_op: bool = False,
                   max_ctas: Optional[int] = None):
        """In-place low-bit sum of a contiguous CUDA tensor over the group.  ``max_ctas`` caps
        the kernel's grid (default: the communicator's setting, 0 = as many CTAs as fit an
        empty GPU): a launch that has to run NEXT TO other kernels (gradient buckets under a
        persistent GEMM) must be small enough to become co-resident with them, because every
        CTA of the cooperative grid has to be on the device before the first flag wait ends."""
        from ..api import ShardPlan

        n = int(tensor.numel())
        if n == 0:
            return None
        plan = ShardPlan(self.world, n)
        res1 = res2 = None
        if ef is not None:
            ef.ensure(plan, tensor.device, stage2)
            res1, res2 = ef.stage1, (ef.stage2 if stage2 else None)
        args = _args(tensor, tensor, res1, res2, n, plan.shard_len, tensor.dtype, bitwidth,
                     block_size, MODE_ALL_REDUCE, stochastic, seed, post_scale,
                     self.max_ctas if max_ctas is None else int(max_ctas), self.rank)
        return self._launch(args, async_op, (tensor, res1, res2))

    def reduce_scatter(self, output: torch.Tensor, input: torch.Tensor, *, bitwidth: int,
                       block_size: int, stochastic: bool = False, seed: Optional[int] = None,
                       ef=None, post_scale: float = 1.0, async_op: bool = False):
        """``output[S] = sum over ranks of dequant(quant(input[rank*S:(rank+1)*S]))``."""
        from ..api import ShardPlan

        S = int(output.numel())
        if int(input.numel()) != S * self.world or input.dtype != output.dtype:
            raise ValueError("reduce_scatter needs input [world*S] and output [S] of one dtype")
        res1 = None
        if ef is not None:
            ef.ensure(ShardPlan(self.world, S * self.world), input.device, False)
            res1 = ef.stage1
        args = _args(input, output, res1, None, S * self.world, S, input.dtype, bitwidth,
                     block_size, MODE_REDUCE_SCATTER, stochastic, seed, post_scale,
                     self.max_ctas, self.rank)
        return self._launch(args, async_op, (input, output, res1))

    def all_gather(self, output: torch.Tensor, input: torch.Tensor, *, bitwidth: int,
                   block_size: int, stochastic: bool = False, seed: Optional[int] = None,
                   ef=None, post_scale: float = 1.0, async_op: bool = False):
        """``output[j*S:(j+1)*S] = dequant(quant(rank j's input[S]))`` on every rank."""
        S = int(input.numel())
        if int(output.numel()) != S * self.world or input.dtype != output.dtype:
            raise ValueError("all_gather needs input [S] and output [world*S] of one dtype")
        res2 = None
        if ef is not None:
            if ef.stage2 is None or ef.stage2.numel() != S:
                ef.stage2 = torch.zeros(S, dtype=torch.float32, device=input.device)
            res2 = ef.stage2
        args = _args(input, output, None, res2, S * self.world, S, input.dtype, bitwidth,
                     block_size, MODE_ALL_GATHER, stochastic, seed, post_scale, self.max_ctas,
                     self.rank)
        return self._launch(args, async_op, (input, output, res2))


class EmulatedWorld:
    """W ranks on one device, run by one cooperative kernel launch per chunk."""

    def __init__(self, world: int, device="cuda:0", region_bytes: int = 8 << 20,
                 timeout_ms: float = 2000.0, ll_max_bytes: Optional[int] = None):
        """``ll_max_bytes``: largest all-reduce (bytes of the tensor) that runs as one
        flag-in-data launch, counted at four bytes per element (``None``: the library's default,
        64 MiB = 16 Mi elements; 0: never)."""
        self.world = world
        self.device = torch.device(device)
        self.comms = [_NativeComm(r, world, region_bytes, self.device) for r in range(world)]
        lib = self.comms[0].lib
        for a in self.comms:
            for b in self.comms:
                if a is not b:
                    lib.bcom_comm_set_peer(a.handle, b.rank, lib.bcom_comm_local_base(b.handle))
            lib.bcom_comm_set_timeout_ms(a.handle, float(timeout_ms))
            if ll_max_bytes is not None:
                lib.bcom_comm_set_ll_max_bytes(a.handle, int(ll_max_bytes))
        self.lib = lib

    def close(self):
        for c in self.comms:
            c.close()

    def status(self) -> List[List[int]]:
        return [c.status() for c in self.comms]

    def phase_times_us(self) -> List[dict]:
        return [c.phase_times_us() for c in self.comms]

    def check_canaries(self) -> None:
        for c in self.comms:
            c.check_canaries()

    def reset(self):
        for c in self.comms:
            c.reset()

    def max_chunk(self, bits: int, block: int) -> int:
        return int(self.lib.bcom_comm_max_chunk(self.comms[0].handle, bits, block))

    def _run(self, arg_list: List[CollArgs]) -> None:
        handles = (ctypes.c_void_p * self.world)(*[c.handle for c in self.comms])
        args = (CollArgs * self.world)(*arg_list)
        with torch.cuda.device(self.device):
            check(self.lib.bcom_collective_emulated(
                handles, args, self.world,
                ctypes.c_void_p(torch.cuda.current_stream(self.device).cuda_stream)),
                "bcom_collective_emulated")

    def all_reduce(self, tensors: List[torch.Tensor], *, bitwidth: int, block_size: int,
                   stochastic: bool = False, seed: Optional[int] = None,
                   res1: Optional[List[torch.Tensor]] = None,
                   res2: Optional[List[torch.Tensor]] = None, post_scale: float = 1.0):
        n = int(tensors[0].numel())
        S = -(-n // self.world)
        self._run([
            _args(t, t, res1[r] if res1 else None, res2[r] if res2 else None, n, S, t.dtype,
                  bitwidth, block_size, MODE_ALL_REDUCE, stochastic, seed, post_scale, 0, r)
            for r, t in enumerate(tensors)])

    def reduce_scatter(self, outputs, inputs, *, bitwidth, block_size, stochastic=False,
                       seed=None, res1=None):
        S = int(outputs[0].numel())
        self._run([
            _args(i, o, res1[r] if res1 else None, None, S * self.world, S, i.dtype, bitwidth,
                  block_size, MODE_REDUCE_SCATTER, stochastic, seed, 1.0, 0, r)
            for r, (i, o) in enumerate(zip(inputs, outputs))])

    def all_gather(self, outputs, inputs, *, bitwidth, block_size, stochastic=False, seed=None,
                   res2=None):
        S = int(inputs[0].numel())
        self._run([
            _args(i, o, None, res2[r] if res2 else None, S * self.world, S, i.dtype, bitwidth,
                  block_size, MODE_ALL_GATHER, stochastic, seed, 1.0, 0, r)
            for r, (i, o) in enumerate(zip(inputs, outputs))])
