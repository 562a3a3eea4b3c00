"""Host-side logic of the fused communicator that needs no GPU: traffic accounting, and the
constructor's choice between its own IPC-mapped blocks and blocks adopted from torch symmetric
memory with an NVLink multicast mapping (all ranks vote; native pieces are stand-ins here)."""

import sys
import types

import torch
import torch.distributed as dist

from bitscom_b200.parallel import fused as F

from _dist import run_ranks


def test_traffic_bytes():
    a = F.CollArgs(n=1000, S=512, dtype=0, bits=4, block=256, mode=F.MODE_ALL_REDUCE)
    assert F.traffic_bytes(a, 2) == (4000, 2 * 1 * (256 + 4))
    a = F.CollArgs(n=4096, S=512, dtype=2, bits=1, block=64, mode=F.MODE_REDUCE_SCATTER)
    assert F.traffic_bytes(a, 8) == (8192, 7 * (64 + 16))
    a = F.CollArgs(n=10, S=3, dtype=1, bits=2, block=8, mode=F.MODE_ALL_GATHER)
    assert F.traffic_bytes(a, 4) == (20, 3 * (1 + 2))


class _FakeLib:
    @staticmethod
    def bcom_comm_block_bytes(region):
        return 4096 + 2 * region

    @staticmethod
    def bcom_comm_set_timeout_ms(handle, ms):
        return 0


class _FakeNative:
    log = []

    def __init__(self, rank, world, region_bytes, device, external_bases=None, multicast_base=0):
        self.lib, self.handle = _FakeLib, object()
        self.external = external_bases is not None
        self.bases, self.mc = external_bases, multicast_base
        _FakeNative.log.append("external" if self.external else "ipc")

    def ipc_handle(self):
        return b"h" * 64

    def open_peers(self, handles):
        assert len(handles) == dist.get_world_size() and all(h == b"h" * 64 for h in handles)
        _FakeNative.log.append("opened")


def _install_fakes(monkey_symm):
    F._NativeComm = _FakeNative
    F._get = lambda: _FakeLib
    torch.cuda.Stream = lambda device=None: object()
    mod = types.ModuleType("torch.distributed._symmetric_memory")
    mod.empty, mod.rendezvous = monkey_symm
    sys.modules["torch.distributed._symmetric_memory"] = mod
    torch.distributed._symmetric_memory = mod


def _ctor_worker(rank, world, scenario):
    import os

    def empty(nbytes, dtype=None, device=None):
        return torch.empty(8, dtype=torch.uint8)

    def rendezvous(buf, group=None):
        if scenario == "one_rank_fails" and rank == 1:
            raise RuntimeError("no fabric handle")
        has_mc = scenario != "no_multicast"
        return types.SimpleNamespace(multicast_ptr=0x7000_0000 if has_mc else 0,
                                     has_multicast_support=has_mc,
                                     buffer_ptrs=[0x1000_0000 * (r + 1) for r in range(world)])

    _install_fakes((empty, rendezvous))
    if scenario != "flag_off":
        os.environ["BITSCOM_NVLS"] = "1"
    else:
        os.environ.pop("BITSCOM_NVLS", None)
    comm = F.FusedLowBitComm(dist.group.WORLD, torch.device("cpu"), region_bytes=1 << 20)
    if scenario == "all_ok":
        assert comm.multicast and comm.native.external and _FakeNative.log == ["external"]
        assert comm.native.mc == 0x7000_0000 and len(comm.native.bases) == world
    else:  # every rank fell back to its own block and the IPC exchange, together
        assert not comm.multicast and not comm.native.external
        assert _FakeNative.log == ["ipc", "opened"]


def test_constructor_uses_multicast_blocks_only_when_every_rank_can():
    for scenario in ("flag_off", "all_ok", "no_multicast", "one_rank_fails"):
        run_ranks(_ctor_worker, 2, scenario)
