"""LowBitGroup path selection and Work semantics against recorded fake collectives
(same behaviours the reference pins in its tests/test_api.py)."""

import time
from types import SimpleNamespace

import pytest
import torch

import bitscom_b200.api as api
from bitscom_b200.api import LowBitGroup


class RecordedWork:
    def __init__(self, future=None):
        self.future = future
        self.waits = 0

    def wait(self):
        self.waits += 1
        return self.future.wait() if self.future is not None else True


class FutureWork(RecordedWork):
    def get_future(self):
        return self.future


@pytest.fixture
def fake(monkeypatch):
    log = {"all_to_all": [], "all_gather": [], "all_reduce": [], "reduce_scatter": [],
           "broadcast": []}
    default_group = object()
    sizes = {"world": 8, "rank": 1}

    def all_to_all(outs, ins, group=None, async_op=False):
        log["all_to_all"].append(SimpleNamespace(group=group, async_op=async_op, n=len(ins)))
        for o, i in zip(outs, ins):
            o.copy_(i)
        return RecordedWork()

    def all_gather(outs, inp, group=None, async_op=False):
        log["all_gather"].append(SimpleNamespace(group=group, async_op=async_op))
        for o in outs:
            o.copy_(inp)
        return RecordedWork()

    def recorder(name):
        def fn(*args, **kwargs):
            log[name].append(SimpleNamespace(args=args, kwargs=kwargs))
            return RecordedWork()
        return fn

    monkeypatch.setattr(api.dist.distributed_c10d, "_get_default_group", lambda: default_group)
    monkeypatch.setattr(api.dist, "get_rank", lambda group=None: sizes["rank"])
    monkeypatch.setattr(api.dist, "get_world_size", lambda group=None: sizes["world"])
    monkeypatch.setattr(api.dist, "all_to_all", all_to_all)
    monkeypatch.setattr(api.dist, "all_gather", all_gather)
    for name in ("all_reduce", "reduce_scatter", "broadcast"):
        monkeypatch.setattr(api.dist, name, recorder(name))
    return SimpleNamespace(log=log, default_group=default_group, sizes=sizes)


def test_default_group_rank_world(fake):
    g = LowBitGroup(bitwidth=4)
    assert g.pg is fake.default_group and g.rank == 1 and g.world_size == 8


@pytest.mark.parametrize("bad", [0, 3, 15, 17])
def test_rejects_bad_bitwidth(bad):
    with pytest.raises(ValueError):
        LowBitGroup(bitwidth=bad, process_group=object())


def test_rejects_bad_block_size():
    with pytest.raises(ValueError):
        LowBitGroup(bitwidth=4, process_group=object(), block_size=0)


def test_dense_sync_waits_and_async_returns_work(fake):
    g = LowBitGroup(bitwidth=8, process_group=object())
    t = torch.ones(16)
    assert g.all_reduce(t) is None
    assert fake.log["all_reduce"][0].kwargs["async_op"] is True
    assert isinstance(g.all_reduce(t, async_op=True), RecordedWork)


def test_simulate_quantization_changes_values(fake):
    g = LowBitGroup(bitwidth=2, process_group=object(), simulate_quantization=True)
    t = torch.linspace(-1, 1, 128)
    before = t.clone()
    g.all_reduce(t)
    assert not torch.equal(before, t)


def test_compress_decompress(fake):
    g = LowBitGroup(bitwidth=8, process_group=object())
    x = torch.randn(32)
    y = g.decompress(g.compress(x))
    assert y.shape == x.shape and y.dtype == x.dtype


def test_lowbit_path_is_two_alltoall_two_allgather(fake):
    fake.sizes.update(world=2, rank=0)
    g = LowBitGroup(bitwidth=4, process_group=object())
    t = torch.tensor([0.0, 1.0])
    assert g.all_reduce(t) is None
    assert not fake.log["all_reduce"]
    assert len(fake.log["all_to_all"]) == 2 and len(fake.log["all_gather"]) == 2


def test_async_lowbit_defers_second_half_to_wait(fake, monkeypatch):
    monkeypatch.delenv("BITSCOM_UNSAFE_FULL_ASYNC_CHAIN", raising=False)
    fake.sizes.update(world=2, rank=0)
    g = LowBitGroup(bitwidth=4, process_group=object())
    work = g.all_reduce(torch.tensor([0.0, 1.0]), async_op=True)
    assert len(fake.log["all_to_all"]) == 2
    assert all(c.async_op for c in fake.log["all_to_all"])
    assert not fake.log["all_gather"] and not work.is_completed()
    assert work.wait() is True
    assert len(fake.log["all_gather"]) == 2 and work.is_completed()


def test_full_async_chain_advances_before_wait(fake, monkeypatch):
    monkeypatch.setenv("BITSCOM_UNSAFE_FULL_ASYNC_CHAIN", "1")
    fake.sizes.update(world=2, rank=0)
    pending = []
    gathers = []

    def all_to_all(outs, ins, group=None, async_op=False):
        for o, i in zip(outs, ins):
            o.copy_(i)
        fut = torch.futures.Future()
        pending.append(fut)
        return FutureWork(fut)

    def all_gather(outs, inp, group=None, async_op=False):
        gathers.append(1)
        for o in outs:
            o.copy_(inp)
        fut = torch.futures.Future()
        fut.set_result(True)
        return FutureWork(fut)

    monkeypatch.setattr(api.dist, "all_to_all", all_to_all)
    monkeypatch.setattr(api.dist, "all_gather", all_gather)
    g = LowBitGroup(bitwidth=4, process_group=object())
    work = g.all_reduce(torch.tensor([0.0, 1.0]), async_op=True)
    assert len(pending) == 2 and not gathers
    for f in pending:
        f.set_result(True)
    deadline = time.time() + 2
    while len(gathers) < 2 and time.time() < deadline:
        time.sleep(0.01)
    assert len(gathers) == 2
    assert work.wait() is True and work.is_completed()


def test_non_sum_is_dense(fake):
    fake.sizes.update(world=2)
    g = LowBitGroup(bitwidth=4, process_group=object())
    g.all_reduce(torch.tensor([0.0, 1.0]), op=torch.distributed.ReduceOp.MAX)
    assert fake.log["all_reduce"] and not fake.log["all_to_all"]


def test_non_divisible_numel_keeps_shape(fake):
    fake.sizes.update(world=2, rank=0)
    g = LowBitGroup(bitwidth=4, process_group=object())
    t = torch.tensor([0.0, 1.0, 2.0])
    g.all_reduce(t)
    assert t.shape == (3,)


def test_world_one_is_dense(fake):
    fake.sizes.update(world=1, rank=0)
    g = LowBitGroup(bitwidth=4, process_group=object())
    g.all_reduce(torch.ones(4))
    assert fake.log["all_reduce"] and not fake.log["all_to_all"]


def test_pipeline_a_selected_with_both_groups(fake, monkeypatch):
    fake.sizes.update(world=2)
    seen = {}

    def pipeline(self, tensor, *, local_group, inter_group, chunk_size, local_quantize):
        seen.update(chunk_size=chunk_size, local_quantize=local_quantize)
        tensor.add_(1.0)

    monkeypatch.setattr(LowBitGroup, "_hierarchical_lowbit_allreduce_pipeline_a", pipeline)
    g = LowBitGroup(bitwidth=4, process_group=object())
    t = torch.tensor([0.0, 1.0])
    assert g.all_reduce(t, local_group=object(), inter_group=object(), chunk_size=32) is None
    assert seen == {"chunk_size": 32, "local_quantize": False}
    assert torch.allclose(t, torch.tensor([1.0, 2.0]))
    work = g.all_reduce(t, local_group=object(), inter_group=object(), async_op=True)
    assert work.wait() is True


def test_local_only_dense_and_quantized(fake, monkeypatch):
    fake.sizes.update(world=2)
    calls = {"flat": 0}

    def flat_engine(self, flat, group):
        calls["flat"] += 1
        return flat + 2.0

    monkeypatch.setattr(LowBitGroup, "_lowbit_allreduce_via_alltoall_group", flat_engine)
    g = LowBitGroup(bitwidth=4, process_group=object())
    local = object()
    t = torch.tensor([0.0, 1.0])
    g.all_reduce(t, local_group=local, chunk_size=16)
    assert calls["flat"] == 0 and fake.log["all_reduce"][0].kwargs["group"] is local
    g.all_reduce(t, local_group=local, local_quantize=True)
    assert calls["flat"] == 1 and torch.allclose(t, torch.tensor([2.0, 3.0]))


def test_dual_stream_guard(fake):
    g = LowBitGroup(bitwidth=4, process_group=object())
    assert g._should_use_dual_stream_pipeline(is_cuda=True, local_size=8, global_size=8) is False
    assert g._should_use_dual_stream_pipeline(is_cuda=True, local_size=4, global_size=8) is True
    assert g._should_use_dual_stream_pipeline(is_cuda=False, local_size=4, global_size=8) is False


def test_passthrough_collectives(fake):
    g = LowBitGroup(bitwidth=4, process_group=object(), simulate_quantization=True)
    x = torch.linspace(-1, 1, 64)
    g.all_gather([torch.empty(64)], x)
    assert len(fake.log["all_gather"]) == 1
    g.reduce_scatter(torch.empty(64), [x, x])
    sent = fake.log["reduce_scatter"][0].args[1]
    assert not torch.equal(sent[0], x)  # went through the quantize round trip
    assert isinstance(g.broadcast(x, src=0, async_op=True), RecordedWork)


def test_all_reduce_stream_cpu_immediate(fake):
    fake.sizes.update(world=2, rank=0)
    g = LowBitGroup(bitwidth=4, process_group=object())
    t = torch.tensor([1.0, 1.0])
    work = g.all_reduce_stream(t, stream=None, post_scale=0.5)
    assert work.wait() is True and len(fake.log["all_to_all"]) == 2
    # identity fake collectives: both "ranks" contribute the same shard
    assert torch.allclose(t, torch.tensor([1.0, 1.0]), atol=2e-3)


def test_scheduled_handle_plumbing():
    class Handle:
        def launch_phase2(self):
            return True

        def launch_restore(self):
            return True

    class PG:
        def progress_lowbit(self, block):
            return block

        def schedule_lowbit_allreduce(self, tensor):
            return Handle()

    g = LowBitGroup(bitwidth=4, process_group=PG())
    assert g.progress_lowbit(True) is True and g.progress_lowbit() is False
    h = g.schedule_lowbit_allreduce(torch.ones(2))
    assert g.launch_lowbit_phase2(h) and g.launch_lowbit_restore(h)
    plain = LowBitGroup(bitwidth=4, process_group=object())
    assert plain.progress_lowbit() is False
    with pytest.raises(RuntimeError):
        plain.schedule_lowbit_allreduce(torch.ones(2))
    with pytest.raises(RuntimeError):
        plain.launch_lowbit_phase2(object())


def test_state_dict_roundtrip(fake):
    fake.sizes.update(world=2, rank=0)
    g = LowBitGroup(bitwidth=2, process_group=object(), error_feedback=True,
                    stage2_error_feedback=True, sr_seed=11, stochastic_rounding=True)
    t = torch.linspace(-1, 1, 64)
    g.all_reduce(t, ef_key="bucket0")
    sd = g.state_dict()
    assert sd["sr_calls"] == 1 and sd["residuals"]["bucket0"]["stage1"].abs().sum() > 0
    h = LowBitGroup(bitwidth=2, process_group=object(), error_feedback=True)
    h.load_state_dict(sd)
    assert torch.equal(h._ef_states["bucket0"].stage1, sd["residuals"]["bucket0"]["stage1"])
