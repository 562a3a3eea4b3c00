"""ZeRO-1 sharded AdamW on CPU ranks (gloo): low-bit reduce-scatter of the flat gradient,
AdamW on the local shard, low-bit all-gather of the updated parameters.  With 8-bit codes the
result tracks a dense AdamW on the averaged gradient closely, and every rank ends each step
with bit-identical parameters."""

import torch

from bitscom_b200 import LowBitGroup
from bitscom_b200.ops.nn import FlatAdamW
from bitscom_b200.parallel.flat import FlatParameters
from bitscom_b200.parallel.zero import ShardedAdamW

from _dist import run_ranks


def test_flat_adamw_host_path_matches_torch():
    torch.manual_seed(0)
    master = torch.randn(1024)
    ref = torch.nn.Parameter(master.clone())
    grad = torch.zeros(1024)
    bf16 = torch.empty(1024, dtype=torch.bfloat16)
    opt = FlatAdamW(master, grad, bf16, lr=1e-2, weight_decay=0.1)
    tref = torch.optim.AdamW([ref], lr=1e-2, weight_decay=0.1, eps=1e-8)
    for step in range(4):
        g = torch.randn(1024, generator=torch.Generator().manual_seed(step))
        grad.copy_(g * 2.0)
        opt.step(grad_scale=0.5)
        ref.grad = g.clone()
        tref.step()
        assert torch.allclose(master, ref.detach(), atol=1e-6)
        assert grad.eq(0).all() and torch.equal(bf16, master.to(torch.bfloat16))


def _zero_worker(rank, world):
    shapes = {"w1": (64, 32), "b1": (64,), "w2": (16, 64)}
    flat = FlatParameters(shapes, "cpu", pad_to=256 * world)
    g0 = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for _, view in flat.named_views():
            view.copy_(torch.randn(view.shape, generator=g0) * 0.1)
    flat.sync_master_from_params()
    ggrp = LowBitGroup(bitwidth=8, error_feedback=True)
    pgrp = LowBitGroup(bitwidth=8, error_feedback=True)
    opt = ShardedAdamW(flat, ggrp, lr=1e-2, param_bits_group=pgrp)

    ref_master = flat.params.float().clone()
    ref_grad = torch.zeros_like(ref_master)
    ref_opt = FlatAdamW(ref_master, ref_grad, None, lr=1e-2)
    for step in range(3):
        grads = [torch.randn(flat.numel, generator=torch.Generator().manual_seed(10 * step + r))
                 * 1e-2 for r in range(world)]
        flat.grads.copy_(grads[rank])
        opt.step()
        ref_grad.copy_(torch.stack(grads).sum(0))
        ref_opt.step(grad_scale=1.0 / world)
        assert flat.grads.eq(0).all()
        pgrp.check_agreement(flat.params)            # every rank: the same bf16 parameters
        err = (flat.params.float() - ref_master).abs().max().item()
        assert err < 0.03, (step, err)               # bf16 copy + 8-bit codes + EF
    # the update really happened and is shard-local: the master shard moved
    lo = rank * opt.shard
    assert not torch.equal(opt.master_shard, torch.zeros_like(opt.master_shard))
    # (AdamW steps have magnitude ~lr whatever the gradient scale, so quantization noise on
    # tiny gradients can move single elements by a few steps' worth)
    assert torch.allclose(opt.master_shard, ref_master[lo:lo + opt.shard], atol=0.03)
    assert (opt.master_shard - ref_master[lo:lo + opt.shard]).abs().mean() < 3e-3


def test_sharded_adamw_tracks_dense_adamw_on_cpu_ranks():
    run_ranks(_zero_worker, 2)


def test_flat_sgd_host_path_matches_torch():
    from bitscom_b200.ops.nn import FlatSGD

    torch.manual_seed(0)
    param = torch.randn(512)
    ref = torch.nn.Parameter(param.clone())
    grad = torch.zeros(512)
    opt = FlatSGD(param, grad, lr=0.1, momentum=0.9, weight_decay=1e-3)
    tref = torch.optim.SGD([ref], lr=0.1, momentum=0.9, weight_decay=1e-3)
    for step in range(4):
        g = torch.randn(512, generator=torch.Generator().manual_seed(step))
        grad.copy_(g * 4.0)
        opt.step(grad_scale=0.25)
        ref.grad = g.clone()
        tref.step()
        assert torch.allclose(param, ref.detach(), atol=1e-6) and grad.eq(0).all()


def test_reshard_state_moves_optimizer_state_between_world_sizes():
    """State of a 4-rank run re-partitioned for 3 ranks (padding changes: 4 x 256 vs 3 x 256)
    and for 1 rank; the single-rank optimizer then steps exactly like a dense AdamW that was
    given the same full state."""
    from bitscom_b200.parallel.zero import reshard_state

    numel = 1500
    g = torch.Generator().manual_seed(3)
    old_world, old_padded = 4, 2048
    full = {k: torch.zeros(old_padded) for k in ("master", "exp_avg", "exp_avg_sq")}
    full["master"][:numel] = torch.randn(numel, generator=g)
    full["exp_avg"][:numel] = torch.randn(numel, generator=g) * 1e-2
    full["exp_avg_sq"][:numel] = torch.rand(numel, generator=g) * 1e-3
    shard = old_padded // old_world
    states = [{"opt": dict({k: v[r * shard:(r + 1) * shard].clone() for k, v in full.items()},
                           step=7),
               "master_shard": full["master"][r * shard:(r + 1) * shard].clone()}
              for r in range(old_world)]

    three = reshard_state(states, 3, numel)
    assert [s["opt"]["master"].numel() for s in three] == [512, 512, 512]   # 1536 = 2 * 768
    for k in ("master", "exp_avg", "exp_avg_sq"):
        joined = torch.cat([s["opt"][k] for s in three])
        assert torch.equal(joined[:numel], full[k][:numel]) and joined[numel:].eq(0).all()
    assert all(s["opt"]["step"] == 7 for s in three)

    one = reshard_state(states, 1, numel)[0]
    flat = FlatParameters({"w": (numel,)}, "cpu", pad_to=256)
    class Solo:  # world 1: the group is never asked to talk
        world_size, rank = 1, 0

    opt = ShardedAdamW(flat, Solo(), lr=1e-2)
    opt.load_state_dict(one)
    ref_master, ref_grad = full["master"][:1536].clone(), torch.zeros(1536)
    ref = FlatAdamW(ref_master, ref_grad, None, lr=1e-2)
    ref.load_state_dict({"step": 7, "exp_avg": full["exp_avg"][:1536],
                         "exp_avg_sq": full["exp_avg_sq"][:1536], "master": ref_master.clone()})
    grad = torch.randn(1536, generator=g) * 1e-2
    flat.grads.copy_(grad)
    ref_grad.copy_(grad)
    opt.step()
    ref.step()
    assert torch.equal(opt.master_shard, ref_master)

    import pytest

    states[2]["opt"]["step"] = 8
    with pytest.raises(ValueError):
        reshard_state(states, 2, numel)


def _bucketed_worker(rank, world):
    """The bucketed optimizer with the buckets announced out of backward, against the
    monolithic one on the same gradients: same wire format per element is not expected (the
    shards differ), so both are compared with a dense AdamW."""
    from bitscom_b200.parallel.zero import BucketedShardedAdamW, bucket_cuts

    shapes = {"emb": (40, 32), "l0.w": (64, 32), "l0.b": (64,), "l1.w": (48, 64), "head": (7,)}
    flat = FlatParameters(shapes, "cpu", pad_to=256 * world)
    g0 = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for _, view in flat.named_views():
            view.copy_(torch.randn(view.shape, generator=g0) * 0.1)
    flat.sync_master_from_params()
    starts = [flat.offsets[k][0] for k in ("emb", "l0.w", "l1.w", "head")]
    cuts = bucket_cuts(starts, flat.numel, world)
    assert cuts[0] == 0 and cuts[-1] == flat.numel and len(cuts) >= 3
    assert all(c % (256 * world) == 0 for c in cuts)
    ggrp = LowBitGroup(bitwidth=8, error_feedback=True)
    pgrp = LowBitGroup(bitwidth=8, error_feedback=True)
    opt = BucketedShardedAdamW(flat, ggrp, cuts, lr=1e-2, param_bits_group=pgrp)
    ref_master = flat.params.float().clone()
    ref_grad = torch.zeros_like(ref_master)
    ref_opt = FlatAdamW(ref_master, ref_grad, None, lr=1e-2)
    for step in range(3):
        grads = [torch.randn(flat.numel, generator=torch.Generator().manual_seed(10 * step + r))
                 * 1e-2 for r in range(world)]
        flat.grads.copy_(grads[rank])
        # backward order: head, l1, l0 announced; the embedding is left to step()
        for key in ("head", "l1.w", "l0.w"):
            opt.ready_from(flat.offsets[key][0])
        launched = sum(opt._launched)
        assert 1 <= launched < len(opt.parts)
        opt.step()
        ref_grad.copy_(torch.stack(grads).sum(0))
        ref_opt.step(grad_scale=1.0 / world)
        assert flat.grads.eq(0).all()
        pgrp.check_agreement(flat.params)
        assert (flat.params.float() - ref_master).abs().max().item() < 0.03
    # residuals are kept per bucket
    assert len({k for k in ggrp._ef_states}) == len(opt.parts)
    # state round trip, and re-partition for another world size and other cuts
    from bitscom_b200.parallel.zero import reshard_bucketed_state

    sd = opt.state_dict()
    opt.load_state_dict(sd)
    states = [None] * world
    import torch.distributed as dist

    dist.all_gather_object(states, sd)
    new_cuts = [0, flat.numel]
    one = reshard_bucketed_state(states, 1, new_cuts, flat.used)[0]
    whole = torch.cat([torch.cat([s["buckets"][b]["opt"]["master"] for s in states])
                       for b in range(len(opt.parts))])
    assert torch.equal(one["buckets"][0]["opt"]["master"][:flat.used], whole[:flat.used])
    assert one["buckets"][0]["opt"]["master"][flat.used:].eq(0).all()


def test_bucketed_sharded_adamw_on_cpu_ranks():
    run_ranks(_bucketed_worker, 2)
