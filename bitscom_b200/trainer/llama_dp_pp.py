"""Llama DP x PP trainer (shape of the reference's
``benchmarks/train_llama7b_dp_pp_lowbit.py``): a (dp, pp) mesh with pp the fast
dimension, one pipeline stage per rank, AdamW, data-parallel gradient all-reduce through
``LowBitGroup``.  Differences, all deliberate:

* the model is this repo's own (``bitscom_b200.models.llama``), bf16 compute with fp32
  master weights and fp32 gradient accumulation, on hand-written sm_100a kernels;
* the schedule is 1F1B (``parallel.pp_schedule``), not GPipe;
* gradients are synchronised per layer-sized slice of the flat gradient buffer with the
  fused low-bit kernel on a side stream while the last micro-batch is still in backward,
  with error feedback, instead of one exposed synchronous call per parameter;
* data is synthetic (uniform token ids), staged in pinned host memory.

Launch with torchrun (one process per GPU) or run single-process for one GPU:

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m bitscom_b200.trainer.llama_dp_pp --pp_size 2 --bitwidth 4 --max_steps 10
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..api import LowBitGroup
from ..models.llama import LlamaConfig, LlamaStage
from ..ops import nn as K
from ..parallel.hooks import GradBucketSync
from ..parallel.pp_schedule import InterleavedRunner, PipelineRunner


@dataclass
class TrainerConfig:
    pp_size: int = 1
    pp_chunks: int = 1            # model chunks per pipeline rank (>= 2: interleaved 1F1B)
    micro_batches: int = 4
    micro_batch_size: int = 1
    seq_length: int = 2048
    bitwidth: int = 4
    block_size: int = 256
    stochastic_rounding: bool = False
    error_feedback: bool = True
    stage2_error_feedback: bool = False
    dp_sync: str = "pipeline_a"   # "pipeline_a" | "flat" | "dense"
    local_size: int = 1           # ranks per local group of pipeline-A
    overlap: bool = True
    sync_max_ctas: int = 148      # grid cap of gradient buckets launched under backward (0: none)
    simulate_quantization: bool = False   # reference flag: quantize round trip before dense ops
    defer_wgrad: bool = True   # pipeline stages send input gradients before weight-gradient GEMMs
    device: str = "cuda"       # "cpu": CPU ranks over gloo with the ops' host paths (plumbing)
    pg_timeout_s: Optional[float] = None  # process-group timeout (None: torch's default)
    lr: float = 1e-4
    weight_decay: float = 0.01
    seed: int = 0


def _init_distributed(device: str = "cuda", timeout_s: Optional[float] = None
                      ) -> Tuple[int, int, int]:
    cuda = device == "cuda"
    extra = {}
    if timeout_s:
        import datetime

        # a collective whose peer is gone then fails after this long instead of the default
        extra["timeout"] = datetime.timedelta(seconds=float(timeout_s))
    if "RANK" in os.environ and int(os.environ.get("WORLD_SIZE", "1")) > 1:
        rank = int(os.environ["RANK"])
        local = int(os.environ.get("LOCAL_RANK", rank))
        if cuda:
            torch.cuda.set_device(local)
        if not dist.is_initialized():
            if cuda:
                dist.init_process_group("nccl", device_id=torch.device("cuda", local), **extra)
            else:
                dist.init_process_group("gloo", **extra)
        return rank, dist.get_world_size(), local
    if cuda:
        torch.cuda.set_device(0)
    return 0, 1, 0


class LlamaTrainer:
    def __init__(self, model_cfg: LlamaConfig, cfg: TrainerConfig):
        self.cfg, self.model_cfg = cfg, model_cfg
        self.rank, self.world, self.local = _init_distributed(cfg.device, cfg.pg_timeout_s)
        if self.world % cfg.pp_size:
            raise RuntimeError(f"world_size {self.world} must be divisible by pp_size "
                               f"{cfg.pp_size}")
        self.pp, self.dp = cfg.pp_size, self.world // cfg.pp_size
        self.pp_rank, self.dp_rank = self.rank % self.pp, self.rank // self.pp
        self.device = torch.device("cuda", self.local) if cfg.device == "cuda" \
            else torch.device("cpu")

        # groups: every rank creates all of them in the same order
        self.pp_group = self.dp_group = None
        if self.world > 1:
            for d in range(self.dp):
                g = dist.new_group([d * self.pp + p for p in range(self.pp)])
                if d == self.dp_rank:
                    self.pp_group = g
            for p in range(self.pp):
                g = dist.new_group([d * self.pp + p for d in range(self.dp)])
                if p == self.pp_rank:
                    self.dp_group = g

        # chunk c of this rank is virtual stage c * pp + pp_rank of pp * chunks; one chunk is
        # the plain contiguous split
        self.chunks = max(1, int(cfg.pp_chunks)) if self.pp > 1 else 1
        if self.chunks > 1 and cfg.micro_batches % self.pp:
            raise RuntimeError(f"interleaved pipeline: micro_batches ({cfg.micro_batches}) must "
                               f"be a multiple of pp_size ({self.pp})")
        if model_cfg.num_layers < self.pp * self.chunks:
            raise RuntimeError(f"{model_cfg.num_layers} layers cannot be cut into "
                               f"{self.pp * self.chunks} virtual stages")
        self.models = [LlamaStage(model_cfg, c * self.pp + self.pp_rank, self.pp * self.chunks,
                                  self.device, seed=cfg.seed) for c in range(self.chunks)]
        self.model = self.models[0]
        self.opts = [K.FlatAdamW(m.flat.master, m.flat.grads, m.flat.params, lr=cfg.lr,
                                 weight_decay=cfg.weight_decay) for m in self.models]
        self.opt = self.opts[0]
        self._layer_chunk = {i: c for c, m in enumerate(self.models)
                             for i in range(*m.layer_range)}
        act_shape = (cfg.micro_batch_size * cfg.seq_length, model_cfg.hidden_size)
        self.runner = None
        if self.pp > 1 and self.chunks > 1:
            self.runner = InterleavedRunner(
                self.pp_rank, self.pp, self.chunks, self.pp_group,
                ring=[self.dp_rank * self.pp + p for p in range(self.pp)], act_shape=act_shape,
                device=self.device, defer_wgrad=cfg.defer_wgrad)
        elif self.pp > 1:
            self.runner = PipelineRunner(
                self.pp_rank, self.pp, self.pp_group,
                prev_rank=self.rank - 1 if self.pp_rank > 0 else None,
                next_rank=self.rank + 1 if self.pp_rank < self.pp - 1 else None,
                act_shape=act_shape, device=self.device, defer_wgrad=cfg.defer_wgrad,
                defer_last=cfg.defer_wgrad)

        self.syncs: List[GradBucketSync] = []
        self._range_indexes: List[dict] = []
        self.sync: Optional[GradBucketSync] = None
        if self.dp > 1:
            self.lowbit = LowBitGroup(
                bitwidth=cfg.bitwidth, process_group=self.dp_group,
                block_size=cfg.block_size, stochastic_rounding=cfg.stochastic_rounding,
                simulate_quantization=cfg.simulate_quantization,
                error_feedback=cfg.error_feedback,
                stage2_error_feedback=cfg.stage2_error_feedback, sr_seed=cfg.seed + 17)
            local_group = inter_group = None
            mode = cfg.dp_sync
            if mode == "pipeline_a":
                local_group, inter_group = self._hierarchy(cfg.local_size)
            for c, m in enumerate(self.models):
                ranges, index = self._sync_ranges(m)
                self._range_indexes.append(index)
                self.syncs.append(GradBucketSync(
                    self.lowbit, m.flat.grads, ranges, mode=mode,
                    local_group=local_group, inter_group=inter_group, overlap=cfg.overlap,
                    max_ctas=cfg.sync_max_ctas or None,
                    key_prefix=("chunk", c) if self.chunks > 1 else None))
            self.sync = self.syncs[0]
        self.step_count = 0
        self._pinned: Optional[torch.Tensor] = None
        self._marks: List[tuple] = []   # per step: CUDA events at the phase boundaries

    # -- topology helpers --------------------------------------------------------------
    def _hierarchy(self, local_size: int):
        """Local groups of ``local_size`` consecutive DP ranks and the group of their
        leaders.  ``local_size == 1`` is the degenerate hierarchy the reference's own
        pipeline-A test uses (``tests/test_pipeline_a_correctness.py:16-22``)."""
        dp_ranks = [d * self.pp + self.pp_rank for d in range(self.dp)]
        if local_size <= 1:
            return None, None  # handled as flat low-bit over the whole DP group
        local = inter = None
        for p in range(self.pp):
            ranks = [d * self.pp + p for d in range(self.dp)]
            for i in range(0, self.dp, local_size):
                g = dist.new_group(ranks[i:i + local_size])
                if p == self.pp_rank and self.rank in ranks[i:i + local_size]:
                    local = g
            g = dist.new_group(ranks[::local_size])
            if p == self.pp_rank:
                inter = g
        return local, inter

    @staticmethod
    def _sync_ranges(model) -> Tuple[List[Tuple[int, int]], dict]:
        """One slice per transformer layer (plus embedding / head) of ``model``, in the order
        backward finishes them (last layer first), and the slice index of every key."""
        flat = model.flat
        names = list(flat.offsets)
        groups: List[Tuple[int, int]] = []
        keys: List[str] = []
        cur_key, start = None, 0
        for name in names + [None]:
            key = name.split(".")[0] if name is not None else None
            off = flat.offsets[name][0] if name is not None else flat.numel
            if cur_key is not None and key != cur_key:
                groups.append((start, off - start))
                keys.append(cur_key)
                start = off
            cur_key = key
        groups.reverse()
        keys.reverse()
        return groups, {k: i for i, k in enumerate(keys)}

    def _layer_done(self, layer: int) -> None:
        """Backward of the last micro-batch has passed ``layer``: its slice, and the
        head / final norm when it is the stage's last layer, are final."""
        if not self.syncs:
            return
        chunk = self._layer_chunk[layer]
        sync, index = self.syncs[chunk], self._range_indexes[chunk]
        if layer == self.models[chunk].layer_range[1] - 1:
            for key in ("lm_head", "final_norm"):
                if key in index:
                    sync.on_ready_overlapped(index[key])
        sync.on_ready_overlapped(index[f"l{layer}"])

    def _layer_done_after_deferred(self, layer: int) -> None:
        """``_layer_done`` for a backward whose weight-gradient GEMMs are queued: the bucket of
        the layer is launched from the queue, right behind those GEMMs."""
        from ..parallel.deferred import DeferredWork

        queue = DeferredWork.active()
        if queue is None:
            self._layer_done(layer)
        else:
            queue.add(lambda: self._layer_done(layer))

    # -- data ---------------------------------------------------------------------------
    def synthetic_batch(self, step: int, pinned: bool = True) -> torch.Tensor:
        """Uniform token ids ``[micro_batches, micro_batch_size, seq]`` for this DP rank."""
        c = self.cfg
        g = torch.Generator().manual_seed(1000003 * (step + 1) + self.dp_rank)
        ids = torch.randint(1, self.model_cfg.vocab_size,
                            (c.micro_batches, c.micro_batch_size, c.seq_length), generator=g)
        return ids.pin_memory() if pinned and self.device.type == "cuda" else ids

    # -- one optimizer step ---------------------------------------------------------------
    def train_step(self, ids_host_or_dev: torch.Tensor) -> Optional[torch.Tensor]:
        """``ids``: ``[micro_batches, micro_batch_size, seq]`` int64, pinned host or device.
        Returns the mean loss as a device scalar on the last stage, else ``None``."""
        c = self.cfg
        t_start = self._event() if self.device.type == "cuda" else None
        ids = ids_host_or_dev.to(self.device, non_blocking=True)
        scale = 1.0 / c.micro_batches
        losses: List[torch.Tensor] = []

        last_mb = c.micro_batches - 1

        def forward_chunk(mb: int, chunk: int, x: Optional[torch.Tensor]):
            model = self.models[chunk]
            # with deferred weight gradients the last backward's GEMMs run after its input
            # gradient has been sent (the deferral that shortens the pipeline's drain); the
            # per-layer bucket launches, which need finished gradients, then ride in the same
            # queue, each behind the weight-gradient GEMMs of its layer
            model.on_layer_backward = None
            if mb == last_mb and self.syncs and c.overlap:
                model.on_layer_backward = self._layer_done_after_deferred if (
                    c.defer_wgrad and self.runner is not None) else self._layer_done
            if not model.is_first:
                model.set_shape(c.micro_batch_size, c.seq_length)
            inp = ids[mb] if model.is_first else x
            tgt = ids[mb] if model.is_last else None
            if model.is_last:
                return model(inp, targets=tgt, ignore_index=0, loss_scale=scale)
            return model(inp)

        if self.runner is None:
            for mb in range(c.micro_batches):
                loss = forward_chunk(mb, 0, None)
                losses.append(loss.detach())
                loss.backward()
        elif self.chunks > 1:
            losses = self.runner.run(c.micro_batches, forward_chunk)
        else:
            losses = self.runner.run(c.micro_batches, lambda mb, x: forward_chunk(mb, 0, x))

        for model in self.models:
            model.on_layer_backward = None
        marks = self._mark_begin(t_start) if self.device.type == "cuda" else None
        for sync in self.syncs:
            sync.finish()
        if marks is not None:
            marks.append(self._event())
        for opt in self.opts:
            opt.step(grad_scale=1.0, zero_grad=True)
        if marks is not None:
            marks.append(self._event())
            self._marks.append(tuple(marks))
            del self._marks[:-64]
        self.step_count += 1
        if self.models[-1].is_last:
            return torch.stack(losses).sum()
        return None

    # -- where the step's time goes ---------------------------------------------------------
    def _event(self):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(self.device))
        return ev

    def _mark_begin(self, t_start):
        return [t_start, self._event()]

    def step_breakdown(self, last: int = 0) -> Optional[dict]:
        """Device time of the phases of the last ``last`` steps (0 = all recorded, at most 64),
        in ms per step, on this rank's compute stream: ``fwd_bwd`` (micro-batches, pipeline
        waits included), ``exposed_grad_sync`` (what the compute stream still had to wait for
        after backward had ended: gradient buckets not hidden behind it) and ``optimizer``.
        Synchronises the device."""
        if not self._marks:
            return None
        torch.cuda.synchronize(self.device)
        rows = self._marks[-last:] if last else self._marks
        out = {"fwd_bwd": 0.0, "exposed_grad_sync": 0.0, "optimizer": 0.0}
        for t0, t1, t2, t3 in rows:
            out["fwd_bwd"] += t0.elapsed_time(t1)
            out["exposed_grad_sync"] += t1.elapsed_time(t2)
            out["optimizer"] += t2.elapsed_time(t3)
        return {k: v / len(rows) for k, v in out.items()}

    def check_kernels(self) -> None:
        """Raise if a GEMM, attention or fused-collective kernel gave up on one of its bounded
        waits since the last check (it then returned early and its output is not valid).
        Synchronises the device, so call it where the step is synchronised anyway, and before
        a checkpoint replaces the last good file."""
        from ..ops import attention as A
        from ..ops import gemm as G

        if self.device.type != "cuda":
            return
        if G.available():
            G.check_status()
        if A.available():
            A.check_status()
        if self.syncs:
            torch.cuda.synchronize(self.device)
            for sync in self.syncs:
                sync.check(wait=True)

    # -- checkpoint -----------------------------------------------------------------------
    def state_dict(self) -> dict:
        sd = {"step": self.step_count, "opt": self.opt.state_dict(),
              "params": self.model.flat.params}
        if self.chunks > 1:   # chunk 0 keeps the single-chunk keys; the others follow
            sd["more_chunks"] = [{"opt": o.state_dict(), "params": m.flat.params}
                                 for o, m in zip(self.opts[1:], self.models[1:])]
        if self.sync is not None:
            sd["lowbit"] = self.lowbit.state_dict()
        return sd

    def load_state_dict(self, sd: dict) -> None:
        self.step_count = int(sd["step"])
        self.opt.load_state_dict(sd["opt"])
        self.model.flat.params.copy_(sd["params"])
        if self.chunks > 1:
            if len(sd.get("more_chunks", ())) != self.chunks - 1:
                raise RuntimeError(f"the checkpoint holds {1 + len(sd.get('more_chunks', ()))} "
                                   f"model chunk(s) per rank, this trainer {self.chunks}")
            for o, m, part in zip(self.opts[1:], self.models[1:], sd["more_chunks"]):
                o.load_state_dict(part["opt"])
                m.flat.params.copy_(part["params"])
        if self.sync is not None and "lowbit" in sd:
            self.lowbit.load_state_dict(sd["lowbit"])

    def grad_sync_description(self) -> str:
        """The gradient synchronisation that actually runs (for benchmark records)."""
        c = self.cfg
        if self.sync is None:
            return "none (dp=1)"
        codec = (f"{c.bitwidth}-bit block {c.block_size}"
                 + (" + error feedback" if c.error_feedback else "")
                 + (" + stage 2" if c.stage2_error_feedback else "")
                 + (" + stochastic rounding" if c.stochastic_rounding else ""))
        if self.sync.mode == "dense":
            return "dense NCCL all-reduce per layer bucket"
        if self.sync.mode == "pipeline_a" and self.sync.local_group is not None:
            return (f"pipeline-A (local groups of {c.local_size}, leaders low-bit) {codec}, "
                    "per layer bucket")
        return f"flat fused low-bit all-reduce {codec}, per layer bucket, overlapped"

    def tokens_per_step(self) -> int:
        c = self.cfg
        return self.dp * c.micro_batches * c.micro_batch_size * c.seq_length


def smoke_step(device) -> None:
    """One tiny forward + backward + optimizer step of the flagship model."""
    cfg = LlamaConfig.tiny(attention=_default_attention())
    model = LlamaStage(cfg, device=device, seed=1)
    ids = torch.randint(1, cfg.vocab_size, (2, 128), device=device)
    loss = model(ids, targets=ids)
    loss.backward()
    K.FlatAdamW(model.flat.master, model.flat.grads, model.flat.params, lr=1e-3).step()
    torch.cuda.synchronize()
    assert torch.isfinite(loss).item()


def _default_attention() -> str:
    try:
        from ..ops import attention as A

        return "tcgen05" if A.available() else "sdpa"
    except Exception:
        return "sdpa"


def _train_loop(args, trainer, loader, tcfg, monitor) -> None:
    step = 0
    resumed = trainer.step_count  # > 0 after --resume: those batches have been trained on
    # BITSCOM_INJECT_EXIT="rank:step[:generation]": the named rank exits before that step (a
    # failure made on the host, for recovery tests; generation = the launcher's restart count)
    inject = None
    generation = int(os.environ.get("BITSCOM_RESTART_COUNT", "0"))
    if os.environ.get("BITSCOM_INJECT_EXIT"):
        parts = [int(v) for v in os.environ["BITSCOM_INJECT_EXIT"].split(":")]
        inject = (parts[0], parts[1], parts[2] if len(parts) > 2 else 0)
    for epoch in range(args.epochs):
        loader.set_epoch(epoch)
        for batch in loader:
            if step >= args.max_steps:
                break
            if step < resumed:
                loader.mark_consumed()
                step += 1
                continue
            if monitor is not None:
                monitor.check()
            if inject and (trainer.rank, step, generation) == inject:
                os._exit(17)  # host-side fault injection: this rank is simply gone
            t0 = time.perf_counter()
            loss = trainer.train_step(batch)
            loader.mark_consumed()
            if loss is not None:
                # one write per line: several ranks share the launcher's pipe
                sys.stdout.write(json.dumps({"step": step, "epoch": epoch,
                                             "loss": float(loss.item()),
                                             "step_s": time.perf_counter() - t0}) + "\n")
                sys.stdout.flush()
            if step % 50 == 0:
                trainer.check_kernels()
            step += 1
            if args.output_dir and args.save_every and step % args.save_every == 0:
                from ..utils.checkpoint import save_checkpoint

                trainer.check_kernels()  # never replace a good file with a failed step's state
                save_checkpoint(args.output_dir, trainer.state_dict(), trainer.rank)


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--pp_size", type=int, default=1)
    ap.add_argument("--pp_chunks", type=int, default=0,
                    help="model chunks per pipeline rank; 2 or more runs the interleaved 1F1B "
                         "schedule (micro_batches must then be a multiple of pp_size).  0 "
                         "(default): four chunks when there are pipeline stages, the layers "
                         "allow it and micro_batches divides evenly (measured on two B200: "
                         "40.1k / 41.3k / 41.9k tokens/s with 1 / 2 / 4 chunks), else one")
    ap.add_argument("--micro_batches", type=int, default=4)
    ap.add_argument("--batch_size", type=int, default=1, help="sequences per micro-batch")
    ap.add_argument("--seq_length", type=int, default=2048)
    ap.add_argument("--bitwidth", type=int, default=4)
    ap.add_argument("--backend", default="lowbit", choices=["lowbit", "nccl"])
    ap.add_argument("--stochastic_rounding", action="store_true")
    ap.add_argument("--simulate_quantization", action="store_true")
    ap.add_argument("--no_error_feedback", action="store_true")
    ap.add_argument("--dp_sync", default="pipeline_a", choices=["pipeline_a", "flat", "dense"])
    ap.add_argument("--local_size", type=int, default=1)
    ap.add_argument("--defer_wgrad", action="store_true", default=True,
                    help="pipeline stages run weight-gradient GEMMs after sending the input "
                         "gradient (shrinks the 1F1B bubble; the default)")
    ap.add_argument("--no_defer_wgrad", dest="defer_wgrad", action="store_false",
                    help="weight-gradient GEMMs inside backward, before the input gradient goes")
    ap.add_argument("--max_steps", type=int, default=10)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--dataset", default="synthetic",
                    help="'synthetic', a text file (one document per line) or a token file "
                         "(.bin/.u16/.i32/.i64/.npy); nothing is downloaded")
    ap.add_argument("--dataset_config", default=None,
                    help="accepted for command-line compatibility with the reference; unused")
    ap.add_argument("--tokenizer", default="bytes",
                    help="'bytes', a SentencePiece .model file or a local tokenizer directory")
    ap.add_argument("--use_auth_token", action="store_true",
                    help="accepted for compatibility; there is no download to authorise")
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--model", default="llama7b", choices=["llama7b", "tiny"])
    ap.add_argument("--output_dir", default=None, help="write a checkpoint here at the end")
    ap.add_argument("--save_every", type=int, default=0,
                    help="also write the checkpoint every N steps (0 = only at the end)")
    ap.add_argument("--resume", default=None,
                    help="continue from the per-rank checkpoint files in this directory "
                         "(same parallel layout as the run that wrote them)")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu",
                    choices=["cuda", "cpu"],
                    help="'cpu' runs the same program on CPU ranks over gloo with the ops' host "
                         "paths (plumbing check; use --model tiny)")
    ap.add_argument("--health_check", action="store_true",
                    help="heartbeats through the rendezvous store: a rank that leaves, fails "
                         "or falls silent is noticed on the host before the next step; the "
                         "survivors write a checkpoint (with --output_dir) and stop")
    ap.add_argument("--health_timeout", type=float, default=30.0)
    ap.add_argument("--pg_timeout", type=float, default=None,
                    help="seconds after which a collective without its peer gives up "
                         "(default: torch's process-group default)")
    args = ap.parse_args(argv)

    mcfg = LlamaConfig.llama7b() if args.model == "llama7b" else LlamaConfig.tiny()
    mcfg.attention = _default_attention() if args.device == "cuda" else "sdpa"
    if args.model == "tiny":
        args.seq_length = min(args.seq_length, mcfg.max_seq)
    chunks = args.pp_chunks
    if chunks <= 0:
        chunks = 1
        if args.pp_size > 1 and args.micro_batches % args.pp_size == 0:
            chunks = max(1, min(4, mcfg.num_layers // args.pp_size))
    tcfg = TrainerConfig(
        pp_size=args.pp_size, pp_chunks=chunks, micro_batches=args.micro_batches,
        micro_batch_size=args.batch_size, seq_length=args.seq_length, bitwidth=args.bitwidth,
        stochastic_rounding=args.stochastic_rounding,
        error_feedback=not args.no_error_feedback,
        dp_sync="dense" if args.backend == "nccl" else args.dp_sync,
        local_size=args.local_size, lr=args.lr,
        simulate_quantization=args.simulate_quantization, defer_wgrad=args.defer_wgrad,
        device=args.device, pg_timeout_s=args.pg_timeout)
    trainer = LlamaTrainer(mcfg, tcfg)
    from ..data import build_loader

    # every pipeline stage of a replica reads the same batches (first stage: inputs, last
    # stage: targets), so the sampler is keyed by the data-parallel rank only
    loader = build_loader(args.dataset, args.tokenizer, seq_length=tcfg.seq_length,
                          vocab_size=mcfg.vocab_size, micro_batches=tcfg.micro_batches,
                          micro_batch_size=tcfg.micro_batch_size, dp_size=trainer.dp,
                          dp_rank=trainer.dp_rank, seed=tcfg.seed)
    if args.resume:
        from ..utils.checkpoint import checkpoint_path, load_checkpoint

        if os.path.exists(checkpoint_path(args.resume, trainer.rank)):
            trainer.load_state_dict(load_checkpoint(args.resume, trainer.rank))
    monitor = None
    if args.health_check and dist.is_initialized() and dist.get_world_size() > 1:
        from ..launch import agent_store
        from ..utils.health import HealthMonitor

        # the launcher's store outlives every rank; without a launcher the rendezvous store
        # (hosted by rank 0) has to do
        store = agent_store() or dist.distributed_c10d._get_default_store()
        generation = os.environ.get("BITSCOM_RESTART_COUNT", "0")
        monitor = HealthMonitor(store, trainer.rank, dist.get_world_size(), interval_s=1.0,
                                timeout_s=args.health_timeout,
                                prefix=f"bitscom/health/gen{generation}")
        if getattr(trainer, "lowbit", None) is not None:
            trainer.lowbit.attach_health(monitor)  # also before every gradient bucket
    try:
        _train_loop(args, trainer, loader, tcfg, monitor)
    except Exception as exc:
        from ..utils.health import PeerLostError

        between_steps = isinstance(exc, PeerLostError)
        lost = exc.ranks if between_steps else {}
        if monitor is not None and not between_steps:
            # a collective that has lost its peer fails by itself (connection reset, process
            # group timeout); give the monitor a moment to say whether that is what happened
            deadline = time.monotonic() + args.health_timeout + 2.0
            while not lost and time.monotonic() < deadline:
                lost = monitor.lost()
                time.sleep(0.1)
        if not lost:
            if monitor is not None:
                monitor.report_failure(exc)
            raise
        print(json.dumps({"stopped": str(PeerLostError(lost)), "step": trainer.step_count,
                          "between_steps": between_steps}), flush=True)
        if args.output_dir and between_steps:
            # nothing of this rank in flight: keep what has been learnt.  (After a failure in
            # the middle of a step the last periodic checkpoint stays the one to resume from.)
            from ..utils.checkpoint import save_checkpoint

            save_checkpoint(args.output_dir, trainer.state_dict(), trainer.rank)
        monitor.close()
        os._exit(3)  # no teardown collectives: the peer would never answer
    if args.output_dir:
        from ..utils.checkpoint import save_checkpoint

        trainer.check_kernels()
        save_checkpoint(args.output_dir, trainer.state_dict(), trainer.rank)
    if dist.is_initialized():
        dist.barrier()
        if monitor is not None:
            monitor.leave()  # after the barrier: nobody is still stepping
        import bitscom_b200

        bitscom_b200.shutdown()  # symmetric blocks released with a handshake among the ranks
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
