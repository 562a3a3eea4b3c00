"""Same-config reference arm for the multi-model benchmark: the UNMODIFIED reference code
(``benchmarks/multimodel_stochastic_e2e_curve.py`` copied beside the installed library under
``baseline/_ref/benchmarks/``) trains ResNet-50 / small BERT / small GPT-2 with ITS
``_run_train`` loop, its bucketed gradient sync (``:207-244``) and its ``bitscom.LowBitGroup``,
on the settings of ``bitscom_b200.bench.multimodel_e2e_curve`` (fp32 torch models on both
sides; only the gradient path differs).

    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        baseline/reference_multimodel.py --models resnet50 --resnet-steps 8

Two substitutions, both forced:
  * the reference script opens ``dist.init_process_group(backend="lowbit")``; that C++ backend
    dies with SIGSEGV in its constructor under torch 2.11 (see ``reference_collective.py``), so
    the group is NCCL.  ``LowBitGroup``'s Python pipeline only ever asks the group for
    ``all_to_all`` / ``all_gather``, which the lowbit backend forwards to NCCL anyway
    (``cpp/src/process_group_lowbit.cc:1779-1786,1660-1668``), so the measured path is the same;
  * ``matplotlib`` (imported by the script for its PNG files) is not installed: a stand-in
    module is registered and no plot is drawn.
If the copy of the script or one of its model packages is missing, one ``unavailable`` line is
printed and the exit code is 0.
"""

from __future__ import annotations

import argparse
import importlib.util
import json
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SCRIPT = os.path.join(REF, "benchmarks", "multimodel_stochastic_e2e_curve.py")


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def _load_reference_script():
    if "matplotlib" not in sys.modules:
        try:
            import matplotlib.pyplot  # noqa: F401
        except Exception:
            plt = types.ModuleType("matplotlib.pyplot")
            root = types.ModuleType("matplotlib")
            root.pyplot = plt
            root.use = lambda *a, **k: None
            sys.modules["matplotlib"], sys.modules["matplotlib.pyplot"] = root, plt
    sys.path.insert(0, REF)
    spec = importlib.util.spec_from_file_location("_reference_multimodel", SCRIPT)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--models", nargs="+", default=["resnet50"],
                    choices=["resnet50", "bert", "gpt2"])
    ap.add_argument("--modes", nargs="+", default=["lowbit_no_sr", "lowbit_sr", "nocompress"])
    ap.add_argument("--bitwidth", type=int, default=4)
    ap.add_argument("--resnet-steps", type=int, default=8)
    ap.add_argument("--resnet-batch-size", type=int, default=16)
    ap.add_argument("--nlp-steps", type=int, default=160)
    ap.add_argument("--nlp-batch-size", type=int, default=4)
    ap.add_argument("--out", default="bench_outputs/reference_multimodel.jsonl")
    cli = ap.parse_args()
    if not os.path.exists(SCRIPT):
        _unavailable("baseline/_ref/benchmarks/multimodel_stochastic_e2e_curve.py is not there: "
                     "copy the reference's benchmarks folder beside the installed library")
        return
    try:
        ref = _load_reference_script()
        import bitscom
        import torch
        import torch.distributed as dist

        assert os.path.realpath(bitscom.__file__).startswith(os.path.realpath(REF))
    except BaseException as exc:
        _unavailable(f"{type(exc).__name__}: {str(exc)[:200]}")
        return

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    world = dist.get_world_size()
    # the reference's own defaults for everything this driver does not set
    args = argparse.Namespace(
        models=cli.models, bitwidth=cli.bitwidth, steps=80, batch_size=8, dataset_size=512,
        resnet_steps=cli.resnet_steps, resnet_batch_size=cli.resnet_batch_size,
        resnet_dataset_size=None, resnet_grad_clip_norm=None, resnet_warmup_ratio=None,
        resnet_min_lr_ratio=None, nlp_steps=cli.nlp_steps, nlp_batch_size=cli.nlp_batch_size,
        nlp_dataset_size=1024, nlp_grad_clip_norm=0.8, nlp_warmup_ratio=0.08,
        nlp_min_lr_ratio=0.05, lr_resnet=2e-4, lr_resnet_sr=1.5e-4, lr_bert=2.5e-4,
        lr_gpt2=2e-4, weight_decay=1e-2, warmup_ratio=0.1, min_lr_ratio=0.1, seed=2026,
        data_seed=17, grad_clip_norm=1.0, grad_bucket_numel=4_000_000,
        disable_grad_bucket=False, smooth_window=4, profile_trace=False,
        profile_model="resnet50", profile_modes=[], profile_steps=0,
        out_dir="bench_outputs", resnet_image_size=224, resnet_num_classes=20, bert_seq_len=64,
        bert_hidden=256, bert_layers=4, bert_heads=4, bert_num_labels=2, gpt2_seq_len=64,
        gpt2_hidden=256, gpt2_layers=4, gpt2_heads=4)
    rows = []
    try:
        for name in cli.models:
            cfg = ref._get_train_cfg(name, args)
            for mode in cli.modes:
                torch.manual_seed(args.seed)
                torch.cuda.manual_seed_all(args.seed)
                if name == "resnet50":
                    model = ref._build_resnet50_model(args.resnet_num_classes)
                    data = ref._build_dataset_resnet50(
                        rank=rank, dataset_size=cfg["dataset_size"],
                        image_size=args.resnet_image_size, num_classes=args.resnet_num_classes,
                        base_seed=args.data_seed)
                elif name == "bert":
                    model = ref._build_bert_model(args.bert_num_labels, args.bert_hidden,
                                                  args.bert_layers, args.bert_heads)
                    data = ref._build_dataset_bert(
                        rank=rank, dataset_size=cfg["dataset_size"], seq_len=args.bert_seq_len,
                        num_labels=args.bert_num_labels, base_seed=args.data_seed)
                else:
                    model = ref._build_gpt2_model(args.gpt2_hidden, args.gpt2_layers,
                                                  args.gpt2_heads)
                    data = ref._build_dataset_gpt2(
                        rank=rank, dataset_size=cfg["dataset_size"], seq_len=args.gpt2_seq_len,
                        base_seed=args.data_seed)
                stats = ref._run_train(
                    model_name=name, mode=mode, model=model, dataset=data, train_cfg=cfg,
                    args=args, rank=rank, world_size=world, lowbit_pg=dist.group.WORLD,
                    nccl_pg=dist.group.WORLD, device=device)
                row = {"impl": "reference", "model": name,
                       "arm": "no_compression" if mode == "nocompress" else mode,
                       "world": world, "bitwidth": cli.bitwidth, "steps": cfg["steps"],
                       "batch_size": cfg["batch_size"],
                       "avg_step_time_ms": float(stats["avg_step_time_ms"]),
                       "throughput_samples_per_s": float(stats["throughput_samples_per_s"]),
                       "first_loss": float(stats["losses"][0]),
                       "final_loss": float(stats["losses"][-1]),
                       "timing": "the reference's own: host clock around synchronize, all steps"}
                rows.append(row)
                if rank == 0:
                    print(json.dumps(row), flush=True)
                del model
                torch.cuda.empty_cache()
    except BaseException as exc:
        _unavailable(f"{type(exc).__name__}: {str(exc)[:300]}")
    if rank == 0 and cli.out and rows:
        os.makedirs(os.path.dirname(cli.out) or ".", exist_ok=True)
        with open(cli.out, "a") as f:
            for r in rows:
                f.write(json.dumps(r) + "\n")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
