"""Command-line entry of the trainers:

    python -m mlperf_training_b200.trainer.cli pretrain  --config <experiment.yaml> [key=value ...]
    python -m mlperf_training_b200.trainer.cli posttrain --config <experiment.yaml> [key=value ...]
    python -m mlperf_training_b200.trainer.cli hstu      --config <experiment.yaml> [key=value ...]
    python -m mlperf_training_b200.trainer.cli flux      --config <experiment.yaml> [key=value ...]
    python -m mlperf_training_b200.trainer.cli <mode>    --config <experiment.yaml> --print-config   # what would run

The experiment YAML is resolved with ``${ENV:default}`` substitution and ``key=value`` overrides
(the reference's ``primus-cli direct -- train pretrain --config $EXP`` surface,
small_llm_pretraining/primus/run_and_time.sh:60-63).  Under ``torchrun`` the process group is
initialised from ``RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT``.
"""
from __future__ import annotations

import argparse
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="b200-train")
    ap.add_argument("mode", choices=["pretrain", "posttrain", "hstu", "flux"])
    ap.add_argument("--config", required=True)
    ap.add_argument("--device", default=None)
    ap.add_argument("--print-config", action="store_true", help="print the resolved experiment of this trainer and exit")
    ap.add_argument("overrides", nargs="*")
    args = ap.parse_intermixed_args(argv)      # key=value overrides may follow the options

    if os.environ.get("B200_QUIET", "0") not in ("", "0"):
        from ..mllog import suppress
        suppress.install()

    import torch
    import torch.distributed as dist
    from ..config.loader import load_experiment

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 and not dist.is_initialized():
        use_cuda = torch.cuda.is_available() and (args.device or "cuda") != "cpu"
        if use_cuda:
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
        dist.init_process_group("nccl" if use_cuda else "gloo")
    exp = load_experiment(args.config, overrides=args.overrides)
    module = {"pretrain": "pre_trainer", "posttrain": "post_trainer", "hstu": "hstu_trainer", "flux": "flux_trainer"}[args.mode]
    resolved = (exp.get("modules") or {}).get(module, {}).get("resolved") or exp
    if args.print_config:
        import yaml
        print(yaml.safe_dump(resolved, sort_keys=False, default_flow_style=False))
        return 0
    if os.environ.get("SELF_CHECK", "0") not in ("", "0"):
        # kernels against their eager oracle before anything is timed; a disagreement stops the run here
        from ..ops.selfcheck import run_selfcheck
        run_selfcheck(args.device or ("cuda" if torch.cuda.is_available() else "cpu"), verbose=int(os.environ.get("RANK", "0")) == 0)
    from ..parallel import health
    try:
        if args.mode == "pretrain":
            from .loop import run
            out = run(resolved, device=args.device)
        elif args.mode == "posttrain":
            from .sft import run as run_sft
            out = run_sft(resolved, device=args.device)
        elif args.mode == "hstu":
            from .hstu import run as run_hstu
            out = run_hstu(resolved, device=args.device)
        else:
            from .flux import run as run_flux
            out = run_flux(resolved, device=args.device)
    except health.RankFailure as e:
        # a peer stopped answering between steps: leave without touching the process group (a collective
        # with a dead peer would hang) and tell the supervisor which kind of failure this was
        print(f"rank failure detected: ranks {e.ranks} are silent; exiting {health.EXIT_RANK_FAILURE}", file=sys.stderr, flush=True)
        health.clean_exit(health.EXIT_RANK_FAILURE)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0 if out is not None else 1


if __name__ == "__main__":
    sys.exit(main())
