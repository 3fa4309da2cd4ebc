"""Command line: ``lset-b200 train|eval --config x.yaml [--section.field value ...]``.

Same commands, flags and exit codes as the reference CLI (lset/cli.py:32-110): ``train`` loads the
YAML, applies dotted overrides, validates, and when ``dp_size * tp_size > 1`` re-executes itself
under ``python -m torch.distributed.run`` (one process per GPU, rendezvous on 127.0.0.1, optional
``--max-restarts`` from ``distributed.max_restarts``) and exits with the launcher's return code;
``eval`` runs the MTEB evaluation; no or unknown command prints the help and exits 1.
"""
from __future__ import annotations

import subprocess
import sys

HELP_TEXT = """\
lset-b200 - embedding-model trainer for NVIDIA B200

Commands:
  train       Train an embedding model
  eval        Evaluate with MTEB

Usage:
  lset-b200 train --config configs/qwen3_embed_quick.yaml [--section.field value ...]
  lset-b200 eval  --config configs/qwen3_embed_quick.yaml [--eval.tasks STS12,STS13 ...]

Examples:
  lset-b200 train --config configs/qwen3_embed_packed.yaml --training.max_steps 100
  lset-b200 train --config configs/distributed_8gpu.yaml --distributed.dp_size 8
  lset-b200 eval  --config configs/qwen3_embed_quick.yaml --eval.tasks STSBenchmark
"""


def _config_path(args):
    for i, a in enumerate(args[:-1]):
        if a == "--config":
            return args[i + 1]
    return None


def _load(args, usage: str):
    from .config import LSETConfig, parse_overrides

    path = _config_path(args)
    if not path:
        print("Error: --config is required\n")
        print(f"Usage: lset-b200 {usage} --config <config.yaml> [overrides...]")
        sys.exit(1)
    cfg = LSETConfig.from_yaml(path)
    overrides = parse_overrides(args)
    cfg.apply_overrides(overrides)
    return cfg, path, overrides


def _rendezvous_port() -> int:
    """``MASTER_PORT`` when the caller set one, else a port that is free right now (two jobs on
    one machine must not meet on the launcher's default port)."""
    import os
    import socket

    if os.environ.get("MASTER_PORT", "").isdigit():
        return int(os.environ["MASTER_PORT"])
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launcher_command(config, config_path: str, overrides) -> list:
    """The torchrun command line that ``train`` re-executes for a multi-GPU job."""
    world = config.distributed.dp_size * config.distributed.tp_size
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
           f"--nproc_per_node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(_rendezvous_port())]
    if config.distributed.max_restarts > 0:
        cmd.append(f"--max-restarts={config.distributed.max_restarts}")
    cmd += ["-m", "lset_b200.train.main", "--config", config_path]
    for k, v in overrides:
        cmd += [f"--{k}", v]
    return cmd


def cmd_train(args):
    cfg, path, overrides = _load(args, "train")
    cfg.validate()
    for field, value in (("model.path", cfg.model.path), ("data.train_path", cfg.data.train_path)):
        if not value:
            print(f"Error: {field} is required for train (set it in the YAML file or with --{field})")
            sys.exit(1)
    if cfg.distributed.dp_size * cfg.distributed.tp_size > 1:
        sys.exit(subprocess.run(launcher_command(cfg, path, overrides)).returncode)
    from .train.main import train

    train(cfg)


def cmd_eval(args):
    cfg, _, _ = _load(args, "eval")
    from .eval.run import run_eval

    run_eval(cfg)


def main(argv=None):
    argv = sys.argv[1:] if argv is None else list(argv)
    if not argv:
        print(HELP_TEXT)
        sys.exit(1)
    command, rest = argv[0], argv[1:]
    if command == "train":
        cmd_train(rest)
    elif command == "eval":
        cmd_eval(rest)
    elif command in ("-h", "--help", "help"):
        print(HELP_TEXT)
    else:
        print(f"Unknown command: {command}\n")
        print(HELP_TEXT)
        sys.exit(1)


if __name__ == "__main__":
    main()
