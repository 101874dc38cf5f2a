"""Command line: ``python -m chatlearn_b200 grpo --config-file X.yaml key=value …``.

Parity: chatlearn/entrypoint.py:29-124 (sub-command per registered algorithm,
dataclass schema merged with an external YAML and dot-list overrides, then
``validate()`` and ``run()``).  Extra: ``--nproc N`` forks N local ranks (one per
GPU, or CPU/gloo ranks with ``--cpu``) when the process was not started by
torchrun; a supervisor watches them and stops the job if one dies.
"""
import argparse
import os
import sys
from typing import Dict, List, Optional, Tuple, Type

from chatlearn_b200.configs import ConfigError, apply_dotlist, load_yaml, missing_keys, resolve, to_dataclass

ALGO_REGISTRY: Dict[str, Tuple[str, str, str]] = {
    # name: (module, algorithm class, config class)
    "grpo": ("chatlearn_b200.algorithm.grpo", "GrpoAlgorithm", "GrpoConfig"),
    "rlhf": ("chatlearn_b200.algorithm.rlhf", "RlhfAlgorithm", "RlhfConfig"),
}


def _load_algo(name: str):
    import importlib
    mod, algo, cfg = ALGO_REGISTRY[name]
    m = importlib.import_module(mod)
    return getattr(m, algo), getattr(m, cfg)


def compose_config(cfg_cls: Type, config_file: Optional[str], overrides: List[str]):
    data = load_yaml(config_file) if config_file else {}
    data = apply_dotlist(data, overrides)
    data = resolve(data)
    cfg = to_dataclass(cfg_cls, data)
    miss = missing_keys(cfg)
    if miss:
        raise ConfigError("missing mandatory config values: " + ", ".join(miss))
    return cfg


class ChatlearnLauncher:
    def __init__(self):
        self.parser = self._create_parser()

    def _create_parser(self):
        p = argparse.ArgumentParser(prog="chatlearn_b200", description="RL post-training launcher")
        sub = p.add_subparsers(dest="algorithm", required=True)
        for name in ALGO_REGISTRY:
            sp = sub.add_parser(name)
            sp.add_argument("--config-file", type=str, default=None)
            sp.add_argument("--nproc", type=int, default=0, help="fork this many local ranks")
            sp.add_argument("--cpu", action="store_true", help="CPU/gloo ranks (plumbing runs)")
            sp.add_argument("overrides", nargs=argparse.REMAINDER, help="key=value overrides")
        return p

    def _run_algorithm(self, name: str, config_file: Optional[str], overrides: List[str]):
        algo_cls, cfg_cls = _load_algo(name)
        cfg = compose_config(cfg_cls, config_file, [o for o in overrides if o != "--"])
        algo = algo_cls(cfg)
        algo.validate()
        return algo.run()

    def run(self, argv=None):
        args = self.parser.parse_args(argv)
        if args.nproc and "RANK" not in os.environ:
            from chatlearn_b200.launcher.local import launch_local
            child = [sys.executable, "-m", "chatlearn_b200", args.algorithm]
            if args.config_file:
                child += ["--config-file", args.config_file]
            if args.cpu:
                child.append("--cpu")
            child += args.overrides
            return launch_local(child, args.nproc, cpu=args.cpu)
        if args.cpu:
            os.environ["CHATLEARN_FORCE_CPU"] = "1"
        return self._run_algorithm(args.algorithm, args.config_file, args.overrides)


def main(argv=None):
    return ChatlearnLauncher().run(argv)


if __name__ == "__main__":
    main()
