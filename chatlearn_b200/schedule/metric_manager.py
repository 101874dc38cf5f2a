"""Scalar metric sinks: logger, TensorBoard, wandb.

Parity: chatlearn/schedule/metric_manager.py:24-121 (``prefix/key`` scalars).  A
JSON-lines file under ``log_dir`` is always written on rank 0 so runs on boxes
without TensorBoard/wandb still leave a machine-readable trace.
"""
import json
import os
from typing import Dict

from chatlearn_b200.utils.logger import logger


class MetricManager:
    def __init__(self, global_args):
        self.args = global_args
        la = global_args.runtime_args.log_args_dict
        self.rank0 = int(os.environ.get("RANK", "0")) == 0
        self.tb = self.wandb = None
        self.jsonl = None
        log_dir = getattr(la, "log_dir", None)
        if not self.rank0:
            return
        if isinstance(log_dir, str) and log_dir and log_dir != "???":
            os.makedirs(log_dir, exist_ok=True)
            self.jsonl = os.path.join(log_dir, "metrics.jsonl")
        if getattr(la, "enable_tensorboard", False):
            try:
                from torch.utils.tensorboard import SummaryWriter
                self.tb = SummaryWriter(la.tensorboard_dir or os.path.join(log_dir, "tensorboard"))
            except Exception as e:  # tensorboard is optional
                logger.warning(f"tensorboard unavailable: {e}")
        if getattr(la, "enable_wandb", False):
            try:
                import wandb
                wandb.init(project=la.wandb_project, dir=la.wandb_dir, name=la.wandb_name,
                           id=la.wandb_id, resume=la.wandb_resume)
                self.wandb = wandb
            except Exception as e:
                logger.warning(f"wandb unavailable: {e}")

    def log(self, prefix: str, step: int, scalars: Dict[str, float]):
        if not self.rank0 or not scalars:
            return
        flat = {f"{prefix}/{k}": float(v) for k, v in scalars.items()
                if isinstance(v, (int, float)) or hasattr(v, "item")}
        logger.info(f"[step {step}] " + " ".join(f"{k}={v:.5g}" for k, v in flat.items()))
        if self.jsonl:
            with open(self.jsonl, "a", encoding="utf-8") as f:
                f.write(json.dumps({"step": step, **flat}) + "\n")
        if self.tb:
            for k, v in flat.items():
                self.tb.add_scalar(k, v, step)
        if self.wandb:
            self.wandb.log(flat, step=step)

    def stop(self):
        if self.tb:
            self.tb.close()
        if self.wandb:
            self.wandb.finish()
