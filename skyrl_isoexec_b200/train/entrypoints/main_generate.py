"""Generation / evaluation only (reference: R/train/entrypoints/main_generate.py): build the policy and its engine,
optionally load a checkpoint, generate on the evaluation prompts and print reward statistics and pass@k.

    python -m skyrl_isoexec_b200.train.entrypoints.main_generate [--config file.yaml] key=value ...
        [generator.eval_n_samples_per_prompt=4] [trainer.resume_mode=latest trainer.ckpt_path=...] [trainer.export_path=out]

With ``trainer.export_path`` set the per-metric result is also written to ``<export_path>/eval.json``.
"""

from __future__ import annotations

import json
import os
import sys

from ..config import SkyRLTrainConfig
from .main_base import BasePPOExp


def run(cfg: SkyRLTrainConfig) -> dict:
    exp = BasePPOExp(cfg)
    tr = exp.get_trainer()
    tr.build_models()
    t = cfg.trainer
    if t.ckpt_path and t.resume_mode != "none":
        tr.load_checkpoints()
    tr.sync_weights()
    out = tr.eval()
    if t.export_path and exp.rank == 0:
        os.makedirs(t.export_path, exist_ok=True)
        with open(os.path.join(t.export_path, "eval.json"), "w") as f:
            json.dump(out, f, indent=1, sort_keys=True)
    return out


def main(argv=None) -> None:
    args = list(sys.argv[1:] if argv is None else argv)
    path = None
    if args and args[0] in ("--config", "-c"):
        path, args = args[1], args[2:]
    cfg = SkyRLTrainConfig.from_file(path, args) if path else SkyRLTrainConfig.from_cli_overrides(args)
    print(json.dumps(run(cfg), sort_keys=True))


if __name__ == "__main__":
    main()
