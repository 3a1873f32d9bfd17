"""Writes a model folder (config.json, model.safetensors) with seeded random weights.

    python -m llm_inference_b200.cli.random_model --preset tiny-b --seed 0 --out /tmp/tiny
    python -m llm_inference_b200.cli.random_model --config my_config.json --seed 3 --out DIR
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from .presets import PRESETS


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    source = parser.add_mutually_exclusive_group(required=True)
    source.add_argument("--preset", choices=sorted(PRESETS))
    source.add_argument("--config", type=Path, help="a config.json to take the sizes from")
    parser.add_argument("--seed", type=int, default=0)
    parser.add_argument("--std", type=float, default=0.02)
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16", help="how the tensors are stored")
    parser.add_argument("--out", type=Path, required=True)
    args = parser.parse_args(argv)

    import torch

    from .. import models  # noqa: F401
    from ..config import parse_config
    from ..weights import write_model_folder

    raw = PRESETS[args.preset] if args.preset else json.loads(args.config.read_text())
    _, config = parse_config(raw)
    dtype = torch.bfloat16 if args.dtype == "bfloat16" else torch.float32
    folder = write_model_folder(args.out, config, args.seed, std=args.std, dtype=dtype)
    print(f"wrote {folder} ({config.architecture}, seed {args.seed})")
    return 0


if __name__ == "__main__":
    sys.exit(main())
