"""Opens a model folder, validates it against the registered architecture and prints its
configuration and tensor table; exits 1 if the folder is invalid (the counterpart of the
reference's ``instinct-inspect-model``, tools/inspect_model.cpp).

    python -m llm_inference_b200.cli.inspect_model DIR
"""

from __future__ import annotations

import argparse
import sys
from dataclasses import asdict
from pathlib import Path


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("model", type=Path)
    args = parser.parse_args(argv)

    from .. import models  # noqa: F401
    from ..config import ConfigError, parse_config, read_config_json
    from ..parts.model import Model
    from ..weights import SafetensorsError, SafetensorsFile, WeightsError, checkpoint_files, load_weights

    try:
        entry, config = parse_config(read_config_json(args.model))
        model = Model(entry.recipe(config))
        load_weights(args.model, model.tensor_specs())
    except (ConfigError, WeightsError, SafetensorsError, FileNotFoundError) as exc:
        print(f"invalid model: {exc}", file=sys.stderr)
        return 1
    print(f"architecture: {entry.name}")
    for key, value in asdict(config).items():
        print(f"  {key}: {value}")
    total = 0
    for path in checkpoint_files(args.model):
        with SafetensorsFile(path) as file:
            for name, info in sorted(file.tensors.items()):
                count = 1
                for s in info.shape:
                    count *= s
                total += count
                print(f"{name}  {str(info.dtype).removeprefix('torch.')}  {list(info.shape)}")
    print(f"{total} parameters stored; valid")
    return 0


if __name__ == "__main__":
    sys.exit(main())
