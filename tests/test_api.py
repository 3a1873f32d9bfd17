"""The Python entry point's checks that need no GPU: names, options and refusals
(python/instinct/__init__.py:27-50 and python/instinct/sampling.py:19-41 in the reference)."""

from __future__ import annotations

import pytest
import torch

import llm_inference_b200 as package
from llm_inference_b200 import SamplingParams, create_engine

from helpers import TINY, make_model_folder


def test_public_names():
    assert set(package.__all__) == {"SamplingParams", "SequenceState", "TokenEvent", "build_info", "create_engine"}
    info = package.build_info()
    assert info["backend"] == "b200" and info["arch"] == "sm_100a" and info["cuda_available"] == torch.cuda.is_available()
    assert {s.value for s in package.SequenceState} == {"waiting", "prefilling", "running", "completed", "cancelled", "rejected"}


@pytest.mark.parametrize(
    "bad",
    [dict(temperature=-0.1), dict(temperature=10.5), dict(temperature=float("nan")), dict(top_p=0.0), dict(top_p=1.01),
     dict(top_k=-1), dict(top_k=1.5), dict(min_p=1.0), dict(min_p=-0.1), dict(seed=1.5)],
)
def test_sampling_parameters_are_validated(bad):
    with pytest.raises(ValueError):
        SamplingParams(**bad)


def test_python_and_scheduler_hold_the_same_sampling_ranges():
    from llm_inference_b200.csrc.host_module import host
    from llm_inference_b200.sampling.params import RANGES

    native = host().sampling_ranges()
    assert {name: tuple(r) for name, r in RANGES.items()} == {name: tuple(r) for name, r in native.items()}
    with pytest.raises(ValueError, match="top_p"):
        host().SamplingParams(0.5, 0.0, 0, 0.0, None)
    with pytest.raises(ValueError, match="temperature.*min_p"):
        SamplingParams(temperature=11.0, min_p=1.0)


def test_sampling_defaults_and_greedy():
    assert SamplingParams() == SamplingParams(temperature=0.0, top_p=1.0, top_k=0, min_p=0.0, seed=None)
    assert SamplingParams().greedy and SamplingParams(temperature=0.8, top_k=1).greedy
    assert not SamplingParams(temperature=0.8, seed=3).greedy


def test_create_engine_refuses_what_it_cannot_run(tmp_path):
    with pytest.raises(ValueError, match="unknown backend"):
        create_engine(tmp_path, backend="mlx")
    with pytest.raises(ValueError, match="model folder"):
        create_engine()
    folder = make_model_folder(tmp_path / "tiny", TINY["A"], seed=1)
    with pytest.raises(ValueError, match="kernels="):
        create_engine(folder, kernels="fast")
    with pytest.raises(ValueError, match="chunk"):
        create_engine(folder, prefill_chunk_size=64, prefill_burst_size=32)
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CPU path"):
            create_engine(folder)
