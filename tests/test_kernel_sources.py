"""Rules that the kernels' sources keep, checked by reading them.

A kernel that is launched with programmatic dependent launch is resident while the kernel in
front of it still runs, and reads that kernel's results after ``griddepcontrol.wait``. A pointer
parameter declared ``__restrict__`` promises the compiler that nothing else touches the data
during the kernel, which allows it to fetch the data (through the read-only path) ahead of the
wait. That happened once to the kernel that merges the attention splits. So in every kernel
that waits for its predecessor only weights, constants and the step's metadata, which are on
the device before the chain starts, may carry the qualifier."""

from __future__ import annotations

import re
from pathlib import Path

KERNELS = Path(__file__).resolve().parent.parent / "llm-inference_b200" / "csrc" / "kernels"

# Parameters that hold weights, constants or step metadata: written before the chain of kernels
# starts, never by a kernel of the chain.
BEFORE_THE_CHAIN = {
    "W", "table", "weight", "bias", "inv_freq", "positions", "token_seq", "seq_kv_len", "block_table",
}


def global_kernels(text: str):
    """(name, parameter list, body) of every ``__global__`` function of a source file."""
    for match in re.finditer(r"__global__\s+void\s+(?:__launch_bounds__\([^)]*\)\s*)?(\w+)\s*\(", text):
        start = match.end()
        depth, at = 1, start
        while depth:
            depth += {"(": 1, ")": -1}.get(text[at], 0)
            at += 1
        params = text[start : at - 1]
        brace = text.index("{", at)
        depth, end = 1, brace + 1
        while depth:
            depth += {"{": 1, "}": -1}.get(text[end], 0)
            end += 1
        yield match.group(1), params, text[brace:end]


def test_kernels_that_wait_for_their_predecessor_keep_restrict_for_what_precedes_the_chain():
    seen = 0
    for path in sorted(KERNELS.glob("*.cu")):
        text = re.sub(r"//[^\n]*", "", path.read_text())
        for name, params, body in global_kernels(text):
            if "wait_for_predecessor" not in body:
                continue
            seen += 1
            for param in params.split(","):
                if "__restrict__" not in param:
                    continue
                pname = param.split()[-1]
                assert pname in BEFORE_THE_CHAIN, (
                    f"{path.name}: {name}({pname}) is __restrict__ in a kernel that runs beside its predecessor")
    assert seen >= 10  # the rule found the kernels it is about


def test_the_rule_reads_a_kernel_as_intended():
    sample = """
    template <typename T>
    __global__ void __launch_bounds__(128)
    demo_kernel(const T* __restrict__ weight, const T* __restrict__ x, int n) {
      wait_for_predecessor();
      if (n) { x[0]; }
    }
    """
    (name, params, body), = list(global_kernels(sample))
    assert name == "demo_kernel" and "wait_for_predecessor" in body
    restricted = [p.split()[-1] for p in params.split(",") if "__restrict__" in p]
    assert restricted == ["weight", "x"] and "x" not in BEFORE_THE_CHAIN
