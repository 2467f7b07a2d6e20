"""Source-level conventions of the CUDA kernels that a CPU box can check."""
import re
from pathlib import Path

CSRC = Path(__file__).resolve().parent.parent / "easy_to_hard_b200" / "ops" / "csrc"


def _kernel_bodies(text):
    """name -> source text of every __global__ function of a file."""
    out = {}
    for m in re.finditer(r"__global__\s+void(?:\s+__launch_bounds__\([^)]*\))?\s+(\w+)\s*\(", text):
        start = text.index("{", m.end())
        depth, i = 0, start
        while True:
            c = text[i]
            depth += c == "{"
            depth -= c == "}"
            if depth == 0:
                break
            i += 1
        out[m.group(1)] = text[start:i]
    return out


def test_every_kernel_given_to_the_pdl_launch_helper_waits_for_its_predecessor():
    """launch() (launch.cuh) may attach programmatic dependent launch: a kernel started that way
    can run before its predecessor has finished, so it must execute griddepcontrol.wait
    (pdl_wait_prior) before it touches global memory."""
    checked = 0
    for src in sorted(CSRC.glob("*.cu")):
        text = src.read_text()
        bodies = _kernel_bodies(text)
        for m in re.finditer(r"[^\w]launch\(\s*(\w+)(?:<[^>]*>)?\s*,", text):
            name = m.group(1)
            if name not in bodies:
                continue
            assert "pdl_wait_prior()" in bodies[name], f"{src.name}: {name}"
            checked += 1
    assert checked >= 8
