"""Tracing helpers on CPU: a disabled PhaseTimer is a no-op, StepProfiler writes a chrome trace
of the chosen steps, and the SFT entry point honours --profile."""
import json

import torch


def test_phase_timer_without_cuda_is_a_noop():
    from easy_to_hard_b200.utils.tracing import PhaseTimer
    t = PhaseTimer()
    with t.phase("x"):
        torch.ones(4).sum()
    assert t.enabled == torch.cuda.is_available()
    if not t.enabled:
        assert t.totals_ms() == {} and t.summary() == {}


def test_step_profiler_writes_a_trace(tmp_path):
    from easy_to_hard_b200.utils.tracing import StepProfiler
    p = StepProfiler(tmp_path / "trace", skip=1, active=2)
    x = torch.randn(64, 64)
    for _ in range(5):
        p.step()
        x = x @ x.t() / 64
    assert p.close() is None                      # already closed after the active window
    outs = sorted(tmp_path.glob("trace*.json"))     # "_rank_<r>" is added under a process group
    assert len(outs) == 1
    events = json.loads(outs[0].read_text())["traceEvents"]
    assert any("mm" in str(e.get("name", "")) for e in events)
    none = StepProfiler(None)
    none.step()
    assert none.close() is None
