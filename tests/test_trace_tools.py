"""Host-side trace post-processing (catccos_b200/trace.py) on a synthetic trace buffer."""
import json

import numpy as np

from catccos_b200 import trace


def _buffer():
    t = np.zeros((4, trace.SLOTS), dtype=np.int64)
    base = 1_000_000_000
    for cta in range(3):                       # the fourth CTA never ran
        t[cta, 0] = base + 100 * cta           # start
        t[cta, 1] = base + 500_000 + 1000 * cta
        t[cta, 3] = 13_000 + cta               # waited for pushed rows
        t[cta, 8], t[cta, 9] = 500, 80_000
        t[cta, 10] = 7 - cta % 2
    t[0, 2] = base + 90_000
    t[0, 4], t[0, 5] = base + 300, base + 180_000
    return t


def test_summary_uses_only_ctas_that_ran():
    s = trace.summarize(_buffer())
    assert s["ctas"] == 3 and abs(s["span_us"] - 502.0) < 1e-9
    assert s["start"] == (0.0, 0.1, 0.2)
    assert s["mma_wait_smem_us"] == (80.0, 80.0, 80.0)
    assert s["prod_wait_us"][1] == 13.001 and s["tiles"] == (6, 7)
    assert s["push_end"] == (180.0, 180.0, 180.0)
    assert trace.summarize(np.zeros((2, trace.SLOTS)))["ctas"] == 0


def test_chrome_trace_has_one_span_per_cta_and_the_push_phase(tmp_path):
    path = tmp_path / "t.json"
    trace.write_chrome_trace(str(path), _buffer(), rank=3, name="pair_agmm")
    ev = json.loads(path.read_text())["traceEvents"]
    spans = [e for e in ev if e["name"] == "pair_agmm"]
    assert len(spans) == 3 and {e["tid"] for e in spans} == {0, 1, 2} and all(e["pid"] == 3 for e in ev)
    assert abs(spans[0]["dur"] - 500.0) < 1e-9 and spans[1]["ts"] == 0.1
    push = [e for e in ev if e["name"] == "push"]
    assert len(push) == 1 and abs(push[0]["dur"] - 179.7) < 1e-9
    assert sum(e["ph"] == "i" for e in ev) == 1
    assert spans[0]["args"]["mma_wait_smem_us"] == 80.0 and spans[0]["args"]["tiles"] == 7
