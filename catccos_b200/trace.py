"""Per-CTA device traces (`catccos_debug_set_trace`) -> summaries and chrome://tracing JSON.

The reference dumps its AscendTimer buffers to `output_timer/timer_rank_N.csv` and converts them
with tests/dynamic_tiling/utils/process.py (tools/README.md:96-125); this is the counterpart for the
`%globaltimer` slots the CUDA kernels fill (TraceSlot in csrc/common.h): slot 0/1 kernel start/end
of the CTA, 2 first wait for pushed rows, 3 total such wait, 4/5 push begin/end, 6 epilogue waits
for peers, 7 epilogue drain time, 8/9 MMA thread waiting for TMEM / for operands, 10 tiles done.
Works on a host copy of the buffer (numpy int64/uint64 array [ctas, 16]); nothing here touches a device."""
import json

import numpy as np

SLOTS = 16
STAMPS = {"start": 0, "end": 1, "prod_wait_first": 2, "push_begin": 4, "push_end": 5}
TOTALS = {"prod_wait_ns": 3, "epi_wait_ns": 6, "epi_store_ns": 7, "mma_wait_tmem_ns": 8, "mma_wait_smem_ns": 9}
TILES = 10


def _as_table(buf):
    t = np.asarray(buf).astype(np.int64).reshape(-1, SLOTS)
    return t[t[:, 0] > 0]            # CTAs that ran


def summarize(buf):
    """{'span_us', 'ctas', per stamp: (min, median, max) in us from the first CTA start, per total: the same in us,
    'tiles': (min, max)}."""
    t = _as_table(buf)
    if len(t) == 0:
        return {"ctas": 0, "span_us": 0.0}
    t0 = t[:, 0].min()
    out = {"ctas": int(len(t)), "span_us": float(t[:, 1].max() - t0) / 1e3}
    for name, s in STAMPS.items():
        col = t[:, s]
        col = col[col > 0]
        if len(col):
            rel = (col - t0) / 1e3
            out[name] = (float(rel.min()), float(np.median(rel)), float(rel.max()))
    for name, s in TOTALS.items():
        col = t[:, s] / 1e3
        out[name.replace("_ns", "_us")] = (float(col.min()), float(np.median(col)), float(col.max()))
    out["tiles"] = (int(t[:, TILES].min()), int(t[:, TILES].max()))
    return out


def to_chrome_trace(buf, rank=0, name="kernel"):
    """Events for chrome://tracing / Perfetto: one track per CTA with the kernel span and, where recorded,
    the push phase; waits appear as counters-in-args (they are totals, not intervals)."""
    t = np.asarray(buf).astype(np.int64).reshape(-1, SLOTS)
    ran = t[:, 0] > 0
    if not ran.any():
        return {"traceEvents": []}
    t0 = t[ran, 0].min()
    ev = []
    for cta in np.nonzero(ran)[0]:
        row = t[cta]
        args = {k.replace("_ns", "_us"): float(row[s]) / 1e3 for k, s in TOTALS.items() if row[s] > 0}
        args["tiles"] = int(row[TILES])
        ev.append({"name": name, "ph": "X", "pid": int(rank), "tid": int(cta), "ts": float(row[0] - t0) / 1e3,
                   "dur": float(row[1] - row[0]) / 1e3, "args": args})
        if row[4] > 0 and row[5] >= row[4]:
            ev.append({"name": "push", "ph": "X", "pid": int(rank), "tid": int(cta), "ts": float(row[4] - t0) / 1e3,
                       "dur": float(row[5] - row[4]) / 1e3})
        if row[2] > 0:
            ev.append({"name": "first wait for pushed rows", "ph": "i", "s": "t", "pid": int(rank), "tid": int(cta),
                       "ts": float(row[2] - t0) / 1e3})
    return {"traceEvents": ev, "displayTimeUnit": "ns"}


def write_chrome_trace(path, buf, rank=0, name="kernel"):
    with open(path, "w") as f:
        json.dump(to_chrome_trace(buf, rank, name), f)
