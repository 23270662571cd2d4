"""Kernel timeline: when every CTA of every kernel of this package entered, got past its wait and left.

Built only when the environment has CISR_TRACE=1 at the time the kernels are compiled and loaded (the libraries
then carry the recording code and get names of their own, so ordinary builds are untouched).  `read()` drains the
records of every loaded library; `write_chrome_trace()` writes them in the Trace Event format that chrome://tracing
and Perfetto open: one row per SM, one slice per CTA, the part before the wait in a lighter slice.
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import Dict, List

import numpy as np

from . import build

KERNEL_NAMES = {
    1: "embedding", 2: "add_rmsnorm", 3: "swiglu", 4: "rotary_table", 5: "rope_store", 6: "page_copy", 7: "table_update",
    8: "attn_prefill", 9: "attn_decode (gather)", 10: "attn_decode (tensor maps)", 11: "attn_merge", 12: "sample",
    13: "decode_advance", 14: "skinny plain", 15: "skinny swiglu", 16: "skinny rope", 17: "gemm_tcgen05", 18: "attention (CUDA cores)", 19: "stream_gemm", 20: "merge + output projection",
}
RECORD = np.dtype([("entered", "<u8"), ("waited", "<u8"), ("left", "<u8"), ("marks", "<u8", (4,)), ("kernel", "<i4"),
                   ("block", "<i4"), ("sm", "<i4"), ("pad", "<i4")])
CAPACITY = 1 << 17


def enabled() -> bool:
    return os.environ.get("CISR_TRACE", "0") not in ("", "0")


def read() -> np.ndarray:
    """All records since the last read, from every loaded library, sorted by entry time."""
    if not enabled():
        raise RuntimeError("the kernel timeline needs CISR_TRACE=1 in the environment before the kernels are loaded")
    parts: List[np.ndarray] = []
    for lib in list(build._loaded.values()):
        if not hasattr(lib, "cisr_trace_read"):
            continue
        lib.cisr_trace_read.restype = ctypes.c_int
        buf = np.zeros(CAPACITY, dtype=RECORD)
        n = lib.cisr_trace_read(buf.ctypes.data_as(ctypes.c_void_p), CAPACITY)
        if n < 0:
            raise RuntimeError("reading the kernel timeline failed")
        parts.append(buf[:n])
    records = np.concatenate(parts) if parts else np.zeros(0, dtype=RECORD)
    return records[np.argsort(records["entered"], kind="stable")]


def summary(records: np.ndarray) -> List[Dict[str, object]]:
    """Per launch (a run of records of one kernel that overlap in time): first entry, last exit, CTAs, medians."""
    launches: List[Dict[str, object]] = []
    if records.size == 0:
        return launches
    t0 = int(records["entered"].min())
    current = None
    for r in records:
        if current is None or r["kernel"] != current["kernel_id"] or int(r["entered"]) - t0 > current["end"] + 50_000:
            current = {"kernel_id": int(r["kernel"]), "kernel": KERNEL_NAMES.get(int(r["kernel"]), str(int(r["kernel"]))),
                       "begin": int(r["entered"]) - t0, "end": int(r["left"]) - t0, "ctas": 0, "released": []}
            launches.append(current)
        current["ctas"] += 1
        current["end"] = max(current["end"], int(r["left"]) - t0)
        if r["waited"]:
            current["released"].append(int(r["waited"]) - t0)
    for launch in launches:
        released = launch.pop("released")
        launch["released"] = int(np.median(released)) if released else None
    return launches


def write_chrome_trace(records: np.ndarray, path: str) -> None:
    events = []
    if records.size:
        t0 = int(records["entered"].min())
        for r in records:
            name = KERNEL_NAMES.get(int(r["kernel"]), str(int(r["kernel"])))
            begin, end = (int(r["entered"]) - t0) / 1e3, (int(r["left"]) - t0) / 1e3
            args = {"block": int(r["block"])}
            if r["waited"]:
                waited = (int(r["waited"]) - t0) / 1e3
                events.append({"name": name + " (before its wait)", "ph": "X", "ts": begin, "dur": max(waited - begin, 0.001),
                               "pid": 0, "tid": int(r["sm"]), "args": args})
                begin = waited
            events.append({"name": name, "ph": "X", "ts": begin, "dur": max(end - begin, 0.001), "pid": 0, "tid": int(r["sm"]),
                           "args": args})
    with open(path, "w") as f:
        json.dump({"traceEvents": events, "displayTimeUnit": "ns"}, f)
