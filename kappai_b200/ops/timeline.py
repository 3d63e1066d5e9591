"""Device timeline of the kernels of a step.

The kernel libraries have a second build (``-DKP_TRACE``) in which thread 0 of
every CTA notes the GPU's global timer when it enters a kernel and when its wait
on the kernel before it is over; the matrix-product kernels also note the end of
a CTA's work.  Read back after a few steps, the records show how the kernels of
a captured step follow and overlap one another: where the time of a decode step
goes when no single kernel is the step.  A traced step runs 10 to 15 % slower
(an atomic a mark), so the figures are for shares and gaps.

    from kappai_b200.ops import timeline
    timeline.enable()                    # before the first kernel library is loaded
    ... run steps ...
    rec = timeline.records()             # and clear
    for k in timeline.kernels(rec): ...

``bench.py --probe timeline`` prints the table for a decode step.
"""
from __future__ import annotations

import ctypes
from typing import Dict, List

import numpy as np

from . import build

MARK_ENTER, MARK_WAITED, MARK_END, MARK_PRODUCER_END = 0, 1, 2, 3
CAPACITY = 1 << 18          # records a library keeps (the rest of a run is dropped)


def enable() -> None:
    """From now on kernel libraries are loaded in their traced build.  Must come before any of them is loaded."""
    if any("." not in k for k in build.loaded_libraries()):
        raise RuntimeError("timeline.enable() must be called before the first kernel library is loaded")
    build.TIMELINE[0] = True


def records() -> np.ndarray:
    """All marks since the last call, of every loaded library, as a structured array (t in ns of the global
    timer, lib = index in build.LIBRARIES, mark, sm, grid = CTAs of the launch, cta); clears them.
    Synchronises the device."""
    dt = np.dtype([("t", np.int64), ("lib", np.int32), ("mark", np.int32), ("sm", np.int32), ("grid", np.int32),
                   ("cta", np.int32)])
    out = []
    buf = np.zeros((CAPACITY, 2), dtype=np.uint64)
    for key, lib in build.loaded_libraries().items():
        if "." in key or not hasattr(lib, "kp_trace_dump"):
            continue
        n = int(lib.kp_trace_dump(ctypes.c_void_p(buf.ctypes.data), ctypes.c_int(CAPACITY)))
        if n <= 0:
            continue
        w = buf[:n, 1]
        tag = (w & np.uint64(0xffffffff)).astype(np.int64)
        info = (w >> np.uint64(32)).astype(np.int64)
        r = np.zeros(n, dtype=dt)
        r["t"] = buf[:n, 0].astype(np.int64)
        r["lib"] = (tag >> 24) - 1
        r["mark"] = (tag >> 16) & 0xff
        r["sm"] = tag & 0xffff
        r["grid"] = info >> 16
        r["cta"] = info & 0xffff
        out.append(r)
    return np.concatenate(out) if out else np.zeros(0, dtype=dt)


def kernels(rec: np.ndarray) -> List[Dict]:
    """The launches in the records, in the order in which they entered: for each the library, the grid, when its
    first CTA entered, when its waits on the kernel before were over (first and last CTA) and, where the kernel
    notes it, when its last CTA was done.  Times in microseconds from the first record."""
    if len(rec) == 0:
        return []
    base = int(rec["t"].min())
    found = []
    for L in np.unique(rec["lib"]):
        r = rec[rec["lib"] == L]
        first = r[(r["mark"] == MARK_ENTER) & (r["cta"] == 0)]
        first = first[np.argsort(first["t"])]
        n_inst = len(first)
        per = [dict() for _ in range(n_inst)]
        grids = first["grid"]
        for mark in np.unique(r["mark"]):
            rm = r[r["mark"] == mark]
            for cta in np.unique(rm["cta"]):
                ts = np.sort(rm["t"][rm["cta"] == cta])
                # the launches of a library follow one another, so the i-th mark of a CTA number belongs to the
                # i-th launch that has that many CTAs
                owners = [i for i in range(n_inst) if grids[i] > cta]
                for i, t in zip(owners, ts):
                    per[i].setdefault(int(mark), []).append(int(t))
        for i in range(n_inst):
            m = per[i]
            us = lambda v: (v - base) / 1e3
            found.append({
                "lib": build.LIBRARIES[int(L)], "grid": int(grids[i]),
                "entered": us(min(m[MARK_ENTER])),
                "waited_first": us(min(m[MARK_WAITED])) if MARK_WAITED in m else None,
                "waited_last": us(max(m[MARK_WAITED])) if MARK_WAITED in m else None,
                "ended": us(max(m[MARK_END])) if MARK_END in m else None,
            })
    found.sort(key=lambda k: k["entered"])
    return found


def table(ks: List[Dict], names: List[str] = None) -> str:
    """A line a launch: when its wait was over, how long until the next launch's wait was over (its time on the
    step's critical path), how early it had entered (the overlap with the kernels before it)."""
    lines = [f"{'kernel':44s} {'CTAs':>6s} {'waited at':>10s} {'took':>8s} {'entered before':>15s}"]
    for i, k in enumerate(ks):
        w = k["waited_first"]
        nxt = next((x["waited_first"] for x in ks[i + 1:] if x["waited_first"] is not None), None)
        took = f"{nxt - w:8.2f}" if (w is not None and nxt is not None) else "        "
        early = f"{w - k['entered']:15.2f}" if w is not None else " " * 15
        name = names[i] if names and i < len(names) else k["lib"]
        lines.append(f"{name[:44]:44s} {k['grid']:6d} {(w if w is not None else k['entered']):10.2f} {took} {early}")
    return "\n".join(lines)
