"""CUDA-event phase timing resolved lazily (mirrors dfsattn/utils/timing.py:24-218).

Events are recorded around a region without synchronising; durations are
computed only when ``dump_csv`` / ``summary`` is called.  Phases recorded by the
native path: ``topk_mask``, ``topk_routing``, ``attention_execution``; the written
table has the reference's columns and categories.
"""
import csv
import os
import time
from typing import Dict, List, Optional

import torch


class AttentionTimingRecorder:
    def __init__(self, enabled: bool = False) -> None:
        self.enabled = enabled
        self._records: List[tuple] = []
        self._metric_records: Dict[str, List[float]] = {}

    def reset(self, enabled: bool) -> None:
        self.enabled = enabled
        self._records.clear()
        self._metric_records.clear()

    def record_metrics(self, metrics: Dict[str, float]) -> None:
        if not self.enabled:
            return
        for name, value in metrics.items():
            self._metric_records.setdefault(name, []).append(float(value))

    def start(self, device):
        if not self.enabled:
            return None
        if torch.device(device).type == "cuda":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record()
            return ev
        return time.perf_counter()

    def stop(self, start, phase: str, step_idx: int, layer_idx: int, device) -> None:
        if not self.enabled or start is None:
            return
        if torch.device(device).type == "cuda":
            end = torch.cuda.Event(enable_timing=True)
            end.record()
        else:
            end = time.perf_counter()
        self._records.append((phase, int(step_idx), int(layer_idx), start, end))

    def _resolve(self):
        rows = []
        if any(isinstance(r[3], torch.cuda.Event) for r in self._records):
            torch.cuda.synchronize()
        for phase, step, layer, start, end in self._records:
            ms = start.elapsed_time(end) if isinstance(start, torch.cuda.Event) else (end - start) * 1e3
            rows.append((phase, step, layer, ms))
        return rows

    def summary(self) -> Dict[str, Dict[str, float]]:
        out: Dict[str, Dict[str, float]] = {}
        for phase, _, _, ms in self._resolve():
            agg = out.setdefault(phase, {"calls": 0, "total_ms": 0.0})
            agg["calls"] += 1
            agg["total_ms"] += ms
        for agg in out.values():
            agg["mean_ms"] = agg["total_ms"] / max(agg["calls"], 1)
        return out

    # raw phase name -> category of the written table (dfsattn/utils/timing.py:148-151): the selector's
    # ``topk_mask`` events are reported as ``top_k_selection``; ``topk_routing`` encloses ``topk_mask`` and
    # is not written, as in the reference
    CATEGORIES = {"topk_mask": "top_k_selection", "attention_execution": "attention_execution"}

    def dump_csv(self, output_path: str, extra_totals: Optional[Dict[str, float]] = None):
        """One aggregate row per category, columns ``phase,total_ms,calls,mean_ms`` as the reference
        writes them (dfsattn/utils/timing.py:140-200); ``extra_totals`` become rows of one call each.
        Returns the same table as a dict (the raw per-phase table stays available from ``summary``)."""
        totals = {name: 0.0 for name in self.CATEGORIES.values()}
        calls = {name: 0 for name in totals}
        for phase, _, _, ms in self._resolve():
            cat = self.CATEGORIES.get(phase)
            if cat is not None:
                totals[cat] += ms
                calls[cat] += 1
        for name, value in (extra_totals or {}).items():
            totals[name] = float(value)
            calls[name] = 1
        os.makedirs(os.path.dirname(output_path) or ".", exist_ok=True)
        with open(output_path, "w", newline="") as f:
            w = csv.DictWriter(f, fieldnames=["phase", "total_ms", "calls", "mean_ms"])
            w.writeheader()
            for name, total in totals.items():
                w.writerow({"phase": name, "total_ms": total, "calls": calls[name],
                            "mean_ms": total / calls[name] if calls[name] else 0.0})
        return {name: {"calls": float(calls[name]), "total_ms": total,
                       "mean_ms": total / calls[name] if calls[name] else 0.0}
                for name, total in totals.items()}
