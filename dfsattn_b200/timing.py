"""CUDA-event phase timing resolved lazily (mirrors dfsattn/utils/timing.py:24-218).

Events are recorded around a region without synchronising; durations are
computed only when ``dump_csv`` / ``summary`` is called.  Phases used by the
native path: ``topk_mask``, ``topk_routing``, ``attention_execution``.
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

    def dump_csv(self, output_path: str, extra_totals: Optional[Dict[str, float]] = None):
        summary = self.summary()
        os.makedirs(os.path.dirname(output_path) or ".", exist_ok=True)
        with open(output_path, "w", newline="") as f:
            w = csv.writer(f)
            w.writerow(["phase", "calls", "total_ms", "mean_ms"])
            for phase, agg in sorted(summary.items()):
                w.writerow([phase, agg["calls"], f"{agg['total_ms']:.6f}", f"{agg['mean_ms']:.6f}"])
            for name, value in (extra_totals or {}).items():
                w.writerow([name, 1, f"{float(value):.6f}", f"{float(value):.6f}"])
            for name, values in sorted(self._metric_records.items()):
                w.writerow([name, len(values), f"{sum(values):.6f}", f"{sum(values) / len(values):.6f}"])
        return summary
