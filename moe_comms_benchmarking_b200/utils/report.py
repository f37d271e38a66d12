"""Result rows, stdout lines and the CSV file, in the reference's formats (run.py:221-238),
plus row-by-row appending and ``--resume`` (the reference keeps all rows in memory and
loses them if the sweep dies, run.py:200,228-238)."""
from __future__ import annotations

import csv
import os
from dataclasses import dataclass

CSV_HEADER = "impl,global_B,num_sms,phase,per_rank_counts,latency_us,timing"
STDOUT_HEADER = "# impl,global_B,num_sms,phase,latency_us,timing"


@dataclass
class Row:
    impl: str
    global_b: int
    num_sms: int
    phase: str
    counts: list
    latency_us: float
    used_graph: bool

    @property
    def timing(self) -> str:
        return "graph" if self.used_graph else "eager"

    def csv_line(self) -> str:
        return (f"{self.impl},{self.global_b},{self.num_sms},{self.phase},\"{self.counts}\","
                f"{self.latency_us:.4f},{self.timing}")

    def stdout_csv_line(self) -> str:
        return f"{self.impl},{self.global_b},{self.num_sms},{self.phase},{self.latency_us:.3f},{self.timing}"

    def progress_line(self, num_layers: int) -> str:
        sms = f" sms={self.num_sms:3d}" if self.num_sms >= 0 else " sms= na"
        return (f"  {self.impl:7s} B={self.global_b:4d}{sms} counts={self.counts} "
                f"decode_step({num_layers}L)={self.latency_us:9.2f}us "
                f"(per-layer={self.latency_us / num_layers:6.2f}us)  [{self.timing}]")

    def key(self):
        return (self.impl, self.global_b, self.num_sms, self.phase)


class CsvSink:
    """Appends each row as soon as it is measured; with ``resume`` existing rows are loaded and
    their keys reported by ``done`` so the sweep can skip them."""

    def __init__(self, path: str | None, resume: bool = False):
        self.path = path
        self.rows: list[Row] = []
        self.done: set = set()
        if path is None:
            return
        if resume and os.path.exists(path):
            for r in load_rows(path):
                self.rows.append(r)
                self.done.add(r.key())
        else:
            with open(path, "w") as f:
                f.write(CSV_HEADER + "\n")

    def add(self, row: Row):
        self.rows.append(row)
        self.done.add(row.key())
        if self.path is not None:
            with open(self.path, "a") as f:
                f.write(row.csv_line() + "\n")
                f.flush()
                os.fsync(f.fileno())


def load_rows(path: str) -> list[Row]:
    out = []
    with open(path, newline="") as f:
        for r in csv.DictReader(f):
            counts = [int(c) for c in r.get("per_rank_counts", "").strip().strip("[]").split(",") if c.strip()]
            out.append(Row(r["impl"], int(r["global_B"]), int(r["num_sms"]), r["phase"], counts,
                           float(r["latency_us"]), r.get("timing", "graph") == "graph"))
    return out
