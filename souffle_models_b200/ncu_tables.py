"""Totals from Nsight Compute CSV exports: summed kernel time, kernel count and DRAM bytes read.

These are the three per-model figures the reference's scripts put into its result tables
(python/extract_ncu_cuda_kernel_latency.py:57-78 sums `gpu__time_duration.sum` to milliseconds,
python/extract_ncu_cuda_mem_read.py:57-78 sums `dram__bytes_read.sum` to MB, and
python/models/run_ncu_mem_souffle.sh:78-80 writes the kernel counts), recomputed here for this library's
launches.  Both CSV shapes ncu produces are read:

* wide  (`ncu -i report.ncu-rep --page raw --csv`): one row per launch, one column per metric, units in row 2;
* long  (`ncu --csv --metrics ...` to a log file): one row per (launch, metric) with "Metric Name" /
  "Metric Unit" / "Metric Value" columns.

Usage:  python -m souffle_models_b200.ncu_tables export.csv [kernel-name-regex]
"""
import csv
import re
import sys
from typing import Dict, List, Optional, Tuple

_TIME_TO_MS = {"msecond": 1.0, "ms": 1.0, "usecond": 1e-3, "us": 1e-3, "nsecond": 1e-6, "ns": 1e-6, "second": 1e3, "s": 1e3}
_BYTES_TO_MB = {"byte": 1.0 / (1024 * 1024), "Kbyte": 1.0 / 1024, "Mbyte": 1.0, "Gbyte": 1024.0, "Tbyte": 1024.0 * 1024}


def _number(text: str) -> float:
    """ncu prints thousands separators and, for metrics it could not collect, N/A or nan: those count as 0
    (as in filter_invalid_ncu_records, extract_ncu_cuda_kernel_latency.py:47-56)."""
    t = text.strip().replace(",", "")
    if not t or t == "N/A" or "nan" in t.lower():
        return 0.0
    return float(t)


def read_launches(path: str) -> List[Dict[str, Tuple[float, str]]]:
    """One dict per kernel launch: {"Kernel Name": (0.0, name), metric: (value, unit), ...}."""
    with open(path, newline="") as f:
        rows = [r for r in csv.reader(f) if r]
    start = next((i for i, r in enumerate(rows) if r[0] == "ID"), None)
    if start is None:
        raise ValueError(f"{path}: no ncu CSV header (a row starting with \"ID\") found")
    header = rows[start]
    launches: List[Dict[str, Tuple[float, str]]] = []
    if "Metric Name" in header:                      # long format
        k_id, k_name = header.index("ID"), header.index("Kernel Name")
        k_m, k_u, k_v = header.index("Metric Name"), header.index("Metric Unit"), header.index("Metric Value")
        by_id: Dict[str, Dict[str, Tuple[float, str]]] = {}
        for r in rows[start + 1:]:
            if len(r) <= k_v:
                continue
            rec = by_id.setdefault(r[k_id], {"Kernel Name": (0.0, r[k_name])})
            rec[r[k_m]] = (_number(r[k_v]), r[k_u])
        launches = list(by_id.values())
    else:                                            # wide format: units in the row after the header
        units = rows[start + 1]
        k_name = header.index("Kernel Name")
        for r in rows[start + 2:]:
            rec = {"Kernel Name": (0.0, r[k_name])}
            for i, h in enumerate(header):
                if i != k_name and i < len(r) and ("__" in h or "." in h):
                    try:
                        rec[h] = (_number(r[i]), units[i] if i < len(units) else "")
                    except ValueError:
                        pass
            launches.append(rec)
    return launches


def totals(path: str, kernel_regex: Optional[str] = None) -> Dict[str, float]:
    """{"kernels": launches counted, "latency_ms": summed gpu__time_duration.sum, "dram_read_mb": summed
    dram__bytes_read.sum} over the launches whose kernel name matches `kernel_regex` (all if None)."""
    pat = re.compile(kernel_regex) if kernel_regex else None
    n, ms, mb = 0, 0.0, 0.0
    for rec in read_launches(path):
        if pat and not pat.search(rec["Kernel Name"][1]):
            continue
        n += 1
        if "gpu__time_duration.sum" in rec:
            v, u = rec["gpu__time_duration.sum"]
            ms += v * _TIME_TO_MS.get(u.strip(), 1e-6)
        if "dram__bytes_read.sum" in rec:
            v, u = rec["dram__bytes_read.sum"]
            mb += v * _BYTES_TO_MB.get(u.strip(), 1.0 / (1024 * 1024))
    return {"kernels": n, "latency_ms": ms, "dram_read_mb": mb}


def main(argv: List[str]) -> int:
    if len(argv) < 2:
        print(__doc__)
        return 2
    t = totals(argv[1], argv[2] if len(argv) > 2 else None)
    print(f"kernels={t['kernels']} latency_ms={t['latency_ms']:.6f} dram_read_mb={t['dram_read_mb']:.3f}")
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv))
