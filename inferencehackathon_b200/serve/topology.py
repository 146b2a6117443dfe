"""``GET /v1/topology``: live GPU stats (``nvidia-smi`` read-only query, static fallback) and the expert -> GPU
placement (optimised placement JSON when present, else ``expert % n_gpus``)
(reference: server/topology.py:8-79)."""
from __future__ import annotations

import json
import os
import subprocess
from pathlib import Path
from typing import List, Optional

OPTIMIZED_PLACEMENT_PATH = Path(os.environ.get("OPTIMIZED_PLACEMENT", "/alloc/data/optimized_placement.json"))
_QUERY = "index,name,memory.total,memory.used,utilization.gpu,temperature.gpu"


def _static_gpus(n: int = 8, name: str = "B200") -> List[dict]:
    return [{"id": i, "name": f"{name}-{i}", "mem_total_mb": 183359, "mem_used_mb": 0, "utilization_pct": 0,
             "temp_c": 0} for i in range(n)]


def _query_gpus() -> List[dict]:
    try:
        text = subprocess.check_output(["nvidia-smi", f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits"],
                                       timeout=5).decode()
        gpus = []
        for line in text.strip().splitlines():
            idx, name, total, used, util, temp = (x.strip() for x in line.split(","))
            gpus.append({"id": int(idx), "name": name, "mem_total_mb": int(total), "mem_used_mb": int(used),
                         "utilization_pct": int(util), "temp_c": int(temp)})
        return gpus or _static_gpus()
    except Exception:
        return _static_gpus()


def _load_placement(num_layers: int, experts_per_layer: int, num_gpus: int, path: Optional[Path] = None) -> dict:
    path = path or OPTIMIZED_PLACEMENT_PATH
    table = {}
    try:
        if path.exists():
            with open(path) as f:
                table = json.load(f)["placement"]
    except Exception:
        table = {}
    if not isinstance(table, dict):
        table = {}

    def gpu_of(L: int, e: int) -> int:
        # a file written for another model or GPU count, or damaged: entries that are missing, not integers or name a
        # GPU that is not there fall back to round robin one by one
        row = table.get(str(L))
        v = row.get(str(e)) if isinstance(row, dict) else None
        if isinstance(v, bool) or not isinstance(v, (int, float, str)):
            return e % num_gpus
        try:
            g = int(v)
        except (ValueError, OverflowError):
            return e % num_gpus
        return g if 0 <= g < num_gpus else e % num_gpus

    return {str(L): {str(e): gpu_of(L, e) for e in range(experts_per_layer)} for L in range(num_layers)}


def build_topology(num_layers: int = 94, experts_per_layer: int = 128, placement_fn=None) -> dict:
    """``placement_fn(expert_id) -> gpu`` (from a live engine) overrides file / round-robin placement."""
    gpus = _query_gpus()
    n = len(gpus)
    if placement_fn is not None:
        placement = {str(L): {str(e): int(placement_fn(e)) for e in range(experts_per_layer)} for L in range(num_layers)}
        source = "engine"
    else:
        placement = _load_placement(num_layers, experts_per_layer, n)
        source = "optimized" if OPTIMIZED_PLACEMENT_PATH.exists() else "round-robin"
    return {"gpus": gpus, "num_layers": num_layers, "experts_per_layer": experts_per_layer, "placement": placement,
            "placement_source": source}
