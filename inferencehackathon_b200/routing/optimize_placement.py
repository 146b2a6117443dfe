"""Command line: routing statistics JSON -> load-balanced expert placement JSON.

``python -m inferencehackathon_b200.routing.optimize_placement routing_stats.json optimized_placement.json
--n-gpus 8`` reads ``{"routing": {"activation_counts": [[...], ...]}}`` (layers x experts) and writes
``{placement, replicas, stats}``, the document the serving topology endpoint and the prefetch scheduler load.
Reference: engine/src/bin/optimize_placement.rs.
"""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np

from .native import optimize_placement


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("stats_json")
    ap.add_argument("out_json")
    ap.add_argument("--n-gpus", type=int, default=8)
    ap.add_argument("--hot-mult", type=float, default=2.0, help="replicate experts above this multiple of the layer mean")
    a = ap.parse_args(argv)
    with open(a.stats_json) as f:
        doc = json.load(f)
    counts = doc.get("routing", doc).get("activation_counts")
    if counts is None:
        print("no routing.activation_counts in", a.stats_json, file=sys.stderr)
        return 2
    _, out = optimize_placement(np.asarray(counts, dtype=np.uint32), a.n_gpus, a.hot_mult)
    with open(a.out_json, "w") as f:
        json.dump(out, f)
    s = out["stats"]
    print(f"layers {s['n_layers']}  experts {s['n_experts']}  gpus {s['n_gpus']}")
    print(f"mean imbalance (max/mean): round-robin {s['round_robin_mean_imbalance']:.3f} -> "
          f"optimised {s['optimized_mean_imbalance']:.3f} ({s['improvement_pct']:+.1f} %)")
    print(f"replicated expert-layers: {s['total_replicated_expert_layers']}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
