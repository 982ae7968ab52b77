"""Default-layout versus planned-layout cost per kernel class, from the JSON a Compile wrote.

The reference ships the same report as an offline tool (tools/analyzer.py:8-94 looks a
node's two records up in ``dp_table.evaluator``, :144-onwards sums them per kernel class
into ``{kernel: (default, planned)}``).  There the node list and the shapes come from the
ONNX file; here the dump itself carries them (``arena.stats.sequence`` lists every node of
the executed sequence with its inputs and output, ``infos`` the logical shape of every
tensor), so the fused kernels, which have no ONNX node of their own, are covered too.

    python -m fluidml_b200.analyzer --json plan.json --output report.json

A cost is what the layout search used: nanoseconds of the GPU cost model (launch floor +
coalescing-aware HBM time, or tensor-core time for contractions), not a measurement.
"""
from __future__ import annotations

import argparse
import json
from typing import Dict, List, Optional, Tuple


class Analyzer:
    """Looks up the cost records of the nodes of one compiled sequence."""

    def __init__(self, dp_table: Dict[str, List[dict]], plan: Dict[str, List[int]], infos: Dict[str, List[int]]):
        self.dp_table = dp_table
        self.plan = plan
        self.infos = infos

    @staticmethod
    def _operand_names(count: int) -> List[str]:
        # the record's field prefixes: input/output, lhs/rhs/output, else input0.. + output
        if count == 2:
            return ["input", "output"]
        if count == 3:
            return ["lhs", "rhs", "output"]
        return ["input%d" % i for i in range(count - 1)] + ["output"]

    def _find(self, kernel: str, tensors: List[str], layouts: List[List[int]]) -> Optional[int]:
        names = self._operand_names(len(tensors))
        for rec in self.dp_table.get(kernel, ()):
            if all(rec.get(n + "_shape") == self.infos[t] and rec.get(n + "_layout") == l
                   for n, t, l in zip(names, tensors, layouts)):
                return int(rec["time_cost"])
        return None

    def find(self, kernel: str, inputs: List[str], output: str) -> Tuple[Optional[int], Optional[int]]:
        """(cost with every operand row-major, cost with the planned layouts); None where the
        search never evaluated that combination (it only visits layouts a neighbour can produce)."""
        tensors = list(inputs) + [output]
        default = [list(range(len(self.infos[t]))) for t in tensors]
        planned = [self.plan.get(t, d) for t, d in zip(tensors, default)]
        return self._find(kernel, tensors, default), self._find(kernel, tensors, planned)


def analyze(dump: dict) -> dict:
    """``{"kernels": {name: [default, planned, nodes]}, "total": [default, planned], "unmatched": [...]}``."""
    analyzer = Analyzer(dump.get("dp_table", {}).get("evaluator", {}), dump.get("plan", {}), dump["infos"])
    kernels: Dict[str, List[int]] = {}
    unmatched: List[str] = []
    for node in dump["arena"]["stats"]["sequence"]:
        kernel = node["kind"] + "Kernel"
        default, planned = analyzer.find(kernel, node["inputs"], node["output"])
        if default is None or planned is None:
            unmatched.append(node["name"])
            continue
        row = kernels.setdefault(kernel, [0, 0, 0])
        row[0] += default
        row[1] += planned
        row[2] += 1
    total = [sum(r[0] for r in kernels.values()), sum(r[1] for r in kernels.values())]
    return {"kernels": kernels, "total": total, "unmatched": unmatched}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="Analyze the compiler execution intermediate results.")
    ap.add_argument("--json", required=True, help="The intermediate json file (third argument of Compile).")
    ap.add_argument("--output", help="The output json file; the table is printed either way.")
    ap.add_argument("--model", help="Accepted for command-line compatibility; the dump already names every node.")
    args = ap.parse_args(argv)
    with open(args.json) as f:
        report = analyze(json.load(f))
    print("%-56s %6s %12s %12s" % ("kernel", "nodes", "default ns", "planned ns"))
    for name in sorted(report["kernels"]):
        d, p, n = report["kernels"][name]
        print("%-56s %6d %12d %12d" % (name, n, d, p))
    print("%-56s %6s %12d %12d" % ("total", "", report["total"][0], report["total"][1]))
    if report["unmatched"]:
        print("%d nodes without both records (layout combination never evaluated)" % len(report["unmatched"]))
    if args.output:
        with open(args.output, "w") as f:
            json.dump(report, f, indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
